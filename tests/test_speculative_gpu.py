"""Speculative decoding through the CUDA kernels: the verification rows (k + 1 per sequence) of the target, the draft
module's own KV cache and its chained steps on rows built on the device.  On the CPU (fp32) the emitted tokens equal plain
greedy decoding exactly (tests/test_speculative.py); in bf16 the verification step and the plain decode step reach the
same logits through differently shaped kernels, so two nearly equal top logits may fall the other way.  What must hold
here: wherever the two runs part, the speculative token is one of the plain run's top candidates within a small
log-probability gap of its best one."""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu

from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.speculative import SpeculativeEngine

from test_model_gpu import ds_args, small_args


def _opts(**kw):
    o = dict(model="preset:x", devices="cuda:0", block_size=16, num_kv_blocks=512, max_tokens_per_batch=1024, max_seqs_per_batch=16)
    o.update(kw)
    return Options(**o)


def _prompts(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _parts_only_at_near_ties(plain, spec, gap=0.2):
    """Sequences equal, or at the first difference the speculative token is among the plain run's top candidates and within
    `gap` of its best log-probability.  Returns how many sequences are equal over their whole length."""
    same = 0
    for p, s in zip(plain, spec):
        pt, st = p.outputs[0].token_ids, s.outputs[0].token_ids
        assert len(pt) == len(st)
        for i, (a, b) in enumerate(zip(pt, st)):
            if a != b:
                lp = p.outputs[0].logprobs[i]
                cand = {t.token_id: t.logprob for t in lp.top_logprobs}
                assert b in cand and lp.logprob - cand[b] < gap, (i, a, b, lp.logprob, cand)
                break
        else:
            same += 1
    return same


def _run_pair(args, model, draft, algorithm, k, prompts, n_new=12, **opt):
    from xllm_wxh_b200.ops import cuda_ops
    plain_sp = SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True, logprobs=True, top_logprobs=4)
    plain = LLM(model="preset:x", devices="cuda:0", engine=LLMEngine(_opts(**opt), model_args=args, model=model)).generate(prompts, plain_sp)
    eng = SpeculativeEngine(_opts(num_speculative_tokens=k, speculative_algorithm=algorithm, **opt), model_args=args, model=model,
                            draft_model=draft)
    spec = LLM(model="preset:x", devices="cuda:0", engine=eng).generate(
        prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    assert cuda_ops.read_status() == 0
    assert eng.stat_draft_tokens > 0 and eng.stat_draft_tokens % k == 0
    return plain, spec, eng


@pytest.mark.parametrize("k", [1, 2])
@pytest.mark.parametrize("sparse", [False, True])
def test_mtp_speculative_gpu(k, sparse):
    """DeepSeek-style target with its MTP module (k = 1: one draft per step; k = 2: the module chained on device-built
    rows); `sparse`: the DeepSeek-V3.2 form, target and draft each with a lightning indexer."""
    from xllm_wxh_b200.models.deepseek_impl import DeepseekForCausalLM
    extra = dict(model_type="deepseek_v32", index_topk=24, index_n_heads=16, index_head_dim=128) if sparse else {}
    args = ds_args(n_layers=2, num_nextn_predict_layers=1, num_experts_per_tok=8, n_group=1, topk_group=1, **extra)
    model = DeepseekForCausalLM(args, device="cuda:0", dtype=torch.bfloat16).init_random(seed=0, std=0.05)
    prompts = _prompts(args.vocab_size, (20, 33, 7, 70))
    plain, spec, eng = _run_pair(args, model, None, "MTP", k, prompts)
    assert _parts_only_at_near_ties(plain, spec) >= 1
    assert all(len(d) == k for d in eng.drafts.values())


@pytest.mark.parametrize("k,graphs", [(2, False), (3, True)])
def test_eagle3_speculative_gpu(k, graphs):
    """Qwen target with an EAGLE-3 draft layer: the draft's attention runs on rows built on the device for its chained
    steps (no step header on the device for those)."""
    from xllm_wxh_b200.models.eagle3 import Eagle3Draft
    from xllm_wxh_b200.models.qwen import QwenForCausalLM
    args = small_args(n_layers=6)
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=0, std=0.05).finalize_weights()
    draft = Eagle3Draft(args, device="cuda:0", target=model).init_random(seed=3, std=0.05)
    prompts = _prompts(args.vocab_size, (20, 33, 7, 150))
    model.capture_layers = None
    try:
        plain, spec, eng = _run_pair(args, model, draft, "Eagle3", k, prompts, enable_graph=graphs)
        assert _parts_only_at_near_ties(plain, spec) >= 1
    finally:
        model.capture_layers = None
