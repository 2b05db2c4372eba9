"""Engine features through the CUDA kernels that the model tests do not reach: prefix-cache reuse, beam search, the
embedding task, penalties with seeded sampling, and the MoE model end to end under CUDA graphs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.models.qwen import QwenForCausalLM

from test_model_gpu import _RefOps, _engine, small_args
from test_speculative_gpu import _parts_only_at_near_ties


def _prompts(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _status_ok():
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0


def test_prefix_cache_reuse_gpu():
    """The second pass over the same prompts computes only what the cached blocks do not cover; its tokens part from the
    first pass at most where two top logits nearly tie (the suffix runs through kernels of another shape)."""
    args = small_args()
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=2, std=0.05)
    llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model, enable_prefix_cache=True))
    prompts = _prompts(args.vocab_size, (200, 75, 130), seed=3)
    first = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True, logprobs=True, top_logprobs=4))
    again = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    assert _parts_only_at_near_ties(first, again) >= 1
    assert again[0].usage.num_cached_tokens >= 192 and again[1].usage.num_cached_tokens >= 64
    assert llm.engine.scheduler.block_manager(0).match_hits > 0
    _status_ok()


def test_beam_search_gpu():
    """Width-3 beams: sorted by cumulative log-probability, distinct, each score the sum of its tokens' log-probabilities
    under the model (re-scored by a plain prefill of prompt + beam with the PyTorch statement of the ops)."""
    from xllm_wxh_b200.api.llm import BeamSearchParams
    args = small_args()
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=6, std=0.08)
    llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model))
    prompt = _prompts(args.vocab_size, (25,), seed=1)[0]
    out = llm.beam_search([prompt], BeamSearchParams(beam_width=3, max_tokens=5))[0]
    beams = [o.token_ids for o in out.outputs]
    scores = [o.cumulative_logprob for o in out.outputs]
    assert len(beams) == 3 and all(len(b) == 5 for b in beams) and len({tuple(b) for b in beams}) == 3
    assert scores == sorted(scores, reverse=True)
    # re-score every beam: log-probability of each of its tokens given prompt + the tokens before it
    from test_model_gpu import _one_step_logits
    for toks, score in zip(beams, scores):
        total = 0.0
        for i, t in enumerate(toks):
            with _RefOps():
                lg = _one_step_logits(_engine(args, model), [prompt + toks[:i]])[0]
            total += float(torch.log_softmax(lg.float(), -1)[t])
        assert abs(total - score) < 0.15, (toks, total, score)
    _status_ok()


def _one_step_embeddings(engine, prompts):
    """Last-token hidden states of one prefill step, L2-normalised (the forward of `_one_step_logits`, pooled)."""
    from xllm_wxh_b200.framework.step_input import StepInput
    for p in prompts:
        engine.add_request(p)
    b = engine.scheduler.schedule()[0]
    w = engine.worker
    T, B, MB, S, P, padded = w.choose_caps(b.num_tokens, b.num_seqs, b.max_blocks, b.num_sample_rows, False)
    L = w.layout_for(T, B, MB, S, P)
    host = w.host_staging(L.total_words)
    assert b.build(L, host.data_ptr(), host.numel(), engine.block_size) == 0
    hdr = host[L.header:L.header + 32].numpy().copy()
    w._dev[:L.total_words].copy_(host[:L.total_words])
    inp = StepInput(w._dev, L, hdr)
    with torch.inference_mode():
        return w.model.pooled_embedding(w.model.forward(inp, w.kv_caches), inp.sample_idx).float().cpu()


def test_embedding_task_gpu():
    """`LLM.embed`: the L2-normalised final hidden state of the last prompt token, against the same model run through
    the PyTorch statement of the ops."""
    args = small_args()
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=7, std=0.05)
    prompts = _prompts(args.vocab_size, (3, 37, 150), seed=4)
    got = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model)).embed(prompts)
    with _RefOps():
        want = _one_step_embeddings(_engine(args, model), prompts)
    for a, eb in zip(got, want):
        ea = torch.tensor(a.outputs[0].embeddings)
        assert ea.shape == (args.hidden_size,) and abs(float(ea.norm()) - 1.0) < 1e-2
        assert float(torch.dot(ea, eb)) > 0.995
    _status_ok()


def test_penalties_and_seeded_sampling_gpu():
    """A seeded sampling request is repeatable and differs between seeds; greedy decoding under a repetition penalty takes
    the arg-max of the penalised logits (prompt tokens: positive logits halved, negative ones doubled)."""
    from test_model_gpu import _one_step_logits
    args = small_args(vocab_size=2048)
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=8, std=0.05)
    llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model))
    prompts = _prompts(args.vocab_size, (30, 12, 50, 21), seed=5)
    sp = lambda seed: SamplingParams(temperature=0.9, top_k=50, top_p=0.95, max_tokens=16, ignore_eos=True, seed=seed)
    a = [o.outputs[0].token_ids for o in llm.generate(prompts, sp(11))]
    b = [o.outputs[0].token_ids for o in llm.generate(prompts, sp(11))]
    c = [o.outputs[0].token_ids for o in llm.generate(prompts, sp(12))]
    assert a == b and a != c
    pen = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, repetition_penalty=2.0))
    checked = 0
    for p, o in zip(prompts, pen):
        lg = _one_step_logits(_engine(args, model), [p])[0].float().clone()
        ids = torch.tensor(sorted(set(p)))
        v = lg[ids]
        lg[ids] = torch.where(v > 0, v / 2.0, v * 2.0)
        top = lg.topk(2)
        if float(top.values[0] - top.values[1]) > 0.03:
            assert o.outputs[0].token_ids[0] == int(top.indices[0])
            checked += 1
    assert checked >= 1
    _status_ok()


def test_moe_model_generates_under_graphs_gpu():
    """Qwen3-MoE end to end: eager against CUDA-graph replay of the same requests."""
    args = small_args(model_type="qwen3_moe", n_routed_experts=16, num_experts_per_tok=4, moe_intermediate_size=256)
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=9, std=0.05)
    prompts = _prompts(args.vocab_size, (7, 40, 19, 64, 3), seed=6)
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True, logprobs=True, top_logprobs=4)
    outs = {}
    for name, kw in {"eager": dict(enable_graph=False), "graph": dict(enable_graph=True)}.items():
        llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model, **kw))
        outs[name] = llm.generate(prompts, sp)
        if name == "graph":
            assert llm.engine.worker._graphs is not None and llm.engine.worker._graphs.num_replays > 0
    assert _parts_only_at_near_ties(outs["eager"], outs["graph"]) >= 3
    _status_ok()
