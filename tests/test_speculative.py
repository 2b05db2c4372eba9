"""Speculative decoding on CPU: with greedy sampling the emitted tokens must equal plain decoding, whatever the drafts
propose (accepted drafts are by construction the tokens the target would have produced)."""
import os

import pytest
import torch

from test_deepseek_cpu import tiny_ds
from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.deepseek_impl import DeepseekForCausalLM
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.speculative import SpeculativeEngine, rejection_sample


def _opts(**kw):
    o = dict(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=256, dtype="float32")
    o.update(kw)
    return Options(**o)


def _prompts(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def test_rejection_sample_rules():
    target = torch.tensor([[5, 6, 7], [5, 9, 7], [1, 2, 3]], dtype=torch.int32)
    draft = torch.tensor([[5, 6], [5, 6], [9, 2]], dtype=torch.int32)
    out, acc = rejection_sample(target, draft, -1.0, 0)
    assert out.tolist() == [[5, 6, 7], [5, 9, -1], [1, -1, -1]] and acc.tolist() == [2, 1, 0]
    out, acc = rejection_sample(target.repeat(200, 1), draft.repeat(200, 1), 0.7, 3)
    assert 0.6 < (acc.float().mean() / 2).item() < 0.95      # forced acceptance rate, first failure stops the chain


def test_mtp_speculative_equals_plain_greedy():
    args = tiny_ds(n_layers=2, num_nextn_predict_layers=1)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    prompts = _prompts(args.vocab_size, (20, 33, 7))
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    plain = LLM(model="preset:x", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)
    eng = SpeculativeEngine(_opts(num_speculative_tokens=1, speculative_algorithm="MTP"), model_args=args, model=model)
    spec = LLM(model="preset:x", devices="cpu", engine=eng).generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert eng.stat_draft_tokens > 0


def test_mtp_fixed_acceptance_rate_override(monkeypatch):
    monkeypatch.setenv("XLLM_FIX_SPECULATIVE_ACCEPTANCE_RATE", "0.7")
    args = tiny_ds(n_layers=2)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    eng = SpeculativeEngine(_opts(num_speculative_tokens=1, speculative_algorithm="MTP"), model_args=args, model=model)
    outs = LLM(model="preset:x", devices="cpu", engine=eng).generate(_prompts(args.vocab_size, (16,) * 8),
                                                                     SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 40 for o in outs)
    assert 0.55 < eng.acceptance_rate() < 0.85
    assert eng.step_count < 8 + 40          # fewer steps than tokens per sequence: drafts were accepted


def test_suffix_speculative_equals_plain_greedy_and_accepts_repeats():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    prompts = [p * 3 for p in _prompts(args.vocab_size, (12, 9))]            # repetitive prompts
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    plain = LLM(model="preset:x", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)
    eng = SpeculativeEngine(_opts(num_speculative_tokens=3, speculative_algorithm="Suffix"), model_args=args, model=model)
    spec = LLM(model="preset:x", devices="cpu", engine=eng).generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
