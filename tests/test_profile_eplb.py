"""Start-up profiler / step-time predictors, and the EPLB runtime (manager, executor, slot tables)."""
import numpy as np
import pytest
import torch

from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import preset
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine
from xllm_wxh_b200.runtime.profile_manager import ProfileManager, TimePredictor


def test_time_predictor_budget():
    p = TimePredictor(prefill_coef=(1.0, 0.01, 1e-6), decode_coef=(1.0, 0.002, 1e-5))
    assert p.prefill_ms(1000) > p.prefill_ms(100) > 0
    assert p.decode_ms(64, 64 * 1000) > p.decode_ms(8, 8 * 1000)
    # fixed cost is paid once in a mixed step
    assert p.mixed_ms(512, 32, 32000) < p.prefill_ms(512) + p.decode_ms(32, 32000)
    b = p.token_budget_for_tpot(10.0, 32, 32000, 8192)
    assert b % 16 == 0 and p.mixed_ms(b, 32, 32000) <= 10.0 < p.mixed_ms(b + 32, 32, 32000)
    assert p.token_budget_for_tpot(0.001, 32, 32000, 8192) == 16          # never below one chunk


def test_profile_manager_fits_and_installs_budget():
    args = preset("tiny-qwen2")
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0)
    opts = Options(model="preset:tiny-qwen2", devices="cpu", block_size=16, num_kv_blocks=512, dtype="float32",
                   max_tokens_per_batch=512, max_seqs_per_batch=32, enable_profile_step_time=True,
                   enable_profile_token_budget=True, max_global_tpot_ms=1e-3, profile_max_prompt_length=256)
    eng = LLMEngine(opts, model_args=args, model=model)
    pm = ProfileManager(eng, opts.profile_max_prompt_length)
    pre = pm.profile_prefill(repeats=1)
    dec = pm.profile_decode(batches=(1, 4, 16), context=32, steps=2)
    assert [n for n, _ in pre] == [32, 64, 128, 256] and all(t > 0 for _, t in pre)
    assert [b for b, _, _ in dec] == [1, 4, 16]
    pred = pm.fit()
    assert pred.prefill_ms(256) >= pred.prefill_ms(32) and pred.decode_ms(16, 16 * 40) > 0
    assert not eng.has_unfinished()
    # an unreachable TPOT target drives the budget to its floor (one chunk + the decode rows)
    pm2 = ProfileManager(eng, 128)
    pm2.samples = pm.samples
    pm2.profile_prefill = lambda *a, **k: None
    pm2.profile_decode = lambda *a, **k: None
    pm2.run()
    assert eng.scheduler.token_budget == 16 + 32
    # the C++ scheduler's latency-aware policies predict with the same coefficients
    m = eng.scheduler.step_time_model()
    assert (m.a0, m.a1, m.a2) == pytest.approx(pm2.predictor.prefill_coef) and (m.b0, m.b1, m.b2) == pytest.approx(pm2.predictor.decode_coef)
    assert m.prefill_ms(256, 0) + m.a0 == pytest.approx(pm2.predictor.prefill_ms(256), rel=1e-6, abs=1e-9)
    eng.scheduler.set_token_budget(10 ** 9)
    assert eng.scheduler.token_budget == 512                               # never above the configured maximum


# ----------------------------------------------------------------------------- EPLB
from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.models.args import ModelArgs
from xllm_wxh_b200.runtime.eplb import EplbManager, build_route_table, initial_placement


def test_initial_placement_and_route_table():
    p = initial_placement(8, 2, 5)               # 4 experts per device + 1 redundant slot each
    assert p.tolist() == [0, 1, 2, 3, 3, 4, 5, 6, 7, 7]
    table, copies = build_route_table(p, 8)
    assert copies.tolist() == [1, 1, 1, 2, 1, 1, 1, 2]
    assert sorted(table[3].tolist()) == [3, 4] and sorted(table[7].tolist()) == [8, 9]
    assert table[0].tolist() == [0, 0]           # padded by repetition
    with pytest.raises(ValueError):
        build_route_table([0, 0, 1], 3)          # expert 2 has no slot


def test_manager_replans_hot_experts_and_respects_threshold():
    m = EplbManager(n_layers=2, n_experts=8, n_devices=2, slots=5, interval=4, threshold=0.9)
    hot = np.ones((2, 8))
    hot[0, 1] = 50.0                              # layer 0: expert 1 is hot; layer 1 stays uniform
    hot[1, :] = 0.0
    assert [m.tick() for _ in range(4)] == [False, False, False, True]
    m.update_expert_load(hot)
    assert m.plan() == 1
    layer, placement = m.next_layer()
    assert layer == 0 and sorted(placement.tolist()).count(1) >= 2          # the hot expert got a replica
    table, copies = build_route_table(placement, 8)
    assert copies[1] >= 2 and copies.sum() == 10
    m.committed(layer, placement)
    # the same load pattern again: cosine similarity 1 -> no new plan
    m.update_expert_load(hot * 3)
    assert m.plan() == 0 and m.next_layer() is None
    # a different pattern -> re-plan
    other = np.ones((2, 8))
    other[0, 6] = 80.0
    m.update_expert_load(other)
    assert m.plan() >= 1


def _moe_args():
    return ModelArgs(model_type="qwen3_moe", dtype="float32", vocab_size=512, hidden_size=64, n_layers=2, n_heads=4, n_kv_heads=2,
                     head_dim=16, intermediate_size=128, qk_norm=True, n_routed_experts=8, num_experts_per_tok=2,
                     moe_intermediate_size=32, norm_topk_prob=True, max_position_embeddings=512)


def test_generation_is_unchanged_while_experts_move():
    """With replicas holding the same weights, outputs must not depend on the placement: generate with frequent
    re-planning (every 2 steps, every plan accepted) and compare with EPLB off."""
    args = _moe_args()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (9, 17, 5, 30)]
    sp = SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True)
    outs = {}
    for name, kw in {"off": {}, "on": dict(enable_eplb=True, redundant_experts_num=2, eplb_update_interval=2,
                                            eplb_update_threshold=1.1)}.items():
        model = QwenForCausalLM(args, device="cpu").init_random(seed=1, std=0.2)
        opts = Options(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32", **kw)
        eng = LLMEngine(opts, model_args=args, model=model)
        llm = LLM(model="preset:x", devices="cpu", engine=eng)
        outs[name] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        if name == "on":
            ex = model.eplb
            assert ex is not None and ex.S == 10 and model.layers[0].mlp.w13.shape[0] == 10
            assert ex.num_activations > 0, "no layer was ever re-planned"
            assert eng.eplb.manager.num_replans >= ex.num_activations
            # some expert really has more than one live slot after balancing
            assert any(int(c.max()) > 1 for c in ex.copies)
    assert outs["on"] == outs["off"]
