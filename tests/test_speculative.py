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


@pytest.mark.parametrize("k", [2, 3])
def test_multi_step_mtp_equals_plain_greedy(k):
    """k > 1: the draft module runs k times in a chain (its own hidden state and its own proposal feed the next step, its
    KV runs ahead of the step's rows).  Whatever it proposes, the emitted tokens are those of plain greedy decoding; and the
    chained proposals are the module's own continuation: a draft model that is the target itself would be accepted whole,
    which the acceptance counters of a second run with a perfect drafter confirm."""
    args = tiny_ds(n_layers=2, num_nextn_predict_layers=1)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    prompts = _prompts(args.vocab_size, (20, 33, 7, 48))
    sp = SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True)
    plain = LLM(model="preset:x", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)
    eng = SpeculativeEngine(_opts(num_speculative_tokens=k, speculative_algorithm="MTP", max_tokens_per_batch=64,
                                  max_tokens_per_chunk_for_prefill=24), model_args=args, model=model)
    spec = LLM(model="preset:x", devices="cpu", engine=eng).generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert eng.stat_draft_tokens > 0 and eng.stat_draft_tokens % k == 0
    # every sequence keeps k drafts between steps
    assert all(len(d) == k for d in eng.drafts.values())


def test_multi_step_mtp_with_forced_acceptance_takes_fewer_steps(monkeypatch):
    monkeypatch.setenv("XLLM_FIX_SPECULATIVE_ACCEPTANCE_RATE", "0.8")
    args = tiny_ds(n_layers=2)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    steps = {}
    for k in (1, 3):
        eng = SpeculativeEngine(_opts(num_speculative_tokens=k, speculative_algorithm="MTP"), model_args=args, model=model)
        outs = LLM(model="preset:x", devices="cpu", engine=eng).generate(_prompts(args.vocab_size, (16,) * 4),
                                                                         SamplingParams(temperature=0.0, max_tokens=36, ignore_eos=True))
        assert all(len(o.outputs[0].token_ids) == 36 for o in outs)
        steps[k] = eng.step_count
    assert steps[3] < steps[1]


def test_mtp_draft_kv_travels_with_the_host_tier():
    """A prefix that left the device cache comes back from the host tier under other block ids: the draft module's KV of
    those blocks comes back with it (the tier's records hold target and draft parts), and tokens stay those of plain decoding."""
    args = tiny_ds(n_layers=2, num_nextn_predict_layers=1)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    prompt = _prompts(args.vocab_size, (70,))[0]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = LLM(model="preset:x", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate([prompt], sp)[0]
    eng = SpeculativeEngine(_opts(num_speculative_tokens=1, speculative_algorithm="MTP", num_kv_blocks=32, host_blocks_factor=2.0),
                            model_args=args, model=model)
    n_target = sum(len(layer) for layer in eng.worker.kv_caches)
    assert len(eng.host_tier.tensors) == n_target + sum(len(layer) for layer in eng.draft_kv)
    assert eng.sleep(1) is False                              # engines with a draft module do not sleep
    llm = LLM(model="preset:x", devices="cpu", engine=eng)
    assert llm.generate([prompt], sp)[0].outputs[0].token_ids == want.outputs[0].token_ids
    assert eng.scheduler.stats()["host_offloaded_blocks"] == 4
    before = [t.clone() for layer in eng.draft_kv for t in layer]
    # the device cache loses everything (target and draft parts alike), once the copies to the host have let go of the blocks
    while eng.scheduler.has_pending_transfers:
        eng.scheduler.schedule()
        eng._publish_transfers_only(1)
    bm = eng.scheduler.block_manager(0)
    assert bm.evict(bm.num_blocks) >= 4
    for layer in list(eng.worker.kv_caches) + list(eng.draft_kv):
        for t in layer:
            t.zero_()
    out = llm.generate([prompt], sp)[0]
    assert out.outputs[0].token_ids == want.outputs[0].token_ids and out.usage.num_cached_tokens == 64
    assert eng.scheduler.stats()["host_loaded_blocks"] == 4
    after = [t for layer in eng.draft_kv for t in layer]
    # the four reloaded blocks carry the draft KV that was computed the first time (somewhere in the cache, under new ids)
    for b, a in zip(before, after):
        old_rows = {tuple(r.flatten().tolist()) for r in b if r.abs().sum() > 0}
        new_rows = {tuple(r.flatten().tolist()) for r in a if r.abs().sum() > 0}
        assert len(old_rows & new_rows) >= 4


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


def test_mtp_export_tool_and_loading_of_the_exported_draft(tmp_path):
    """Full checkpoint with an MTP block at layer `num_hidden_layers` (two of its matrices fp8 block-scaled) -> export ->
    the draft directory has the reference tool's layout and loads into the same MTP module as the full checkpoint."""
    import json
    from xllm_wxh_b200.models.deepseek_impl import DeepseekMTP
    from xllm_wxh_b200.ops import reference as ref
    from xllm_wxh_b200.tools import export_mtp
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, save_safetensors
    args = tiny_ds(hidden_size=256, q_lora_rank=128, kv_lora_rank=128, moe_intermediate_size=128, intermediate_size=256,
                   qk_nope_head_dim=32, v_head_dim=32, n_heads=4, num_nextn_predict_layers=1)
    target = DeepseekForCausalLM(args, device="cpu").init_random(seed=1, std=0.05)
    mtp = DeepseekMTP(args, device="cpu", target=target).init_random(seed=2, std=0.05)
    n = args.n_layers
    sd = dict(target.state_dict())
    msd = {k: v for k, v in mtp.state_dict().items() if k.startswith(f"model.layers.{n}.")}
    p = f"model.layers.{n}."
    msd.update({p + "enorm.weight": mtp.enorm, p + "hnorm.weight": mtp.hnorm, p + "eh_proj.weight": mtp.eh_proj.w,
                p + "shared_head.norm.weight": mtp.shared_head_norm, p + "embed_tokens.weight": target.embed,
                p + "shared_head.head.weight": target.lm_head})
    quantised = []
    for k in list(msd):
        v = msd[k]
        if v.dim() == 2 and "proj" in k and "eh_proj" not in k and v.shape[0] % 128 == 0 and v.shape[1] % 128 == 0 and len(quantised) < 2:
            w8, s = ref.quant_weight_128x128(v)
            msd[k], msd[k.replace(".weight", ".weight_scale_inv")] = w8, s
            quantised.append(k)
    assert len(quantised) == 2
    src = tmp_path / "full"
    src.mkdir()
    save_safetensors(str(src / "model-00001-of-00002.safetensors"), sd)
    save_safetensors(str(src / "model-00002-of-00002.safetensors"), msd)
    cfg = {"model_type": "deepseek_v3", "architectures": ["DeepseekV3ForCausalLM"], "num_hidden_layers": n,
           "num_nextn_predict_layers": 1, "first_k_dense_replace": 1, "hidden_size": args.hidden_size,
           "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}
    (src / "config.json").write_text(json.dumps(cfg))
    (src / "tokenizer_config.json").write_text("{}")
    assert export_mtp.detect_model_type(cfg) == "deepseek_v3"
    assert export_mtp.detect_model_type({**cfg, "index_topk": 2048}) == "deepseek_v32"
    dst = tmp_path / "draft"
    assert export_mtp.main(["--input-dir", str(src), "--output-dir", str(dst)]) == 0
    out_cfg = json.loads((dst / "config.json").read_text())
    assert out_cfg["num_hidden_layers"] == 1 and out_cfg["model_type"] == "deepseek_v3_mtp"
    assert out_cfg["architectures"] == ["DeepseekMTPForCausalLM"] and out_cfg["first_k_dense_replace"] == 0
    assert out_cfg["quantization_config"] == "" and (dst / "tokenizer_config.json").exists()
    ck = CheckpointReader(str(dst))
    keys = set(ck.keys())
    assert {"model.enorm.weight", "model.hnorm.weight", "model.eh_proj.weight", "model.shared_head.norm.weight",
            "model.embed_tokens.weight", "model.shared_head.head.weight", "model.layers.0.input_layernorm.weight"} <= keys
    assert not any("weight_scale_inv" in k for k in keys) and not any(k.startswith(f"model.layers.{n}.") for k in keys)
    q0 = quantised[0].replace(p, "model.layers.0.")
    assert ck.get(q0).dtype == torch.bfloat16
    index = json.loads((dst / "model.safetensors.index.json").read_text())["weight_map"]
    assert set(index) == keys and set(index.values()) == {"mtp_layer_parameters.safetensors"}
    # both directories load into the same module
    from_full = DeepseekMTP(args, device="cpu", target=target).load_weights(CheckpointReader(str(src)))
    from_draft = DeepseekMTP(args, device="cpu", target=target).load_weights(ck)
    for name in ("enorm", "hnorm", "shared_head_norm"):
        assert torch.equal(getattr(from_full, name), getattr(mtp, name)) and torch.equal(getattr(from_draft, name), getattr(mtp, name))
    assert torch.equal(from_draft.eh_proj.w, mtp.eh_proj.w)
    a, b, c = mtp.state_dict(), from_full.state_dict(), from_draft.state_dict()
    for k in a:
        if not k.startswith(p):
            continue
        tol = 0.07 * a[k].abs().max() if k in quantised else 1e-6
        assert (a[k].float() - b[k].float()).abs().max() <= tol, k
        assert (a[k].float() - c[k].float()).abs().max() <= max(tol, 0.01 * a[k].abs().max()), k      # bf16 after dequantisation
    with pytest.raises(ValueError):
        export_mtp.export(str(src), str(tmp_path / "x"), model_type="llama")


# ----------------------------------------------------------------------------- EAGLE-3
def _qwen_small():
    from xllm_wxh_b200.models.args import ModelArgs
    return ModelArgs(model_type="qwen3", dtype="float32", vocab_size=512, hidden_size=128, n_layers=6, n_heads=4, n_kv_heads=2,
                     head_dim=32, intermediate_size=256, qk_norm=True, max_position_embeddings=512)


@pytest.mark.parametrize("k,draft_vocab", [(1, 0), (3, 0), (2, 128)])
def test_eagle3_speculative_equals_plain_greedy(k, draft_vocab):
    """An EAGLE-3 draft (one layer over the target's layer-2 / middle / high hidden states, optionally with its own smaller
    vocabulary mapped through d2t) proposes k tokens per step; the emitted tokens are those of plain greedy decoding."""
    from xllm_wxh_b200.models.eagle3 import Eagle3Draft, default_capture_layers
    args = _qwen_small()
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    draft = Eagle3Draft(args, device="cpu", target=model, draft_vocab_size=draft_vocab).init_random(seed=3, std=0.08)
    prompts = _prompts(args.vocab_size, (20, 33, 7))
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    plain = LLM(model="preset:x", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)
    model.capture_layers = None
    eng = SpeculativeEngine(_opts(num_speculative_tokens=k, speculative_algorithm="Eagle3"), model_args=args, model=model,
                            draft_model=draft)
    assert model.capture_layers == default_capture_layers(6) == [2, 3]
    spec = LLM(model="preset:x", devices="cpu", engine=eng).generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert eng.stat_draft_tokens > 0
    if draft_vocab:
        # proposals are target ids out of the draft's hot-token table
        hot = (draft.d2t + torch.arange(draft_vocab)).tolist()
        assert all(t in hot for d in eng.drafts.values() for t in d)
    model.capture_layers = None


def test_eagle3_draft_that_copies_the_target_is_accepted():
    """Sanity of the plumbing (token shift, hidden-state rows, d2t): a 'draft' that answers with the target's own next
    token (it runs the target's last layers on the captured state) would be accepted every time; here the cheaper check:
    the draft's proposals do not depend on how the step was batched."""
    from xllm_wxh_b200.models.eagle3 import Eagle3Draft
    args = _qwen_small()
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    draft = Eagle3Draft(args, device="cpu", target=model).init_random(seed=3, std=0.08)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompts = _prompts(args.vocab_size, (18, 25))
    rates = []
    for chunk in (512, 7):                       # whole prompts against 7-token chunks: same drafts, same acceptance
        model.capture_layers = None
        eng = SpeculativeEngine(_opts(num_speculative_tokens=2, speculative_algorithm="Eagle3", max_tokens_per_chunk_for_prefill=chunk,
                                      max_tokens_per_batch=max(64, chunk)), model_args=args, model=model, draft_model=draft)
        LLM(model="preset:x", devices="cpu", engine=eng).generate(prompts, sp)
        rates.append((eng.stat_draft_tokens, eng.stat_accepted_tokens))
    assert rates[0] == rates[1]
    model.capture_layers = None


def test_eagle3_checkpoint_roundtrip(tmp_path):
    import json
    from xllm_wxh_b200.models.eagle3 import Eagle3Draft
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, save_safetensors
    args = _qwen_small()
    model = QwenForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    draft = Eagle3Draft(args, device="cpu", target=model, draft_vocab_size=128).init_random(seed=3, std=0.08)
    save_safetensors(str(tmp_path / "model.safetensors"), draft.state_dict())
    loaded = Eagle3Draft(args, device="cpu", target=model).load_weights(CheckpointReader(str(tmp_path)))
    assert loaded.draft_vocab == 128 and loaded.n_captured == 2 and torch.equal(loaded.d2t, draft.d2t)
    for k, v in draft.state_dict().items():
        assert torch.equal(loaded.state_dict()[k], v), k


@pytest.mark.parametrize("mode", ["PUSH", "PULL"])
@pytest.mark.parametrize("sparse", [False, True])
def test_mtp_draft_kv_travels_with_the_prefill_decode_hand_over(mode, sparse):
    """A PREFILL and a DECODE instance that both speculate with the MTP module: the hand-over moves the draft module's KV of
    the prompt's blocks together with the target's, so the decode instance's draft attends to the whole prompt; tokens
    equal plain greedy decoding on one engine.  `sparse`: DeepSeek-V3.2, whose index-key caches (target and draft) travel too."""
    from test_deepseek_cpu import tiny_v32
    from xllm_wxh_b200.parallel.kv_transfer import LocalCopyTransfer
    from xllm_wxh_b200.runtime.disagg_pd import DecodeCoordinator, InProcTransport, PrefillCoordinator
    from xllm_wxh_b200.runtime.master import LLMMaster
    args = (tiny_v32 if sparse else tiny_ds)(n_layers=2, num_nextn_predict_layers=1)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    prompts = _prompts(args.vocab_size, (40, 23, 9))
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in
            LLM(model="preset:x", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)]
    kw = dict(num_speculative_tokens=1, speculative_algorithm="MTP", enable_disagg_pd=True, kv_cache_transfer_mode=mode)
    p_eng = SpeculativeEngine(_opts(instance_role="PREFILL", **kw), model_args=args, model=model)
    d_eng = SpeculativeEngine(_opts(instance_role="DECODE", **kw), model_args=args, model=model)
    assert len(p_eng.transfer_caches()) == len(p_eng.worker.kv_caches) + len(p_eng.draft_kv)
    p_master, d_master = LLMMaster(p_eng.opt, p_eng), LLMMaster(d_eng.opt, d_eng)
    tp, td = InProcTransport.pair()
    dec = DecodeCoordinator(d_master)
    dec.attach(td)
    PrefillCoordinator(p_master, tp)
    move = LocalCopyTransfer(p_eng.transfer_caches(), d_eng.transfer_caches())
    if mode == "PUSH":
        p_eng.kv_transfer = move
    else:
        d_eng.kv_sources[0] = move
    p_master.idle_wait = lambda: d_master.step()
    llm = LLM(model="preset:x", devices="cpu", engine=p_eng)
    llm.master = p_master
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    assert move.bytes_moved > 0 and d_eng.stat_draft_tokens > 0
    # the decode instance's draft cache holds the prompt's draft KV that the prefill instance computed
    moved_rows = sum(int((t.abs().sum(dim=tuple(range(1, t.dim()))) > 0).sum()) for layer in d_eng.draft_kv for t in layer)
    assert moved_rows > 0


def test_multi_step_mtp_on_deepseek_v32_equals_plain_greedy():
    """DeepSeek-V3.2 under speculation: the verification rows (k + 1 per sequence) each rank their own causal keys, the
    draft module carries an indexer and an index-key cache of its own, and the emitted tokens stay those of plain
    greedy decoding of the sparse model."""
    from test_deepseek_cpu import tiny_v32
    args = tiny_v32(n_layers=2, num_nextn_predict_layers=1)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    prompts = _prompts(args.vocab_size, (20, 33, 7, 48))
    sp = SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True)
    plain = LLM(model="preset:x", devices="cpu", engine=LLMEngine(_opts(), model_args=args, model=model)).generate(prompts, sp)
    eng = SpeculativeEngine(_opts(num_speculative_tokens=2, speculative_algorithm="MTP", max_tokens_per_batch=64,
                                  max_tokens_per_chunk_for_prefill=24), model_args=args, model=model)
    assert eng.draft.indexer_on and len(eng.draft_kv[0]) == 2
    spec = LLM(model="preset:x", devices="cpu", engine=eng).generate(prompts, sp)
    for a, b in zip(plain, spec):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert eng.stat_draft_tokens > 0
