"""DeepSeek-V3-style model (MLA absorbed form, sigmoid group-limited routing, shared expert, YaRN) on CPU in fp32,
through the engine, against the plain non-absorbed oracle."""
import pytest
import torch

from oracle import deepseek_greedy
from xllm_wxh_b200 import LLM, SamplingParams
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import ModelArgs
from xllm_wxh_b200.models.deepseek_impl import DeepseekForCausalLM
from xllm_wxh_b200.ops import reference as ref
from xllm_wxh_b200.runtime.engine import LLMEngine


def tiny_ds(**kw):
    base = dict(model_type="deepseek_v3", dtype="float32", vocab_size=512, hidden_size=128, n_layers=3, n_heads=4, n_kv_heads=4,
                head_dim=48, intermediate_size=256, n_routed_experts=16, num_experts_per_tok=4, moe_intermediate_size=64,
                n_shared_experts=1, first_k_dense_replace=1, scoring_func="sigmoid", topk_method="noaux_tc", n_group=4, topk_group=2,
                routed_scaling_factor=2.5, q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                rope_theta=1e4, rope_scaling_type="yarn", rope_scaling_factor=4.0, rope_original_max_position=64, rope_mscale=1.0,
                rope_mscale_all_dim=1.0, max_position_embeddings=512)
    base.update(kw)
    return ModelArgs(**base)


def _yarn(args):
    inv = ref.yarn_inv_freq(args.qk_rope_head_dim, args.rope_theta, args.rope_scaling_factor, args.rope_original_max_position,
                            args.rope_beta_fast, args.rope_beta_slow)
    m_all = ref.yarn_mscale(args.rope_scaling_factor, args.rope_mscale_all_dim)
    mscale = ref.yarn_mscale(args.rope_scaling_factor, args.rope_mscale) / m_all
    return inv, mscale, (args.qk_nope_head_dim + args.qk_rope_head_dim) ** -0.5 * m_all * m_all


@pytest.mark.parametrize("q_lora", [64, 0])
def test_deepseek_greedy_matches_oracle(q_lora):
    args = tiny_ds(q_lora_rank=q_lora)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=0, std=0.08)
    sd = {k: v.float() for k, v in model.state_dict().items()}
    inv, mscale, sscale = _yarn(args)
    eng = LLMEngine(Options(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32",
                            max_tokens_per_chunk_for_prefill=24), model_args=args, model=model)
    llm = LLM(model="preset:x", devices="cpu", engine=eng)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (20, 37, 5)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == deepseek_greedy(sd, args, p, 10, inv, mscale, sscale)


def test_deepseek_checkpoint_roundtrip_fp8_block_scaled(tmp_path):
    """Write a bf16 checkpoint and an fp8 128x128 block-scaled one (HF `weight_scale_inv` layout); load both."""
    import json
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, save_safetensors
    args = tiny_ds(hidden_size=256, q_lora_rank=128, kv_lora_rank=128, moe_intermediate_size=128, intermediate_size=256,
                   qk_nope_head_dim=32, v_head_dim=32, n_heads=4)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=1, std=0.05)
    sd = model.state_dict()
    d = tmp_path / "bf16"
    d.mkdir()
    save_safetensors(str(d / "model.safetensors"), sd)
    loaded = DeepseekForCausalLM(args, device="cpu").load_weights(CheckpointReader(str(d)))
    for (k, a), (_, b) in zip(sorted(sd.items()), sorted(loaded.state_dict().items())):
        assert torch.equal(a, b), k
    # fp8 variant of the 2-D projection weights
    q = tmp_path / "fp8"
    q.mkdir()
    sdq = {}
    for k, v in sd.items():
        if v.dim() == 2 and "proj" in k and v.shape[0] % 128 == 0 and v.shape[1] % 128 == 0:
            w8, s = ref.quant_weight_128x128(v)
            sdq[k], sdq[k.replace(".weight", ".weight_scale_inv")] = w8, s
        else:
            sdq[k] = v
    save_safetensors(str(q / "model.safetensors"), sdq)
    deq = DeepseekForCausalLM(args, device="cpu").load_weights(CheckpointReader(str(q)))
    a, b = sd["model.layers.0.mlp.down_proj.weight"], deq.state_dict()["model.layers.0.mlp.down_proj.weight"]
    assert (a - b).abs().max() < 0.07 * a.abs().max()


def tiny_v32(**kw):
    base = dict(model_type="deepseek_v32", index_topk=12, index_n_heads=32, index_head_dim=32)   # many heads: no score is exactly 0
    base.update(kw)
    return tiny_ds(**base)


@pytest.mark.parametrize("interleave,chunk", [(False, 24), (True, 64), (False, 512)])
def test_deepseek_v32_sparse_attention_matches_oracle(interleave, chunk):
    """DeepSeek-V3.2: with index_topk = 12 every prompt below is longer than what a query may read, so the engine's path
    (index keys in their own paged cache, per-token top-k in chunked prefill and in batched decode, attention over the
    kept slots) must produce the tokens of the oracle, which masks a dense attention with the same ranking."""
    args = tiny_v32(index_rope_interleave=interleave)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=3, std=0.08)
    assert model.indexer_on and len(model.kv_cache_shapes(8, 16)[0]) == 2
    sd = {k: v.float() for k, v in model.state_dict().items()}
    assert "model.layers.0.self_attn.indexer.k_norm.bias" in sd
    inv, mscale, sscale = _yarn(args)
    eng = LLMEngine(Options(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=128, dtype="float32",
                            max_tokens_per_chunk_for_prefill=chunk), model_args=args, model=model)
    llm = LLM(model="preset:x", devices="cpu", engine=eng)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (20, 45, 5)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == deepseek_greedy(sd, args, p, 10, inv, mscale, sscale)
    # the ranking matters: the same weights with every key kept give other tokens for at least one prompt
    dense = tiny_v32(index_topk=4096, index_rope_interleave=interleave)
    assert any(o.outputs[0].token_ids != deepseek_greedy(sd, dense, p, 10, inv, mscale, sscale) for p, o in zip(prompts, outs))


def test_deepseek_v32_checkpoint_roundtrip_and_short_context_is_dense(tmp_path):
    """The indexer's tensors travel through a checkpoint under `self_attn.indexer.*`; while no sequence is longer than
    index_topk the selection is skipped and the output equals that of the same weights without an indexer."""
    import json
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, save_safetensors
    args = tiny_v32(index_topk=64)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=4, std=0.08)
    d = tmp_path / "v32"
    d.mkdir()
    save_safetensors(str(d / "model.safetensors"), model.state_dict())
    loaded = DeepseekForCausalLM(args, device="cpu").load_weights(CheckpointReader(str(d)))
    for a, b in zip(model.layers, loaded.layers):
        for n in ("wq_b", "wk", "weights_proj", "k_norm_w", "k_norm_b"):
            assert torch.equal(getattr(a.indexer, n), getattr(b.indexer, n))
    sd = {k: v.float() for k, v in model.state_dict().items()}
    inv, mscale, sscale = _yarn(args)
    eng = LLMEngine(Options(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=64, dtype="float32"), model_args=args,
                    model=loaded)
    llm = LLM(model="preset:x", devices="cpu", engine=eng)
    prompt = torch.randint(0, args.vocab_size, (30,), generator=torch.Generator().manual_seed(2)).tolist()
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0].outputs[0].token_ids
    assert out == deepseek_greedy(sd, tiny_ds(), prompt, 8, inv, mscale, sscale)


def test_deepseek_v32_without_indexer_configuration_is_refused():
    with pytest.raises(ValueError, match="index_topk"):
        DeepseekForCausalLM(tiny_ds(model_type="deepseek_v32"), device="cpu")


@pytest.mark.parametrize("padded", [False, True])
@pytest.mark.parametrize("lens,q_lens", [([20, 45, 5], [20, 45, 5]), ([40], [40]), ([33, 18, 50, 7], [1, 1, 1, 1]), ([30, 41], [3, 3])])
def test_lightning_indexer_select_against_brute_force(lens, q_lens, padded):
    """`select` (one sequence: shared keys; several: keys gathered per token; a captured step: padded rows and the full
    block-table width) keeps exactly the causal top-k of a score computed one token at a time."""
    import types
    from xllm_wxh_b200.models.indexer import LightningIndexer
    torch.manual_seed(0)
    args = ModelArgs(model_type="deepseek_v32", index_topk=12, index_n_heads=32, index_head_dim=32, qk_rope_head_dim=16)
    ix = LightningIndexer(args, "cpu", torch.float32)
    bs, nblk = 16, 40
    cache = torch.randn(nblk, bs, 32)
    B = len(lens) + (2 if padded else 0)
    bt = torch.zeros(B, 6 if padded else 4, dtype=torch.int32)
    perm, o = torch.randperm(nblk - 1) + 1, 0
    for i, L in enumerate(lens):
        nb = (L + bs - 1) // bs
        bt[i, :nb] = perm[o:o + nb].int()
        o += nb
    pos, seq = [], []
    for i, (L, n) in enumerate(zip(lens, q_lens)):
        pos += list(range(L - n, L))
        seq += [i] * n
    n_real = len(pos)
    if padded:
        pos, seq = pos + [0, 0, 0], seq + [-1, -1, -1]
    T = len(pos)
    q, w = torch.randn(T, 32, 32), torch.randn(T, 32)
    inp = types.SimpleNamespace(block_tables=bt, padded=padded, max_kv=max(lens), n_seqs=len(lens),
                                positions=torch.tensor(pos, dtype=torch.int32), token_seq=torch.tensor(seq, dtype=torch.int32))
    sel, sl = ix.select(q, w, cache, inp)
    assert sel.dtype == torch.int32 and sl.dtype == torch.int32 and sel.shape == (T, 12)
    assert int(sel.min()) >= 0 and int(sel.max()) < nblk * bs
    flat = cache.view(-1, 32)
    for t in range(n_real):
        i, p = seq[t], pos[t]
        slots = torch.tensor([int(bt[i, s // bs]) * bs + s % bs for s in range(p + 1)])
        sc = (torch.relu(q[t] @ flat[slots].t()) * w[t][:, None]).sum(0)
        want = slots[sc.topk(min(12, p + 1)).indices].tolist()
        assert int(sl[t]) == min(12, p + 1) and sel[t, :int(sl[t])].tolist() == want, t


def test_deepseek_v32_index_keys_travel_with_the_host_tier():
    """Prefix blocks that go device -> host -> device carry the index-key cache beside the latent cache: the second pass
    over prompts longer than index_topk, served from host blocks, gives the oracle's tokens (stale index keys would change
    the ranking)."""
    args = tiny_v32(n_layers=2)
    model = DeepseekForCausalLM(args, device="cpu").init_random(seed=5, std=0.08)
    sd = {k: v.float() for k, v in model.state_dict().items()}
    inv, mscale, sscale = _yarn(args)
    o = Options(model="preset:x", devices="cpu", block_size=16, num_kv_blocks=12, dtype="float32", host_blocks_factor=4.0,
                max_tokens_per_batch=64, max_seqs_per_batch=2)
    llm = LLM(model="preset:x", devices="cpu", engine=LLMEngine(o, model_args=args, model=model))
    eng = llm.engine
    assert eng.host_tier is not None
    per_block = sum(t[0].numel() * t.element_size() for layer in eng.worker.kv_caches for t in layer)
    assert eng.host_tier.stride >= per_block and len(eng.worker.kv_caches[0]) == 2
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, args.vocab_size, (64,), generator=g).tolist() for _ in range(4)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = [deepseek_greedy(sd, args, p, 6, inv, mscale, sscale) for p in prompts]
    first = [llm.generate([p], sp)[0] for p in prompts]              # 11 device blocks: each request evicts the one before
    assert [o_.outputs[0].token_ids for o_ in first] == want
    again = [llm.generate([p], sp)[0] for p in prompts]
    assert [o_.outputs[0].token_ids for o_ in again] == want
    st = eng.scheduler.stats()
    assert st["host_loaded_blocks"] >= 6 and sum(o_.usage.num_cached_tokens for o_ in again) >= 6 * 16
