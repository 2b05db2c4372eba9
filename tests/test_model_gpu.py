"""Whole-model checks on a GPU: the kernel path against the PyTorch statement of the same model, eager against
CUDA-graph replay, and the engine end to end."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from xllm_wxh_b200 import LLM, SamplingParams, ops
from xllm_wxh_b200.config import Options
from xllm_wxh_b200.models.args import ModelArgs
from xllm_wxh_b200.models.qwen import QwenForCausalLM
from xllm_wxh_b200.runtime.engine import LLMEngine


def small_args(**kw):
    base = dict(model_type="qwen3", vocab_size=2048, hidden_size=512, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=128,
                intermediate_size=1536, qk_norm=True, rope_theta=1e6, max_position_embeddings=4096, dtype="bfloat16")
    base.update(kw)
    return ModelArgs(**base)


def _engine(args, model=None, **kw):
    o = dict(model="preset:x", devices="cuda:0", block_size=16, num_kv_blocks=512, max_tokens_per_batch=2048,
             max_seqs_per_batch=64)
    o.update(kw)
    return LLMEngine(Options(**o), model_args=args, model=model)


class _RefOps:
    """Routes the `ops` entry points to the PyTorch reference for tensors on the GPU."""
    def __enter__(self):
        import xllm_wxh_b200.ops as o
        self.saved = o._cuda
        from xllm_wxh_b200.ops import reference as r

        class Shim:
            rms_norm = staticmethod(r.rms_norm)
            add_rms_norm = staticmethod(r.add_rms_norm)
            linear = staticmethod(r.linear)
            silu_and_mul = staticmethod(r.silu_and_mul)
            embedding = staticmethod(r.embedding)
            rope_qknorm_kvwrite = staticmethod(r.rope_qknorm_kvwrite)
            moe_router = staticmethod(r.moe_router)
            moe_experts = staticmethod(lambda x, w13, w2, w, ids, e0=0, interleaved=False: r.moe_experts(x, w13, w2, w, ids, e0))

            @staticmethod
            def paged_attention(q, kc, vc, inp, scale, window=-1):
                return r.paged_attention(q, kc, vc, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale, window)
        o._cuda = lambda: Shim
        return self

    def __exit__(self, *a):
        import xllm_wxh_b200.ops as o
        o._cuda = self.saved


def _one_step_logits(engine, prompts):
    for p in prompts:
        engine.add_request(p)
    batches = engine.scheduler.schedule()
    b = batches[0]
    w = engine.worker
    T, B, MB, S, P, padded = w.choose_caps(b.num_tokens, b.num_seqs, b.max_blocks, b.num_sample_rows, False)
    L = w.layout_for(T, B, MB, S, P)
    host = w.host_staging(L.total_words)
    assert b.build(L, host.data_ptr(), host.numel(), engine.block_size) == 0
    from xllm_wxh_b200.framework.step_input import StepInput
    hdr = host[L.header:L.header + 32].numpy().copy()
    w._dev[:L.total_words].copy_(host[:L.total_words])
    inp = StepInput(w._dev, L, hdr)
    with torch.inference_mode():
        hidden = w.model.forward(inp, w.kv_caches)
        return w.model.logits(hidden, inp.sample_idx).float().cpu()


@pytest.mark.parametrize("kind", ["qwen3", "qwen2", "qwen3_moe"])
def test_forward_matches_reference_ops(kind):
    args = {"qwen3": small_args(), "qwen2": small_args(model_type="qwen2", qk_norm=False, attention_bias=True),
            "qwen3_moe": small_args(model_type="qwen3_moe", n_routed_experts=16, num_experts_per_tok=4,
                                    moe_intermediate_size=256)}[kind]
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=1, std=0.05)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (5, 64, 130, 33)]
    got = _one_step_logits(_engine(args, model), prompts)
    with _RefOps():
        want = _one_step_logits(_engine(args, model), prompts)
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert cos.min().item() > 0.995, cos
    assert (got - want).abs().max().item() < 0.05 * want.abs().max().item() + 0.05


def test_generate_eager_equals_graph_and_overlap():
    args = small_args()
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=2, std=0.05)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (7, 40, 19, 64, 3)]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    outs = {}
    for name, kw in {"eager": dict(enable_graph=False), "graph": dict(enable_graph=True),
                     "overlap": dict(enable_graph=True, enable_schedule_overlap=True)}.items():
        llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model, **kw))
        outs[name] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        if name == "graph":
            ge = llm.engine.worker._graphs
            assert ge is not None and ge.num_replays > 0 and ge.num_captures <= 4
    assert outs["eager"] == outs["graph"] == outs["overlap"]
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0


def test_generate_with_prefill_steps_in_graphs():
    """Steps that carry prefill tokens (pure prefill and chunked prefill mixed with decodes) replayed from CUDA graphs
    give the same tokens as eager execution."""
    args = small_args()
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=5, std=0.05)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (7, 150, 19, 64, 3, 90, 33, 200)]
    sp = [SamplingParams(temperature=0.0, max_tokens=6 + 3 * i, ignore_eos=True) for i in range(len(prompts))]
    outs = {}
    for name, kw in {"eager": dict(enable_graph=False),
                     "graph": dict(enable_graph=True, enable_prefill_piecewise_graph=True, max_tokens_per_batch=192,
                                   max_tokens_per_chunk_for_prefill=64)}.items():
        if name == "eager":
            kw.update(max_tokens_per_batch=192, max_tokens_per_chunk_for_prefill=64)
        llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model, **kw))
        if name == "graph":
            llm.engine.worker._graph_executor().capture_after = 1      # capture every shape at its first appearance
        outs[name] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        if name == "graph":
            ge = llm.engine.worker._graphs
            assert ge is not None and ge.num_replays >= ge.num_captures > 0
            assert any(k[-1] == 1 for k in ge.graphs), "no step with prefill tokens was captured"
    assert outs["eager"] == outs["graph"]
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0


def test_sampling_requests_and_logprobs_end_to_end():
    args = small_args()
    model = QwenForCausalLM(args, device="cuda:0").init_random(seed=3, std=0.05)
    llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, model))
    outs = llm.generate([[1, 2, 3, 4, 5], [9, 8, 7]],
                        [SamplingParams(temperature=0.9, top_k=20, top_p=0.9, max_tokens=12, ignore_eos=True, seed=7,
                                        repetition_penalty=1.2, logprobs=True, top_logprobs=3),
                         SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)])
    assert len(outs[0].outputs[0].token_ids) == 12 and len(outs[1].outputs[0].token_ids) == 5
    lps = outs[0].outputs[0].logprobs
    assert len(lps) == 12 and all(l.logprob <= 1e-4 for l in lps) and len(lps[0].top_logprobs) == 3


@pytest.mark.parametrize("scales", ["tensor", "channel"])
def test_fp8_checkpoint_is_served_in_fp8(tmp_path, monkeypatch, scales):
    """A dense checkpoint with e4m3 projection weights and per-tensor (or per-channel) scales keeps them in fp8 on the GPU:
    the GEMMs run on quantised operands with per-token activation scales.  Against the same checkpoint dequantised to bf16
    at load, the logits agree up to the activation-quantisation error, and greedy decoding runs through CUDA graphs."""
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader, save_safetensors
    args = small_args(qk_norm=True)
    sd = QwenForCausalLM(args, device="cpu", dtype=torch.float32).init_random(seed=6, std=0.05).state_dict()
    q = {}
    for k, v in sd.items():
        if k.endswith("_proj.weight"):
            amax = v.abs().amax(dim=None if scales == "tensor" else 1, keepdim=scales == "channel").clamp_min(1e-8)
            sc = (amax / 448.0).float()
            q[k] = (v / sc).to(torch.float8_e4m3fn)
            q[k.replace(".weight", ".weight_scale")] = sc.reshape(-1) if scales == "channel" else sc.reshape(1)
        else:
            q[k] = v.to(torch.bfloat16)
    save_safetensors(str(tmp_path / "model.safetensors"), q)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (5, 64, 130, 33)]

    def build(fp8: bool):
        monkeypatch.setenv("XLLM_FP8_LINEAR", "1" if fp8 else "0")
        m = QwenForCausalLM(args, device="cuda:0").load_weights(CheckpointReader(str(tmp_path))).finalize_weights()
        assert m.fp8_linears == fp8
        assert (m.layers[0].attn.qkv_w.dtype == torch.float8_e4m3fn) == fp8
        return m

    m8, m16 = build(True), build(False)
    got = _one_step_logits(_engine(args, m8), prompts)
    want = _one_step_logits(_engine(args, m16), prompts)
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert cos.min().item() > 0.99, cos
    # half the weight bytes of the projections
    assert m8.weight_bytes() < 0.75 * m16.weight_bytes()
    llm = LLM(model="preset:x", devices="cuda:0", engine=_engine(args, m8, enable_graph=True))
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 8 for o in outs)
    assert cuda_ops.read_status() == 0


# ----------------------------------------------------------------------------- DeepSeek (MLA + MoE) on the GPU
def ds_args(**kw):
    """The production head shape (latent 512 + rope 64, nope 128, v 128), which the MLA kernels serve, on a small model."""
    base = dict(model_type="deepseek_v3", dtype="bfloat16", vocab_size=1024, hidden_size=512, n_layers=3, n_heads=16, n_kv_heads=16,
                head_dim=192, intermediate_size=1024, n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=256,
                n_shared_experts=1, first_k_dense_replace=1, scoring_func="sigmoid", topk_method="noaux_tc", n_group=2, topk_group=1,
                routed_scaling_factor=1.5, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                v_head_dim=128, rope_theta=1e4, max_position_embeddings=2048)
    base.update(kw)
    return ModelArgs(**base)


def _ds_checkpoint(args, path):
    """Random DeepSeek weights (bf16-representable) written as a safetensors checkpoint both devices load from."""
    import dataclasses
    from xllm_wxh_b200.models.deepseek_impl import DeepseekForCausalLM
    from xllm_wxh_b200.utils.safetensors_io import save_safetensors
    cpu_args = dataclasses.replace(args, dtype="float32", quant=type(args.quant)())
    sd = DeepseekForCausalLM(cpu_args, device="cpu", dtype=torch.float32).init_random(seed=4, std=0.05).state_dict()
    save_safetensors(str(path / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in sd.items()})
    return str(path)


def _ds_generate(args, device, prompts, ckpt, **opt):
    from xllm_wxh_b200.models.deepseek_impl import DeepseekForCausalLM
    from xllm_wxh_b200.utils.safetensors_io import CheckpointReader
    dt = torch.float32 if device == "cpu" else torch.bfloat16
    model = DeepseekForCausalLM(args, device=device, dtype=dt).load_weights(CheckpointReader(ckpt))
    o = dict(model="preset:x", devices=device, block_size=16, num_kv_blocks=256, max_tokens_per_batch=1024, max_seqs_per_batch=16,
             dtype="float32" if device == "cpu" else "auto")
    o.update(opt)
    eng = LLMEngine(Options(**o), model_args=args, model=model)
    outs = LLM(model="preset:x", devices=device, engine=eng).generate(
        prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=True))
    return [o.outputs[0].token_ids for o in outs], [[l.logprob for l in o.outputs[0].logprobs] for o in outs]


def _agreeing_diffs(want_t, want_lp, got_t, got_lp):
    """|log-probability difference| at the positions two greedy runs can be compared at: while they have produced the same
    tokens (where an arg-max between two nearly equal logits falls the other way the sequences part)."""
    diffs, total = [], 0
    for wt, gt, wl, gl in zip(want_t, got_t, want_lp, got_lp):
        total += len(wt)
        for i in range(len(wt)):
            if wt[i] != gt[i]:
                break
            diffs.append(abs(wl[i] - gl[i]))
    return sorted(diffs), total


@pytest.mark.parametrize("mla_kernel", ["tcgen05", "mma_sync"])
@pytest.mark.parametrize("routing", ["all_experts", "top2_of_a_group"])
def test_deepseek_gpu_matches_cpu_reference(monkeypatch, tmp_path, mla_kernel, routing):
    """The whole MLA + MoE model through the CUDA kernels (bf16) against the PyTorch statement of the same model on the
    CPU in fp32, same checkpoint: greedy tokens and their log-probabilities, prefill and decode steps.
    `all_experts`: every routed expert is active, so nothing discrete separates the two runs and every log-probability
    must agree closely.  `top2_of_a_group`: group-limited sigmoid routing; a near-tie between two experts may fall the
    other way in bf16 and moves that token's logits, so most, not all, positions must agree."""
    import dataclasses
    monkeypatch.setenv("XLLM_MLA_TC", "1" if mla_kernel == "tcgen05" else "0")
    g = torch.Generator().manual_seed(0)
    args = ds_args() if routing == "top2_of_a_group" else ds_args(num_experts_per_tok=8, n_group=1, topk_group=1)
    ckpt = _ds_checkpoint(args, tmp_path)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (5, 70, 33, 130)]
    want_t, want_lp = _ds_generate(dataclasses.replace(args, dtype="float32"), "cpu", prompts, ckpt)
    got_t, got_lp = _ds_generate(args, "cuda:0", prompts, ckpt)
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0
    diffs, total = _agreeing_diffs(want_t, want_lp, got_t, got_lp)
    # The random model's logits are flat, so an arg-max often sits on a near-tie and the two runs part early; what must
    # hold: the prefill step's top log-probability agrees for every prompt (whichever of two tied tokens was taken), and
    # so does every later position that is still comparable.
    first = [abs(a[0] - b[0]) for a, b in zip(want_lp, got_lp)]
    assert max(first) < 0.12, first
    assert len(diffs) >= len(prompts)
    if routing == "all_experts":
        assert diffs[-1] < 0.12, diffs[-5:]
    else:
        assert diffs[int(0.75 * len(diffs))] < 0.12, diffs


@pytest.mark.parametrize("graphs", [False, True])
def test_deepseek_v32_sparse_attention_gpu_matches_cpu_reference(tmp_path, graphs):
    """DeepSeek-V3.2 with index_topk = 24 below the prompt lengths: index keys, per-token ranking and the attention over
    the kept slots on the GPU (bf16) against the same model on the CPU in fp32, same checkpoint.  A key on the edge of the
    kept set may fall the other way in bf16, which moves that token's logits a little, so most positions must agree."""
    import dataclasses
    from xllm_wxh_b200.ops import cuda_ops
    g = torch.Generator().manual_seed(0)
    args = ds_args(model_type="deepseek_v32", index_topk=24, index_n_heads=16, index_head_dim=128, num_experts_per_tok=8, n_group=1,
                   topk_group=1)
    ckpt = _ds_checkpoint(args, tmp_path)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (5, 70, 33, 130)]
    want_t, want_lp = _ds_generate(dataclasses.replace(args, dtype="float32"), "cpu", prompts, ckpt)
    before = cuda_ops.launch_count
    got_t, got_lp = _ds_generate(args, "cuda:0", prompts, ckpt, enable_graph=graphs)
    assert cuda_ops.read_status() == 0 and cuda_ops.launch_count > before
    first = [abs(a[0] - b[0]) for a, b in zip(want_lp, got_lp)]
    assert sorted(first)[len(first) // 2] < 0.12, first
    diffs, total = _agreeing_diffs(want_t, want_lp, got_t, got_lp)
    assert len(diffs) >= len(prompts) and diffs[len(diffs) // 2] < 0.12, diffs


def test_deepseek_fp8_block_scaled_gpu_close_to_bf16(tmp_path):
    """Block-scaled fp8 weights (128 x 128 scales, dynamic 1 x 128 activation scales) through the fp8 GEMMs and the fp8
    grouped GEMM of the experts: close to the bf16 model of the same checkpoint (quantised at load); decode under CUDA
    graphs."""
    import dataclasses
    from xllm_wxh_b200.models.args import QuantArgs
    g = torch.Generator().manual_seed(1)
    args = ds_args(num_experts_per_tok=8, n_group=1, topk_group=1)
    ckpt = _ds_checkpoint(args, tmp_path)
    prompts = [torch.randint(0, args.vocab_size, (n,), generator=g).tolist() for n in (9, 64, 200)]
    want_t, want_lp = _ds_generate(args, "cuda:0", prompts, ckpt)
    q = dataclasses.replace(args, quant=QuantArgs(method="fp8", weight_block_size=[128, 128]))
    got_t, got_lp = _ds_generate(q, "cuda:0", prompts, ckpt, enable_graph=True)
    from xllm_wxh_b200.ops import cuda_ops
    assert cuda_ops.read_status() == 0
    diffs, total = _agreeing_diffs(want_t, want_lp, got_t, got_lp)
    first = [abs(a[0] - b[0]) for a, b in zip(want_lp, got_lp)]
    assert max(first) < 0.35, first                                      # e4m3 weights and activations against bf16
    assert diffs[int(0.75 * len(diffs))] < 0.35, diffs
    assert all(len(t) == 6 for t in got_t)
