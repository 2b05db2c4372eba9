"""Hot ops.  A CUDA tensor runs the hand-written sm_100a kernel from `libxllm_kernels.so`
(loaded by `cuda_ops`; missing library on a CUDA device is an error, never a silent fallback);
a CPU tensor runs the PyTorch statement of the same op from `reference`, which is also the oracle
the kernels are tested against."""
from __future__ import annotations

from . import reference as ref


def _cuda():
    from . import cuda_ops
    return cuda_ops


def rms_norm(x, w, eps):
    return _cuda().rms_norm(x, w, eps) if x.is_cuda else ref.rms_norm(x, w, eps)


def add_rms_norm(x, residual, w, eps):
    return _cuda().add_rms_norm(x, residual, w, eps) if x.is_cuda else ref.add_rms_norm(x, residual, w, eps)


def linear(x, w, bias=None):
    return _cuda().linear(x, w, bias) if x.is_cuda else ref.linear(x, w, bias)


def silu_and_mul(x):
    return _cuda().silu_and_mul(x) if x.is_cuda else ref.silu_and_mul(x)


def embedding(ids, table):
    return _cuda().embedding(ids, table) if table.is_cuda else ref.embedding(ids, table)


def rope_qknorm_kvwrite(qkv, positions, slots, cos_sin, q_w, k_w, eps, k_cache, v_cache, n_q, n_kv, head_dim):
    f = _cuda().rope_qknorm_kvwrite if qkv.is_cuda else ref.rope_qknorm_kvwrite
    return f(qkv, positions, slots, cos_sin, q_w, k_w, eps, k_cache, v_cache, n_q, n_kv, head_dim)


def paged_attention(q, k_cache, v_cache, inp, scale, sliding_window=-1):
    """q [T, Hq, D]; `inp` is a StepInput (q_cu, kv_lens, block_tables, n_seqs, n_decode ...)."""
    if q.is_cuda:
        return _cuda().paged_attention(q, k_cache, v_cache, inp, scale, sliding_window)
    return ref.paged_attention(q, k_cache, v_cache, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale,
                               sliding_window)


def sample(logits, inp):
    """Penalties -> temperature -> top-k/top-p -> sample/argmax (+logprobs).  Returns
    (tokens int32 [S], logprobs | None, top_vals | None, top_ids | None)."""
    if logits.is_cuda:
        return _cuda().sample(logits, inp)
    lg = logits.float()
    S = lg.shape[0]
    if inp.any_penalty:
        ref.apply_penalties(lg, inp.pen_cu[:S + 1], inp.pen_ids, inp.pen_counts, inp.rep_pen[:S], inp.freq_pen[:S],
                            inp.pres_pen[:S])
    return ref.sample(lg, inp.temperature[:S], inp.top_k[:S], inp.top_p[:S], inp.seed_lo[:S], inp.seed_hi[:S],
                      inp.any_logprobs, inp.max_top_logprobs)


def topk_candidates(logits, inp, id_offset: int, width: int):
    """Candidates of one vocabulary slice for vocabulary-parallel sampling (values, global ids, overflow flag)."""
    if logits.is_cuda:
        return _cuda().topk_candidates(logits, inp, id_offset, width)
    S = logits.shape[0]
    return ref.topk_candidates(logits, inp.temperature[:S], inp.top_k[:S], id_offset, width)


def moe_router(logits, top_k, scoring="softmax", renorm=True, bias=None, n_group=1, topk_group=1, route_scale=1.0):
    f = _cuda().moe_router if logits.is_cuda else ref.moe_router
    return f(logits, top_k, scoring, renorm, bias, n_group, topk_group, route_scale)


def moe_experts(x, w13, w2, weights, ids, expert_offset=0, interleaved=False):
    """`interleaved`: w13 rows were re-ordered by `finalize_weights` for the fused SwiGLU epilogue (CUDA only)."""
    if x.is_cuda:
        return _cuda().moe_experts(x, w13, w2, weights, ids, expert_offset, interleaved)
    assert not interleaved
    return ref.moe_experts(x, w13, w2, weights, ids, expert_offset)


def gate_up_swiglu(x, w, interleaved=False):
    """silu(x Wg^T) * (x Wu^T) with W = [gate rows; up rows] (or the interleaved layout on CUDA: one fused kernel)."""
    if x.is_cuda and interleaved:
        return _cuda().linear_swiglu(x, w)
    assert not interleaved
    return silu_and_mul(linear(x, w))


# ----------------------------------------------------------------------------- MLA (DeepSeek)
def mla_prepare(q, kv_a, positions, slots, cos_sin, kv_norm_w, eps, cache, w_kc, nope, rope, kv_lora):
    """Latent RMSNorm + interleaved RoPE of k_pe -> one [kv_lora + rope] cache row per token; RoPE of q_pe; q_nope absorbed
    into the latent space with W_kc.  Returns (q_lat [T, Hh, kv_lora], q_pe [T, Hh, rope])."""
    if q.is_cuda:
        return _cuda().mla_prepare(q, kv_a, positions, slots, cos_sin, kv_norm_w, eps, cache, w_kc, nope, rope, kv_lora)
    import torch
    T = q.shape[0]
    cs = cos_sin.index_select(0, positions.long())
    cos, sin = cs[:, :rope // 2], cs[:, rope // 2:]
    latent = ref.rms_norm(kv_a[:, :kv_lora], kv_norm_w, eps)
    k_pe = ref.apply_rope_interleaved(kv_a[:, None, kv_lora:], cos, sin)[:, 0]
    cache.view(-1, kv_lora + rope).index_copy_(0, slots.long(), torch.cat([latent, k_pe], -1).to(cache.dtype))
    q_pe = ref.apply_rope_interleaved(q[..., nope:], cos, sin)
    q_lat = torch.einsum("thn,hnc->thc", q[..., :nope].float(), w_kc.float()).to(q.dtype)
    return q_lat, q_pe


def mla_attention(q_lat, q_pe, cache, inp, scale, kv_lora):
    if q_lat.is_cuda:
        return _cuda().mla_attention(q_lat, q_pe, cache, inp, scale, kv_lora)
    return ref.mla_attention(q_lat, q_pe, cache, inp.q_cu, inp.kv_lens, inp.block_tables, inp.n_seqs, scale, kv_lora)


def mla_attention_sparse(q_lat, q_pe, cache, sel, sel_len, scale, kv_lora):
    """MLA attention in which query token t reads only the cache slots `sel[t, :sel_len[t]]` (what a lightning indexer
    kept for it; the selection is causal already, so no mask applies).  Layouts as `mla_attention`."""
    if q_lat.is_cuda:
        return _cuda().mla_attention_sparse(q_lat, q_pe, cache, sel, sel_len, scale, kv_lora)
    return ref.mla_attention_sparse(q_lat, q_pe, cache, sel, sel_len, scale, kv_lora)


def mla_v_up(o_lat, w_vc):
    """[T, Hh, kv_lora] x W_vc [Hh, v, kv_lora] -> [T, Hh * v]."""
    if o_lat.is_cuda:
        return _cuda().mla_v_up(o_lat, w_vc)
    import torch
    return torch.einsum("thc,hvc->thv", o_lat.float(), w_vc.float()).to(o_lat.dtype).reshape(o_lat.shape[0], -1)


def linear_fp8_block(x, wq, wscale):
    """Block-scaled fp8 linear: dynamic 1x128 activation scales, 128x128 weight scales."""
    if x.is_cuda:
        return _cuda().linear_fp8_block(x, wq, wscale)
    return ref.linear_fp8_block(x, wq, wscale, x.dtype)


def moe_experts_q(x, layer, weights, ids, expert_offset=0):
    """Routed experts of a layer object carrying `w13`, `w2` and optional fp8 block scales `w13_scale`, `w2_scale`."""
    if layer.w13_scale is None:
        return moe_experts(x, layer.w13, layer.w2, weights, ids, expert_offset, layer.interleaved)
    if x.is_cuda:
        return _cuda().moe_experts_fp8(x, layer.w13, layer.w13_scale, layer.w2, layer.w2_scale, weights, ids, expert_offset)
    import torch
    w13 = torch.stack([ref.dequant_weight_128x128(layer.w13[e], layer.w13_scale[e]) for e in range(layer.w13.shape[0])]).to(x.dtype)
    w2 = torch.stack([ref.dequant_weight_128x128(layer.w2[e], layer.w2_scale[e]) for e in range(layer.w2.shape[0])]).to(x.dtype)
    # activations go through the same 1x128 quantisation as on the GPU path
    return ref.moe_experts_fp8(x, w13, w2, weights, ids, expert_offset)


# ----------------------------------------------------------------------------- fp8 with per-row activation / per-channel weight scales
def quant_rows_fp8(x):
    return _cuda().quant_rows_fp8(x) if x.is_cuda else ref.quant_rows_fp8(x)


def rms_norm_quant_fp8(x, w, eps):
    """(e4m3 RMSNorm(x) * w, row scales)."""
    if x.is_cuda:
        return _cuda().rms_norm_quant_fp8(x, w, eps)
    return ref.quant_rows_fp8(ref.rms_norm(x, w, eps))


def add_rms_norm_quant_fp8(x, residual, w, eps):
    """(e4m3 RMSNorm(x + residual) * w, row scales, x + residual)."""
    if x.is_cuda:
        return _cuda().add_rms_norm_quant_fp8(x, residual, w, eps)
    h, res = ref.add_rms_norm(x, residual, w, eps)
    q, s = ref.quant_rows_fp8(h)
    return q, s, res


def linear_fp8_scaled(xq, xs, wq, col_scale=None, tensor_scale=1.0, bias=None, swiglu=False, cpu_dtype=None):
    """(xq wq^T) * xs[m] * tensor_scale * col_scale[n] (+ bias).  `swiglu`: silu(gate) * up of the result (on CUDA `wq` then
    holds the interleaved gate / up rows and the GEMM epilogue applies it; on the CPU the plain [gate; up] rows)."""
    if xq.is_cuda:
        return _cuda().linear_fp8_scaled(xq, xs, wq, col_scale, tensor_scale, bias, swiglu)
    import torch
    y = ref.linear_fp8_scaled(xq, xs, wq, col_scale, tensor_scale, bias, out_dtype=cpu_dtype or torch.float32)
    return silu_and_mul(y) if swiglu else y
