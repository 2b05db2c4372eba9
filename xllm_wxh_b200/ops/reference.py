"""Plain-PyTorch statements of every hot op.

These are (a) the CPU execution path of the engine (the tiny-Qwen2 fp32 configuration runs
entirely on them) and (b) the oracle each CUDA kernel is tested against.  The math follows the
reference's kernels: RMSNorm `cast(x*rstd)*w` (xllm/core/kernels/cuda/norm.cu:42-172), neox RoPE
with a `[cos|sin]` cache (rope.cu:27-53, rotary_embedding.cpp:28-50), fused per-head q/k RMSNorm +
RoPE (fused_qknorm_rope.cu:75-280), paged cache write (reshape_paged_cache.cu:23-59), SwiGLU
(activation.cu:46-99), sampling (framework/sampling/sampler.cpp:28-107, logits_utils.cpp).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd).to(x.dtype) * w


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    r = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(r, w, eps), r


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return torch.nn.functional.linear(x, w, bias)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (torch.nn.functional.silu(g) * u).to(x.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return table.index_select(0, ids.long().clamp_min(0))


def build_cos_sin_cache(rot_dim: int, max_pos: int, theta: float, dtype=torch.float32, device="cpu",
                        inv_freq: Optional[torch.Tensor] = None, mscale: float = 1.0) -> torch.Tensor:
    """[max_pos, rot_dim]: first half cos, second half sin (fp32 math, then cast)."""
    if inv_freq is None:
        inv_freq = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq.float())
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).to(dtype).to(device)


def yarn_inv_freq(rot_dim: int, theta: float, factor: float, orig_max: int, beta_fast: float, beta_slow: float) -> torch.Tensor:
    """YaRN frequency blend (reference: rotary_embedding_util.cpp:272-300; HF DeepSeek modelling code)."""
    pos_freqs = theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim)
    extra, inter = 1.0 / pos_freqs, 1.0 / (factor * pos_freqs)

    def corr_dim(n_rot):
        return (rot_dim * math.log(orig_max / (n_rot * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(rot_dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    mask = 1.0 - ramp
    return inter * (1 - mask) + extra * mask


def llama3_inv_freq(rot_dim: int, theta: float, factor: float, low_freq_factor: float, high_freq_factor: float,
                    orig_max: int) -> torch.Tensor:
    """Llama-3 frequency scaling: wavelengths beyond the original context / low_freq_factor are slowed by `factor`, those
    below the original context / high_freq_factor stay, the band between is blended linearly."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    wavelen = 2 * math.pi / inv
    low_wl, high_wl = orig_max / low_freq_factor, orig_max / high_freq_factor
    smooth = ((orig_max / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)).clamp(0, 1)
    blended = (1 - smooth) * inv / factor + smooth * inv
    out = torch.where(wavelen > low_wl, inv / factor, inv)
    mid = (wavelen <= low_wl) & (wavelen >= high_wl)
    return torch.where(mid, blended, out)


def scaled_cos_sin_cache(args, rot_dim: int, dtype=torch.float32, device="cpu") -> torch.Tensor:
    """cos / sin table of a dense model under its rope scaling ("", linear, llama3, yarn)."""
    kind, theta, f = args.rope_scaling_type, args.rope_theta, args.rope_scaling_factor
    inv, mscale = None, 1.0
    if kind == "linear":
        inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim)) / f
    elif kind == "llama3":
        inv = llama3_inv_freq(rot_dim, theta, f, args.rope_low_freq_factor, args.rope_high_freq_factor,
                              args.rope_original_max_position)
    elif kind == "yarn":
        inv = yarn_inv_freq(rot_dim, theta, f, args.rope_original_max_position, args.rope_beta_fast, args.rope_beta_slow)
        mscale = args.rope_attention_factor or yarn_mscale(f, 1.0)
    return build_cos_sin_cache(rot_dim, args.max_position_embeddings, theta, dtype=dtype, device=device, inv_freq=inv, mscale=mscale)


def yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def apply_rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, H, D]; cos/sin [T, D/2]; pairs are (x[i], x[i+D/2])."""
    d2 = x.shape[-1] // 2
    a, b = x[..., :d2].float(), x[..., d2:].float()
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


def apply_rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, H, D]; pairs are (x[2i], x[2i+1]) (GPT-J style, used by MLA)."""
    a, b = x[..., 0::2].float(), x[..., 1::2].float()
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    out = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    return out.to(x.dtype)


def rope_qknorm_kvwrite(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, cos_sin: torch.Tensor,
                        q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """Per-head q/k RMSNorm (optional) -> neox RoPE -> K,V scattered into the paged cache.
    Returns q as [T, n_q*head_dim]."""
    T = qkv.shape[0]
    q, k, v = qkv.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
    q = q.reshape(T, n_q, head_dim)
    k = k.reshape(T, n_kv, head_dim)
    v = v.reshape(T, n_kv, head_dim)
    if q_w is not None:
        q = rms_norm(q, q_w, eps)
        k = rms_norm(k, k_w, eps)
    cs = cos_sin.index_select(0, positions.long())
    rot = cos_sin.shape[-1]
    cos, sin = cs[:, : rot // 2], cs[:, rot // 2:]
    q = apply_rope_neox(q, cos, sin)
    k = apply_rope_neox(k, cos, sin)
    kc = k_cache.view(-1, n_kv, head_dim)
    vc = v_cache.view(-1, n_kv, head_dim)
    kc.index_copy_(0, slots.long(), k.to(kc.dtype))
    vc.index_copy_(0, slots.long(), v.to(vc.dtype))
    return q.reshape(T, n_q * head_dim)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, q_cu: torch.Tensor,
                    kv_lens: torch.Tensor, block_tables: torch.Tensor, n_seqs: int, scale: float,
                    sliding_window: int = -1) -> torch.Tensor:
    """Causal attention of ragged query rows over paged KV.
    q [T, Hq, D]; caches [n_blocks, block, Hkv, D]; sequence i owns q rows q_cu[i]:q_cu[i+1], which are the
    last rows of its kv_lens[i] tokens."""
    T, Hq, D = q.shape
    block = k_cache.shape[1]
    Hkv = k_cache.shape[2]
    Dv = v_cache.shape[-1]
    group = Hq // Hkv
    out = torch.zeros(T, Hq, Dv, dtype=q.dtype, device=q.device)
    q_cu_h = q_cu.tolist()
    kv_h = kv_lens.tolist()
    for i in range(n_seqs):
        qs, qe = q_cu_h[i], q_cu_h[i + 1]
        L = kv_h[i]
        if qe <= qs or L <= 0:
            continue
        nb = (L + block - 1) // block
        blocks = block_tables[i, :nb].long()
        k = k_cache.index_select(0, blocks).reshape(nb * block, Hkv, D)[:L].float()
        v = v_cache.index_select(0, blocks).reshape(nb * block, Hkv, Dv)[:L].float()
        qi = q[qs:qe].float()                       # [n, Hq, D]
        n = qe - qs
        k = k.repeat_interleave(group, dim=1)       # [L, Hq, D]
        v = v.repeat_interleave(group, dim=1)
        s = torch.einsum("nhd,lhd->hnl", qi, k) * scale
        qpos = torch.arange(L - n, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        mask = kpos <= qpos
        if sliding_window > 0:
            mask &= kpos > qpos - sliding_window
        s = s.masked_fill(~mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qe] = torch.einsum("hnl,lhd->nhd", p, v).to(q.dtype)
    return out.reshape(T, Hq * Dv)


# ----------------------------------------------------------------------------- sampling
def apply_penalties(logits: torch.Tensor, pen_cu: torch.Tensor, pen_ids: torch.Tensor, pen_counts: torch.Tensor,
                    rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> torch.Tensor:
    """In place.  Row r owns entries pen_cu[r]:pen_cu[r+1] of (token id, count); a count holds the occurrences in the whole
    sequence in its low half and those among the generated tokens in its high half.  Frequency and presence penalties use
    the generated count (prompt tokens alone are not penalised), the repetition penalty applies to every listed id."""
    cu = pen_cu.tolist()
    for r in range(logits.shape[0]):
        a, b = cu[r], cu[r + 1]
        if b <= a:
            continue
        ids = pen_ids[a:b].long()
        cnt = ((pen_counts[a:b] >> 16) & 0xFFFF).to(logits.dtype)
        sc = logits[r, ids]
        sc = sc - cnt * freq[r] - (cnt > 0).to(logits.dtype) * pres[r]
        sc = torch.where(sc < 0, sc * rep[r], sc / rep[r])
        logits[r, ids] = sc
    return logits


def top_k_top_p_filter(logits: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor) -> torch.Tensor:
    """Sort-based masking, the reference's formulation (logits_utils.cpp:61-160)."""
    V = logits.shape[-1]
    sorted_logits, idx = logits.sort(dim=-1, descending=True)
    k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k).clamp(max=V).long()
    ranks = torch.arange(V, device=logits.device)[None, :]
    mask = ranks >= k[:, None]
    probs = torch.softmax(sorted_logits.masked_fill(mask, float("-inf")), dim=-1)
    cum = probs.cumsum(-1)
    mask |= (cum - probs) > top_p[:, None]
    sorted_logits = sorted_logits.masked_fill(mask, float("-inf"))
    return torch.empty_like(logits).scatter_(-1, idx, sorted_logits)


def _uniform_from_seed(seed_lo: torch.Tensor, seed_hi: torch.Tensor) -> torch.Tensor:
    """One uniform in (0,1) per row from a 64-bit seed (splitmix64 finaliser), identical on host and device."""
    s = (seed_lo.to(torch.int64) & 0xFFFFFFFF) | (seed_hi.to(torch.int64) << 32)
    out = []
    for v in s.tolist():
        z = (v + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
        z = z ^ (z >> 31)
        out.append(((z >> 40) + 0.5) / float(1 << 24))
    return torch.tensor(out, dtype=torch.float32, device=seed_lo.device)


def topk_candidates(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, id_offset: int, width: int):
    """The top_k largest logits of every row of a vocabulary slice, ties at the k-th included (the arg-max for rows with
    temperature 0), in index order: (values fp32 [S, width], global ids int32 [S, width], overflow int32 [1])."""
    lg = logits.float()
    S, V = lg.shape
    vals = torch.full((S, width), float("-inf"), dtype=torch.float32, device=lg.device)
    ids = torch.full((S, width), -1, dtype=torch.int32, device=lg.device)
    over = torch.zeros(1, dtype=torch.int32, device=lg.device)
    for r in range(S):
        k = 1 if float(temperature[r]) == 0.0 else int(top_k[r])
        if k == 1:
            i = int(lg[r].argmax())
            vals[r, 0], ids[r, 0] = lg[r, i], i + id_offset
            continue
        if k <= 0 or k > width:
            over[0] = 1
            continue
        kth = torch.topk(lg[r], min(k, V)).values[-1]
        keep = (lg[r] >= kth).nonzero().flatten()
        if keep.numel() > width:
            over[0] = 1
            keep = keep[:width]
        vals[r, :keep.numel()] = lg[r, keep]
        ids[r, :keep.numel()] = (keep + id_offset).int()
    return vals, ids, over


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed_lo: torch.Tensor, seed_hi: torch.Tensor, want_logprobs: bool = False, max_top_logprobs: int = 0):
    """logits [S, V] (any float dtype).  Greedy where temperature == 0, else inverse-CDF sampling of the
    top-k/top-p filtered distribution in vocabulary order with one uniform per row.
    Returns (tokens int32 [S], logprobs fp32 [S] | None, top_vals | None, top_ids | None)."""
    lg = logits.float()
    greedy = temperature == 0
    t = torch.where(greedy, torch.ones_like(temperature), temperature)
    lg = lg / t[:, None]
    tokens = lg.argmax(-1)
    if not bool(greedy.all()):
        filt = top_k_top_p_filter(lg, top_k, top_p)
        probs = torch.softmax(filt, dim=-1)
        u = _uniform_from_seed(seed_lo, seed_hi).to(lg.device)
        cdf = probs.cumsum(-1)
        total = cdf[:, -1:]
        pick = (cdf < (u[:, None] * total)).sum(-1).clamp(max=lg.shape[-1] - 1)
        # never land on a masked token because of rounding
        ok = probs.gather(-1, pick[:, None]).squeeze(-1) > 0
        pick = torch.where(ok, pick, filt.argmax(-1))
        tokens = torch.where(greedy, tokens, pick)
    lp = tv = ti = None
    if want_logprobs:
        logp = torch.log_softmax(lg, dim=-1)
        lp = logp.gather(-1, tokens[:, None]).squeeze(-1)
        if max_top_logprobs > 0:
            tv, ti = logp.topk(max_top_logprobs, dim=-1)
            ti = ti.int()
    return tokens.int(), lp, tv, ti


# ----------------------------------------------------------------------------- MoE
def moe_router(logits: torch.Tensor, top_k: int, scoring: str = "softmax", renorm: bool = True,
               bias: Optional[torch.Tensor] = None, n_group: int = 1, topk_group: int = 1,
               route_scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router (reference: moe_topk_softmax_kernels.cuh:324-611, moe_topk_sigmoid_kernels.cuh:165-383,
    group-limited rule of the MLU `moe_active_topk` op, param.h:402-442).
    Returns (weights fp32 [T, k], expert ids int32 [T, k])."""
    lf = logits.float()
    scores = torch.softmax(lf, dim=-1) if scoring == "softmax" else torch.sigmoid(lf)
    sel = scores + bias.float()[None, :] if bias is not None else scores
    T, E = scores.shape
    if n_group > 1:
        g = sel.view(T, n_group, E // n_group)
        gscore = g.topk(2, dim=-1).values.sum(-1) if bias is not None else g.max(-1).values
        keep = gscore.topk(topk_group, dim=-1).indices
        gmask = torch.zeros(T, n_group, dtype=torch.bool, device=logits.device).scatter_(1, keep, True)
        sel = sel.masked_fill(~gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E), float("-inf"))
    ids = sel.topk(top_k, dim=-1).indices
    w = scores.gather(-1, ids)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return (w * route_scale).float(), ids.int()


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor,
                expert_offset: int = 0) -> torch.Tensor:
    """sum_k w_k * down_e(silu(gate_e x) * up_e x) over the experts held locally.
    w13 [E_local, 2I, H] (gate rows then up rows), w2 [E_local, H, I]."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E_local = w13.shape[0]
    for e in range(E_local):
        hit = (ids == e + expert_offset)
        tok = hit.any(-1).nonzero().squeeze(-1)
        if tok.numel() == 0:
            continue
        wk = (weights * hit).sum(-1)[tok]
        h = linear(x[tok], w13[e])
        h = silu_and_mul(h)
        y = linear(h, w2[e])
        out.index_add_(0, tok, y.float() * wk[:, None])
    return out.to(x.dtype)


def moe_experts_fp8(x, w13_deq, w2_deq, weights, ids, expert_offset=0):
    """As `moe_experts`, with the expert inputs passed through 1x128 e4m3 quantisation (what the fp8 GEMMs see)."""
    def fq(t):
        q, s = quant_act_1x128(t)
        return (q.float().view(t.shape[0], -1, 128) * s[..., None]).view(t.shape).to(t.dtype)
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(w13_deq.shape[0]):
        hit = (ids == e + expert_offset)
        tok = hit.any(-1).nonzero().squeeze(-1)
        if tok.numel() == 0:
            continue
        wk = (weights * hit).sum(-1)[tok]
        h = silu_and_mul(linear(fq(x[tok]), w13_deq[e]))
        y = linear(fq(h), w2_deq[e])
        out.index_add_(0, tok, y.float() * wk[:, None])
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- fp8 block scaling
FP8_MAX = 448.0


def quant_act_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token, per-128-column dynamic e4m3 quantisation.  x [T, K] -> (q fp8 [T, K], scale fp32 [T, K/128])."""
    T, K = x.shape
    g = x.float().view(T, K // 128, 128)
    amax = g.abs().amax(-1).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (g / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(T, K), scale


def quant_weight_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [N, K] -> (q fp8 [N, K], scale fp32 [ceil(N/128), ceil(K/128)]) (DeepSeek-V3 `weight_scale_inv`)."""
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blk = wp.view(nb, 128, kb, 128)
    amax = blk.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (blk / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(nb * 128, kb * 128)[:N, :K]
    return q.to(torch.float8_e4m3fn), scale


def dequant_weight_128x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    s = scale.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return q.float() * s


def linear_fp8_block(x: torch.Tensor, wq: torch.Tensor, wscale: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    """Block-scaled fp8 linear: dynamic 1x128 activation quant, 128x128 weight scales, fp32 accumulate."""
    xq, xs = quant_act_1x128(x)
    xd = xq.float().view(x.shape[0], -1, 128) * xs[..., None]
    return (xd.view(x.shape[0], -1) @ dequant_weight_128x128(wq, wscale).t()).to(out_dtype)


# ----------------------------------------------------------------------------- MLA
def mla_attention(q_lat: torch.Tensor, q_pe: torch.Tensor, cache: torch.Tensor, q_cu: torch.Tensor, kv_lens: torch.Tensor,
                  block_tables: torch.Tensor, n_seqs: int, scale: float, kv_lora: int) -> torch.Tensor:
    """Absorbed-form MLA over a single latent cache [n_blocks, block, kv_lora + rope].
    q_lat [T, H, kv_lora], q_pe [T, H, rope].  Returns [T, H, kv_lora] (caller applies W_vc)."""
    T, H, _ = q_lat.shape
    block = cache.shape[1]
    W = cache.shape[-1]
    out = torch.zeros(T, H, kv_lora, dtype=q_lat.dtype, device=q_lat.device)
    qc, kl = q_cu.tolist(), kv_lens.tolist()
    for i in range(n_seqs):
        qs, qe, L = qc[i], qc[i + 1], kl[i]
        if qe <= qs or L <= 0:
            continue
        nb = (L + block - 1) // block
        kv = cache.index_select(0, block_tables[i, :nb].long()).reshape(nb * block, W)[:L].float()
        lat, pe = kv[:, :kv_lora], kv[:, kv_lora:]
        n = qe - qs
        s = (torch.einsum("nhc,lc->hnl", q_lat[qs:qe].float(), lat) +
             torch.einsum("nhr,lr->hnl", q_pe[qs:qe].float(), pe)) * scale
        qpos = torch.arange(L - n, L, device=q_lat.device)[:, None]
        kpos = torch.arange(L, device=q_lat.device)[None, :]
        s = s.masked_fill(~(kpos <= qpos)[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qe] = torch.einsum("hnl,lc->nhc", p, lat).to(q_lat.dtype)
    return out


def mla_attention_sparse(q_lat: torch.Tensor, q_pe: torch.Tensor, cache: torch.Tensor, sel: torch.Tensor, sel_len: torch.Tensor,
                         scale: float, kv_lora: int) -> torch.Tensor:
    """Absorbed-form MLA in which token t attends to the cache slots sel[t, :sel_len[t]] only (no mask: the selection is
    causal).  q_lat [T, H, kv_lora], q_pe [T, H, rope], cache [n_blocks, block, kv_lora + rope]; returns [T, H, kv_lora]."""
    T, H, _ = q_lat.shape
    W = cache.shape[-1]
    flat = cache.reshape(-1, W)
    out = torch.empty(T, H, kv_lora, dtype=q_lat.dtype, device=q_lat.device)
    step = max(1, (1 << 24) // max(1, sel.shape[1] * W))
    for a in range(0, T, step):
        b = min(T, a + step)
        rows = flat[sel[a:b].long().clamp(0, flat.shape[0] - 1)].float()                 # [t, k, W]
        lat, pe = rows[..., :kv_lora], rows[..., kv_lora:]
        s = (torch.einsum("thc,tkc->thk", q_lat[a:b].float(), lat) + torch.einsum("thr,tkr->thk", q_pe[a:b].float(), pe)) * scale
        dead = torch.arange(sel.shape[1], device=sel.device)[None, :] >= sel_len[a:b, None]
        p = torch.softmax(s.masked_fill(dead[:, None, :], float("-inf")), dim=-1)
        out[a:b] = torch.einsum("thk,tkc->thc", p, lat).to(q_lat.dtype)
    return out


# ----------------------------------------------------------------------------- fp8 with per-row / per-channel scales
def quant_rows_fp8(x: torch.Tensor):
    """One dynamic scale per row: scale = max|x| / 448, q = e4m3(x / scale)."""
    xf = x.float()
    s = xf.abs().amax(-1).clamp_min(1e-10) / 448.0
    q = (xf / s[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, s


def linear_fp8_scaled(xq, xs, wq, col_scale=None, tensor_scale: float = 1.0, bias=None, out_dtype=torch.bfloat16):
    y = (xq.float() @ wq.float().t()) * xs[:, None].float() * tensor_scale
    if col_scale is not None:
        y = y * col_scale.float()[None, :]
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)
