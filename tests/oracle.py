"""Independent fp32 restatement of the decoder math used as the token-for-token oracle.

Written against the model definition only (HF-style dense attention over the full sequence, no paging,
no scheduler, no fused ops), so that agreement with the engine checks the engine's paged KV, batching,
chunked prefill and kernels — not a shared code path."""
import math

import torch


def rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope(x, pos, theta):
    # x [T, H, D], neox pairing (i, i + D/2)
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    f = pos.float()[:, None] * inv[None, :]
    c, s = f.cos()[:, None, :], f.sin()[:, None, :]
    a, b = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def forward_full(sd, args, tokens):
    """Logits [T, V] for one sequence of token ids (fp32)."""
    T = len(tokens)
    H, D, nq, nkv = args.hidden_size, args.head_dim, args.n_heads, args.n_kv_heads
    x = sd["model.embed_tokens.weight"].float()[torch.tensor(tokens)]
    pos = torch.arange(T)
    for i in range(args.n_layers):
        p = f"model.layers.{i}."
        h = rms(x, sd[p + "input_layernorm.weight"].float(), args.rms_norm_eps)
        q = h @ sd[p + "self_attn.q_proj.weight"].float().t()
        k = h @ sd[p + "self_attn.k_proj.weight"].float().t()
        v = h @ sd[p + "self_attn.v_proj.weight"].float().t()
        if p + "self_attn.q_proj.bias" in sd:
            q = q + sd[p + "self_attn.q_proj.bias"].float()
            k = k + sd[p + "self_attn.k_proj.bias"].float()
            v = v + sd[p + "self_attn.v_proj.bias"].float()
        q, k, v = q.view(T, nq, D), k.view(T, nkv, D), v.view(T, nkv, D)
        if p + "self_attn.q_norm.weight" in sd:
            q = rms(q, sd[p + "self_attn.q_norm.weight"].float(), args.rms_norm_eps)
            k = rms(k, sd[p + "self_attn.k_norm.weight"].float(), args.rms_norm_eps)
        q, k = rope(q, pos, args.rope_theta), rope(k, pos, args.rope_theta)
        g = nq // nkv
        k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool))[None], float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, nq * D)
        x = x + a @ sd[p + "self_attn.o_proj.weight"].float().t()
        h = rms(x, sd[p + "post_attention_layernorm.weight"].float(), args.rms_norm_eps)
        if p + "mlp.gate.weight" in sd:
            x = x + moe(sd, args, p, h)
        else:
            gate = h @ sd[p + "mlp.gate_proj.weight"].float().t()
            up = h @ sd[p + "mlp.up_proj.weight"].float().t()
            x = x + (torch.nn.functional.silu(gate) * up) @ sd[p + "mlp.down_proj.weight"].float().t()
    x = rms(x, sd["model.norm.weight"].float(), args.rms_norm_eps)
    head = sd.get("lm_head.weight", sd["model.embed_tokens.weight"]).float()
    return x @ head.t()


def moe(sd, args, p, h):
    logits = h @ sd[p + "mlp.gate.weight"].float().t()
    probs = torch.softmax(logits, -1)
    w, idx = probs.topk(args.num_experts_per_tok, -1)
    if args.norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            g = h[t] @ sd[p + f"mlp.experts.{e}.gate_proj.weight"].float().t()
            u = h[t] @ sd[p + f"mlp.experts.{e}.up_proj.weight"].float().t()
            out[t] += w[t, j] * ((torch.nn.functional.silu(g) * u) @ sd[p + f"mlp.experts.{e}.down_proj.weight"].float().t())
    return out


def greedy_generate(sd, args, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward_full(sd, args, toks)[-1].argmax()))
    return toks[len(prompt):]


# ----------------------------------------------------------------------------- DeepSeek (MLA + MoE), non-absorbed form
def _rope_interleaved(x, pos, inv_freq, mscale):
    f = pos.float()[:, None] * inv_freq[None, :]
    c, s = (f.cos() * mscale)[:, None, :], (f.sin() * mscale)[:, None, :]
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)


def deepseek_forward_full(sd, args, tokens, inv_freq, mscale, softmax_scale, n_layers=None):
    """Logits [T, V] with MLA written the plain way: expand k_nope / v from the normalised latent through kv_b_proj,
    score over the 192-wide q/k, softmax, weighted sum of v."""
    T = len(tokens)
    H, nh = args.hidden_size, args.n_heads
    nope, rope, vd, c = args.qk_nope_head_dim, args.qk_rope_head_dim, args.v_head_dim, args.kv_lora_rank
    x = sd["model.embed_tokens.weight"].float()[torch.tensor(tokens)]
    pos = torch.arange(T)
    for i in range(n_layers or args.n_layers):
        p = f"model.layers.{i}."
        x = x + _ds_attention(sd, args, p, rms(x, sd[p + "input_layernorm.weight"].float(), args.rms_norm_eps), pos, inv_freq,
                              mscale, softmax_scale)
        h = rms(x, sd[p + "post_attention_layernorm.weight"].float(), args.rms_norm_eps)
        x = x + _ds_mlp(sd, args, p, h)
    x = rms(x, sd["model.norm.weight"].float(), args.rms_norm_eps)
    return x @ sd["lm_head.weight"].float().t(), x


def _rope_halves(x, pos, inv_freq, mscale):
    f = pos.float()[:, None] * inv_freq[None, :]
    c, s = (f.cos() * mscale)[:, None, :], (f.sin() * mscale)[:, None, :]
    d2 = x.shape[-1] // 2
    a, b = x[..., :d2], x[..., d2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def _ds_index_keep(sd, args, p, h, qa, pos, inv_freq, mscale):
    """DeepSeek-V3.2 lightning indexer, the plain way over a whole sequence: keep[t, s] is True where key s is among the
    `index_topk` causal keys with the highest score sum_h w[t, h] relu(q[t, h] . k[s])."""
    import scipy.linalg
    T = h.shape[0]
    nh, d, r = args.index_n_heads, args.index_head_dim, args.qk_rope_head_dim
    ip = p + "self_attn.indexer."
    rope = _rope_interleaved if args.index_rope_interleave else _rope_halves
    had = torch.tensor(scipy.linalg.hadamard(d), dtype=torch.float32) / d ** 0.5
    q = (qa @ sd[ip + "wq_b.weight"].float().t()).view(T, nh, d)
    q = torch.cat([rope(q[..., :r], pos, inv_freq, mscale), q[..., r:]], -1) @ had
    k = torch.nn.functional.layer_norm(h @ sd[ip + "wk.weight"].float().t(), (d,), sd[ip + "k_norm.weight"].float(),
                                       sd[ip + "k_norm.bias"].float(), 1e-6)
    k = torch.cat([rope(k[:, None, :r], pos, inv_freq, mscale)[:, 0], k[:, r:]], -1) @ had
    w = h @ sd[ip + "weights_proj.weight"].float().t()
    score = (torch.relu(torch.einsum("thd,sd->ths", q, k)) * w[:, :, None]).sum(1) * d ** -0.5 * nh ** -0.5
    keep = torch.zeros(T, T, dtype=torch.bool)
    for t in range(T):
        best = score[t, :t + 1].topk(min(args.index_topk, t + 1)).indices
        keep[t, best] = True
    return keep


def _ds_attention(sd, args, p, h, pos, inv_freq, mscale, softmax_scale):
    T = h.shape[0]
    nh, nope, rope, vd, c = args.n_heads, args.qk_nope_head_dim, args.qk_rope_head_dim, args.v_head_dim, args.kv_lora_rank
    keep = None
    if p + "self_attn.q_a_proj.weight" in sd:
        qa = rms(h @ sd[p + "self_attn.q_a_proj.weight"].float().t(), sd[p + "self_attn.q_a_layernorm.weight"].float(), args.rms_norm_eps)
        q = qa @ sd[p + "self_attn.q_b_proj.weight"].float().t()
        if p + "self_attn.indexer.wk.weight" in sd and args.index_topk > 0:
            keep = _ds_index_keep(sd, args, p, h, qa, pos, inv_freq, mscale)
    else:
        q = h @ sd[p + "self_attn.q_proj.weight"].float().t()
    q = q.view(T, nh, nope + rope)
    kva = h @ sd[p + "self_attn.kv_a_proj_with_mqa.weight"].float().t()
    lat = rms(kva[:, :c], sd[p + "self_attn.kv_a_layernorm.weight"].float(), args.rms_norm_eps)
    k_pe = _rope_interleaved(kva[:, None, c:], pos, inv_freq, mscale)            # [T, 1, rope]
    q_pe = _rope_interleaved(q[..., nope:], pos, inv_freq, mscale)
    kv = (lat @ sd[p + "self_attn.kv_b_proj.weight"].float().t()).view(T, nh, nope + vd)
    k = torch.cat([kv[..., :nope], k_pe.expand(T, nh, rope)], -1)
    qq = torch.cat([q[..., :nope], q_pe], -1)
    s = torch.einsum("qhd,khd->hqk", qq, k) * softmax_scale
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool))[None], float("-inf"))
    if keep is not None:
        s = s.masked_fill(~keep[None], float("-inf"))
    a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), kv[..., nope:]).reshape(T, nh * vd)
    return a @ sd[p + "self_attn.o_proj.weight"].float().t()


def _ds_mlp(sd, args, p, h):
    silu = torch.nn.functional.silu
    if p + "mlp.gate.weight" not in sd:
        return (silu(h @ sd[p + "mlp.gate_proj.weight"].float().t()) * (h @ sd[p + "mlp.up_proj.weight"].float().t())) @ \
            sd[p + "mlp.down_proj.weight"].float().t()
    scores = torch.sigmoid(h @ sd[p + "mlp.gate.weight"].float().t())
    bias = sd.get(p + "mlp.gate.e_score_correction_bias")
    sel = scores + (bias.float() if bias is not None else 0)
    T, E = scores.shape
    g = sel.view(T, args.n_group, E // args.n_group)
    gs = g.topk(2, -1).values.sum(-1)
    keep = gs.topk(args.topk_group, -1).indices
    mask = torch.zeros(T, args.n_group, dtype=torch.bool).scatter_(1, keep, True)
    sel = sel.masked_fill(~mask[:, :, None].expand(T, args.n_group, E // args.n_group).reshape(T, E), float("-inf"))
    idx = sel.topk(args.num_experts_per_tok, -1).indices
    w = scores.gather(-1, idx)
    w = w / w.sum(-1, keepdim=True) * args.routed_scaling_factor
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            gg = h[t] @ sd[p + f"mlp.experts.{e}.gate_proj.weight"].float().t()
            uu = h[t] @ sd[p + f"mlp.experts.{e}.up_proj.weight"].float().t()
            out[t] += w[t, j] * ((silu(gg) * uu) @ sd[p + f"mlp.experts.{e}.down_proj.weight"].float().t())
    if p + "mlp.shared_experts.gate_proj.weight" in sd:
        out = out + (silu(h @ sd[p + "mlp.shared_experts.gate_proj.weight"].float().t()) *
                     (h @ sd[p + "mlp.shared_experts.up_proj.weight"].float().t())) @ sd[p + "mlp.shared_experts.down_proj.weight"].float().t()
    return out


def deepseek_greedy(sd, args, prompt, n_new, inv_freq, mscale, softmax_scale):
    toks = list(prompt)
    for _ in range(n_new):
        lg, _ = deepseek_forward_full(sd, args, toks, inv_freq, mscale, softmax_scale)
        toks.append(int(lg[-1].argmax()))
    return toks[len(prompt):]
