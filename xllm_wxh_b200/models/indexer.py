"""Lightning indexer of DeepSeek-V3.2 (sparse MLA): for every query token it ranks the keys of its sequence with a cheap
score and keeps the `index_topk` best; the MLA attention then reads only those cache rows.

    q_idx[t, h, :] = hadamard(rope_front(W_qb q_latent[t]))                    h < index_n_heads, 128 wide
    k_idx[s, :]    = hadamard(rope_front(layer_norm(W_k x[s])))                one 128-wide key per token, cached per slot
    score[t, s]    = sum_h w[t, h] * relu(q_idx[t, h] . k_idx[s]) * d^-1/2 * n_heads^-1/2,     w = W_w x[t]
    keep[t]        = top-k over the causal keys s <= pos[t]

What the reference does in its MLU layer (xllm/core/layers/mlu/indexer.cpp:102-160 weights, 267-318 q / k preprocessing,
536-566 selection; deepseek_v2_attention.cpp:356-403: the attention runs with the indexer's per-token block table of
single-slot blocks and per-token context lengths).  Here the result has the same form - `sel [T, k]` cache slot ids and
`sel_len [T]` - and `ops.mla_attention_sparse` reads it as a block table with blocks of one slot.

The selection is written with tensor operations only (no host read of a length), so that it can sit inside a captured
step: shapes depend on the number of tokens and on the block-table width, never on the lengths themselves.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional, Tuple

import torch

from .. import ops
from ..ops import reference as ref

_HADAMARD: Dict[Tuple[int, str, torch.dtype], torch.Tensor] = {}


def hadamard_matrix(n: int, device, dtype) -> torch.Tensor:
    """Sylvester Hadamard matrix of order n (a power of two), scaled by n^-1/2 (orthonormal)."""
    key = (n, str(device), dtype)
    h = _HADAMARD.get(key)
    if h is None:
        assert n & (n - 1) == 0, "Hadamard order must be a power of two"
        h = torch.ones(1, 1, dtype=torch.float32)
        while h.shape[0] < n:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
        h = (h / math.sqrt(n)).to(device=device, dtype=dtype)
        _HADAMARD[key] = h
    return h


def _rotate(x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """x [..., d] times the Hadamard matrix; d that is no power of two is zero-padded and cut back."""
    d, n = x.shape[-1], h.shape[0]
    x2 = x.reshape(-1, d)
    if d != n:
        x2 = torch.nn.functional.pad(x2, (0, n - d))
    return ops.linear(x2.contiguous(), h)[:, :d].reshape(x.shape)


class LightningIndexer:
    """Weights of one layer's indexer (replicated on every tensor-parallel rank, as in the reference) and its two steps:
    `write_keys` (one key per token into the index cache), `queries` (per-head queries and head weights) and `select`
    (scores, causal top-k)."""

    def __init__(self, args, device, dtype):
        self.n_heads, self.dim, self.rope = args.index_n_heads, args.index_head_dim, args.qk_rope_head_dim
        self.topk = args.index_topk
        self.interleave = bool(args.index_rope_interleave)
        self.scale = self.dim ** -0.5 * self.n_heads ** -0.5
        self.eps = 1e-6
        self.device, self.dtype = torch.device(device), dtype
        self.wq_b = self.wk = self.weights_proj = self.k_norm_w = self.k_norm_b = None

    # ------------------------------------------------------------------ weights
    NAMES = ("wq_b.weight", "wk.weight", "weights_proj.weight", "k_norm.weight", "k_norm.bias")

    def init_random(self, wi, prefix: str, q_in: int, hidden: int):
        self.wq_b = wi.normal(prefix + "wq_b.weight", (self.n_heads * self.dim, q_in))
        self.wk = wi.normal(prefix + "wk.weight", (self.dim, hidden))
        self.weights_proj = wi.normal(prefix + "weights_proj.weight", (self.n_heads, hidden))
        self.k_norm_w = wi.ones((self.dim,))
        self.k_norm_b = wi.normal(prefix + "k_norm.bias", (self.dim,))
        return self

    def load(self, ckpt, prefix: str, get_dense):
        """`get_dense(name)` returns the tensor in the model dtype on the device (fp8 block-scaled tensors dequantised)."""
        self.wq_b, self.wk = get_dense(prefix + "wq_b.weight"), get_dense(prefix + "wk.weight")
        self.weights_proj = get_dense(prefix + "weights_proj.weight")
        self.k_norm_w, self.k_norm_b = get_dense(prefix + "k_norm.weight"), get_dense(prefix + "k_norm.bias")
        return self

    def state(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {prefix + "wq_b.weight": self.wq_b, prefix + "wk.weight": self.wk, prefix + "weights_proj.weight": self.weights_proj,
                prefix + "k_norm.weight": self.k_norm_w, prefix + "k_norm.bias": self.k_norm_b}

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.wq_b, self.wk, self.weights_proj, self.k_norm_w, self.k_norm_b))

    # ------------------------------------------------------------------ step 1: projections + cache write
    def _rope_front(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """RoPE on the first `rope` features of x [T, H, d] (the indexer keeps its rotary part in front)."""
        fn = ref.apply_rope_interleaved if self.interleave else ref.apply_rope_neox
        return torch.cat([fn(x[..., :self.rope], cos, sin), x[..., self.rope:]], -1)

    def _cos_sin(self, positions: torch.Tensor, cos_sin: torch.Tensor):
        cs = cos_sin.index_select(0, positions.long().clamp(min=0))
        return cs[:, :self.rope // 2], cs[:, self.rope // 2:]

    def write_keys(self, x: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, cos_sin: torch.Tensor,
                   idx_cache: torch.Tensor) -> None:
        """x [T, hidden] (the attention's input): one index key per token into `idx_cache` [blocks, block, d] at `slots`.
        Runs on every step, also while the sequences are short, because later steps rank these keys."""
        had = hadamard_matrix(1 << (self.dim - 1).bit_length(), x.device, x.dtype)
        cos, sin = self._cos_sin(positions, cos_sin)
        k = ops.linear(x, self.wk).float()
        k = torch.nn.functional.layer_norm(k, (self.dim,), self.k_norm_w.float(), self.k_norm_b.float(), self.eps).to(x.dtype)
        k = _rotate(self._rope_front(k[:, None, :], cos, sin)[:, 0], had)
        flat = idx_cache.view(-1, self.dim)
        # padded rows of a captured step point into the reserved block 0, so a plain scatter is enough
        flat.index_copy_(0, slots.long().clamp(0, flat.shape[0] - 1), k.to(flat.dtype))

    def queries(self, x: torch.Tensor, q_in: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """q_in [T, q_lora] (the normalised query latent) -> (q_idx [T, n_heads, d], head weights w [T, n_heads])."""
        T = x.shape[0]
        had = hadamard_matrix(1 << (self.dim - 1).bit_length(), x.device, x.dtype)
        cos, sin = self._cos_sin(positions, cos_sin)
        q = ops.linear(q_in, self.wq_b).view(T, self.n_heads, self.dim)
        q = _rotate(self._rope_front(q, cos, sin), had)
        return q, ops.linear(x, self.weights_proj)

    # ------------------------------------------------------------------ step 2: scores + causal top-k
    def select(self, q: torch.Tensor, w: torch.Tensor, idx_cache: torch.Tensor, inp, chunk_elems: int = 1 << 20
               ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns (sel [T, k] int32 cache slots, best first, sel_len [T] int32 = min(pos + 1, k)), k = min(index_topk,
        keys the block tables of this step can name).  Entries of a row beyond its `sel_len` are not meaningful."""
        T = q.shape[0]
        bs = idx_cache.shape[1]
        flat = idx_cache.view(-1, self.dim)
        n_slots = flat.shape[0]
        bt = inp.block_tables
        S = bt.shape[1] * bs if inp.padded else min(bt.shape[1], (max(1, inp.max_kv) + bs - 1) // bs) * bs
        nb = S // bs
        k_eff = min(self.topk, S)
        pos = inp.positions[:T].long()
        seq = inp.token_seq[:T].long().clamp(0, bt.shape[0] - 1)
        off = torch.arange(bs, device=q.device)
        kpos = torch.arange(S, device=q.device)
        sel = torch.empty((T, k_eff), dtype=torch.int32, device=q.device)
        wf = w.float() * self.scale

        def ranked(score, slots, p):            # score [t, S], slots [S] or [t, S], p [t]
            score = score.masked_fill(kpos[None, :] > p[:, None], float("-inf"))
            top = score.topk(k_eff, dim=-1).indices
            return (slots[top] if slots.dim() == 1 else slots.gather(1, top)).to(torch.int32)

        if q.is_cuda and os.environ.get("XLLM_INDEX_SCORES_KERNEL", "1") != "0":
            # one kernel for the scores (ops/cuda_ops.py::index_scores); the top-k and the slot lookup stay tensor
            # operations.  Tokens in groups that keep the score matrix below 128 MB.
            from ..ops import cuda_ops
            tseq, tpos = inp.token_seq[:T], inp.positions[:T]
            step = max(1, (1 << 25) // S)
            served = True
            for a in range(0, T, step):
                b = min(T, a + step)
                score = cuda_ops.index_scores(q[a:b], wf[a:b], idx_cache, bt, tseq[a:b], tpos[a:b], S)
                if score is None:                       # a shape the kernel does not serve: the tensor path below
                    served = False
                    break
                top = score.topk(k_eff, dim=-1).indices
                blocks = bt.index_select(0, seq[a:b])[:, :nb].long().gather(1, top // bs)
                sel[a:b] = (blocks * bs + top % bs).clamp_(0, n_slots - 1).to(torch.int32)
            if served:
                return sel, (pos + 1).clamp(1, k_eff).to(torch.int32)
        if not inp.padded and inp.n_seqs == 1:
            # one sequence (a prefill chunk): its keys are gathered once and shared by every query token
            slots = ((bt[0, :nb].long()[:, None] * bs + off[None, :]).reshape(S)).clamp_(0, n_slots - 1)
            keys = flat.index_select(0, slots)                                            # [S, d]
            step = max(1, chunk_elems * 32 // (S * self.n_heads))
            for a in range(0, T, step):
                b = min(T, a + step)
                logit = torch.einsum("thd,sd->ths", q[a:b], keys)
                score = (torch.relu(logit).float() * wf[a:b, :, None]).sum(1)
                sel[a:b] = ranked(score, slots, pos[a:b])
        else:
            step = max(1, chunk_elems // S)
            for a in range(0, T, step):
                b = min(T, a + step)
                slots = (bt[seq[a:b], :nb].long()[:, :, None] * bs + off[None, None, :]).reshape(b - a, S).clamp_(0, n_slots - 1)
                keys = flat[slots]                                                        # [t, S, d]
                logit = torch.einsum("thd,tsd->ths", q[a:b], keys)
                score = (torch.relu(logit).float() * wf[a:b, :, None]).sum(1)
                sel[a:b] = ranked(score, slots, pos[a:b])
        sel_len = (pos + 1).clamp(1, k_eff).to(torch.int32)
        return sel, sel_len

    def wanted(self, inp, block_size: int) -> bool:
        """Whether this step needs the selection at all: a sequence of at most `index_topk` keys keeps every key.  A
        captured step decides by what its block tables can name, since its lengths change from replay to replay."""
        if inp.padded:
            return inp.block_tables.shape[1] * block_size > self.topk
        return inp.max_kv > self.topk
