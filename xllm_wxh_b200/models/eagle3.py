"""EAGLE-3 draft model: one decoder layer that reads the target's hidden states of three layers.

Reference: the Eagle3 worker (xllm/core/runtime/eagle3_worker_impl.cpp:44-102: the draft receives an embedding placeholder
of 3 x hidden per token, draft token ids are mapped to target ids through `d2t`) and the draft model definition
(xllm/models/llm/npu/qwen3_eagle3.h: `embed_tokens`, `fc` 3H -> H, one `midlayer`, `norm`, `lm_head` over the draft
vocabulary; the target captures the inputs of layers 2, L/2 and L-3, models/llm/npu/qwen3.h:107-123).

Per token the draft sees the embedding of the NEXT token and a hidden state h: for rows that the target has just run, h is
`fc` of the three captured target states; for rows the draft chains on its own (second and later proposals of a step), h
is the draft's own output of the previous row.  The layer normalises both, runs attention on their concatenation [2H],
adds the result to h, then a SwiGLU MLP.  Checkpoint names are those of the public EAGLE-3 draft checkpoints.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..ops import reference as ref
from ..parallel.comm import Comm
from .args import ModelArgs
from .qwen import WeightInit, _DT


def default_capture_layers(n_layers: int) -> List[int]:
    """Layers whose INPUT the target hands to the draft: low, middle, high (qwen3.h:113-115)."""
    return sorted({min(2, n_layers - 1), n_layers // 2, max(0, n_layers - 3)})


class Eagle3Draft:
    is_mtp = True

    def __init__(self, args: ModelArgs, comm: Optional[Comm] = None, device="cpu", dtype: Optional[torch.dtype] = None,
                 target=None, draft_vocab_size: int = 0, n_captured: int = 0):
        self.args, self.comm = args, comm or Comm()
        self.device = torch.device(device)
        self.dtype = dtype or _DT[args.dtype]
        self.target = target
        self.n_q, self.n_kv, self.head_dim = args.n_heads, args.n_kv_heads, args.head_dim
        self.scale = args.head_dim ** -0.5
        self.n_captured = n_captured or len(default_capture_layers(args.n_layers))
        self.draft_vocab = draft_vocab_size or args.vocab_size
        self.cos_sin = ref.scaled_cos_sin_cache(args, args.head_dim, dtype=torch.float32, device=self.device)
        self.embed = target.embed if target is not None else None
        self.fc = self.hidden_norm = self.input_norm = self.qkv_w = self.o_w = self.q_norm = self.k_norm = None
        self.post_norm = self.gate_up_w = self.down_w = self.norm = self.lm_head = None
        self.d2t = None                      # [draft vocab] int64: target id = draft id + d2t[draft id] (None: identity)

    # ------------------------------------------------------------------ weights
    def kv_cache_shapes(self, num_blocks: int, block_size: int):
        shp = (num_blocks, block_size, self.n_kv, self.head_dim)
        return [(shp, shp)]

    def init_random(self, seed: int = 0, std: float = 0.02):
        a = self.args
        wi = WeightInit(seed, std, self.dtype, self.device)
        H, D, I = a.hidden_size, a.head_dim, a.intermediate_size
        if self.embed is None:
            self.embed = wi.normal("embed_tokens.weight", (a.vocab_size, H))
        self.fc = wi.normal("fc.weight", (H, self.n_captured * H))
        self.hidden_norm, self.input_norm, self.post_norm, self.norm = wi.ones((H,)), wi.ones((H,)), wi.ones((H,)), wi.ones((H,))
        q = wi.normal("midlayer.self_attn.q_proj.weight", (self.n_q * D, 2 * H))
        k = wi.normal("midlayer.self_attn.k_proj.weight", (self.n_kv * D, 2 * H))
        v = wi.normal("midlayer.self_attn.v_proj.weight", (self.n_kv * D, 2 * H))
        self.qkv_w = torch.cat([q, k, v], 0)
        self.o_w = wi.normal("midlayer.self_attn.o_proj.weight", (H, self.n_q * D))
        self.gate_up_w = torch.cat([wi.normal("midlayer.mlp.gate_proj.weight", (I, H)), wi.normal("midlayer.mlp.up_proj.weight", (I, H))], 0)
        self.down_w = wi.normal("midlayer.mlp.down_proj.weight", (H, I))
        self.lm_head = wi.normal("lm_head.weight", (self.draft_vocab, H))
        if self.draft_vocab != a.vocab_size:
            # a deterministic "hot token" table for random-initialised drafts: evenly spread target ids
            hot = torch.linspace(0, a.vocab_size - 1, self.draft_vocab, device=self.device).long()
            self.d2t = hot - torch.arange(self.draft_vocab, device=self.device)
        return self

    def load_weights(self, ckpt) -> "Eagle3Draft":
        dev = lambda t: t.to(self.device, self.dtype).contiguous()
        g = lambda name: ckpt.get(name) if ckpt.has(name) else ckpt.get("model." + name)
        has = lambda name: ckpt.has(name) or ckpt.has("model." + name)
        if has("embed_tokens.weight"):
            self.embed = dev(g("embed_tokens.weight"))
        elif self.embed is None:
            raise ValueError("the EAGLE-3 draft checkpoint has no embed_tokens and no target model shares its own")
        self.fc = dev(g("fc.weight"))
        self.n_captured = self.fc.shape[1] // self.args.hidden_size
        p = "midlayer."
        self.hidden_norm, self.input_norm = dev(g(p + "hidden_norm.weight")), dev(g(p + "input_layernorm.weight"))
        self.post_norm, self.norm = dev(g(p + "post_attention_layernorm.weight")), dev(g("norm.weight"))
        self.qkv_w = dev(torch.cat([g(p + "self_attn.q_proj.weight"), g(p + "self_attn.k_proj.weight"),
                                    g(p + "self_attn.v_proj.weight")], 0))
        self.o_w = dev(g(p + "self_attn.o_proj.weight"))
        if has(p + "self_attn.q_norm.weight"):
            self.q_norm, self.k_norm = dev(g(p + "self_attn.q_norm.weight")), dev(g(p + "self_attn.k_norm.weight"))
        self.gate_up_w = dev(torch.cat([g(p + "mlp.gate_proj.weight"), g(p + "mlp.up_proj.weight")], 0))
        self.down_w = dev(g(p + "mlp.down_proj.weight"))
        self.lm_head = dev(g("lm_head.weight"))
        self.draft_vocab = self.lm_head.shape[0]
        if has("d2t"):
            self.d2t = g("d2t").to(self.device).long()
        D = self.head_dim
        self.n_q = self.o_w.shape[1] // D
        self.n_kv = (self.qkv_w.shape[0] // D - self.n_q) // 2
        return self

    def state_dict(self):
        D, H = self.head_dim, self.args.hidden_size
        q, k, v = self.qkv_w.split([self.n_q * D, self.n_kv * D, self.n_kv * D], 0)
        I = self.gate_up_w.shape[0] // 2
        sd = {"fc.weight": self.fc, "midlayer.hidden_norm.weight": self.hidden_norm, "midlayer.input_layernorm.weight": self.input_norm,
              "midlayer.post_attention_layernorm.weight": self.post_norm, "norm.weight": self.norm,
              "midlayer.self_attn.q_proj.weight": q, "midlayer.self_attn.k_proj.weight": k, "midlayer.self_attn.v_proj.weight": v,
              "midlayer.self_attn.o_proj.weight": self.o_w, "midlayer.mlp.gate_proj.weight": self.gate_up_w[:I],
              "midlayer.mlp.up_proj.weight": self.gate_up_w[I:], "midlayer.mlp.down_proj.weight": self.down_w,
              "lm_head.weight": self.lm_head}
        if self.d2t is not None:
            sd["d2t"] = self.d2t
        return {k_: v_.contiguous() for k_, v_ in sd.items()}

    def finalize_weights(self):
        return self

    # ------------------------------------------------------------------ forward
    def forward_mtp(self, inp, kv_caches, prev_hidden: torch.Tensor) -> torch.Tensor:
        """`inp.tokens`: the tokens that FOLLOW the positions of `prev_hidden`.  `prev_hidden` [T, n_captured * H]: captured
        target states (fused by `fc`), or [T, H]: the draft's own previous output.  Returns the layer output [T, H]
        (before the final norm), which is also what a chained step takes as its `prev_hidden`."""
        a = self.args
        eps = a.rms_norm_eps
        h = prev_hidden.to(self.dtype)
        if h.shape[-1] != a.hidden_size:
            h = ops.linear(h, self.fc)
        e = ops.embedding(inp.tokens, self.embed)
        x = torch.cat([ops.rms_norm(e, self.input_norm, eps), ops.rms_norm(h, self.hidden_norm, eps)], dim=-1)
        kv = kv_caches[0]
        qkv = ops.linear(x, self.qkv_w)
        q = ops.rope_qknorm_kvwrite(qkv, inp.positions, inp.slots, self.cos_sin, self.q_norm, self.k_norm, eps, kv[0], kv[1],
                                    self.n_q, self.n_kv, self.head_dim)
        attn = ops.paged_attention(q.view(-1, self.n_q, self.head_dim), kv[0], kv[1], inp, self.scale, -1)
        y = ops.linear(attn, self.o_w)
        x2, residual = ops.add_rms_norm(y, h, self.post_norm, eps)
        act = ops.silu_and_mul(ops.linear(x2, self.gate_up_w))
        return (ops.linear(act, self.down_w).float() + residual.float()).to(self.dtype)

    def logits(self, hidden: torch.Tensor, sample_idx: Optional[torch.Tensor], gather: bool = True) -> torch.Tensor:
        sel = hidden.index_select(0, sample_idx.long()) if sample_idx is not None else hidden
        return ops.linear(ops.rms_norm(sel, self.norm, self.args.rms_norm_eps), self.lm_head)

    def propose(self, hidden: torch.Tensor, sample_idx: Optional[torch.Tensor]) -> torch.Tensor:
        """Greedy proposal in TARGET token ids (draft id + d2t[draft id], eagle3_worker_impl.cpp:88-100)."""
        ids = self.logits(hidden, sample_idx).argmax(-1)
        if self.d2t is not None:
            ids = ids + self.d2t.index_select(0, ids)
        return ids.int()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.fc, self.qkv_w, self.o_w, self.gate_up_w, self.down_w, self.lm_head)
                   if t is not None)
