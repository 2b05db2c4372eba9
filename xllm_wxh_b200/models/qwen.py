"""Qwen2 / Qwen3 dense and Qwen3-MoE decoders.

Structure follows the reference's model definitions (xllm/models/llm/llm_model_base.h:38-259,
qwen2.h:30-123, qwen3.h:30-283, qwen3_moe.h:30-279; layers/common/qwen2_attention.cpp:42-193,
dense_mlp.cpp:26-107, layers/qwen3_moe_decoder_layer.cpp:34-155): embedding, N pre-norm decoder
layers carrying (x, residual), final RMSNorm, `logits(hidden[selected])` through lm_head (tied to the
embedding when the config says so).  Weights use the HF names of those architectures.

Each decoder layer is expressed around the row-parallel step "GEMM -> all-reduce -> +residual ->
RMSNorm" (`Comm.row_linear_add_rms_norm`), so that the tensor-parallel build can replace that whole
chain by one fused kernel pair.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..ops import reference as ref
from ..parallel.comm import Comm
from .args import ModelArgs
from .registry import register_model

_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _randn(shape, std, gen, dtype, device):
    # generated in fp32 on the target device, chunked along dim 0 to bound the transient
    out = torch.empty(shape, dtype=dtype, device=device)
    rows = shape[0]
    per = max(1, (64 << 20) // max(1, math.prod(shape[1:])))
    for s in range(0, rows, per):
        e = min(rows, s + per)
        out[s:e] = (torch.randn((e - s,) + tuple(shape[1:]), generator=gen, device=device, dtype=torch.float32) * std).to(dtype)
    return out


class WeightInit:
    """Deterministic N(0, std) initialisation: each named parameter draws from its own stream, so a
    tensor-parallel shard holds exactly the rows/columns of the single-GPU tensor."""

    def __init__(self, seed: int, std: float, dtype: torch.dtype, device):
        self.seed, self.std, self.dtype, self.device = seed, std, dtype, torch.device(device)

    def normal(self, name: str, shape, rows: Optional[Tuple[int, int]] = None, cols: Optional[Tuple[int, int]] = None,
               dtype=None) -> torch.Tensor:
        import zlib
        gen = torch.Generator(device=self.device)
        gen.manual_seed((self.seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFF)
        full = _randn(tuple(shape), self.std, gen, dtype or self.dtype, self.device)
        if rows is not None:
            full = full[rows[0]:rows[1]]
        if cols is not None:
            full = full[:, cols[0]:cols[1]]
        return full.contiguous()

    def ones(self, shape) -> torch.Tensor:
        return torch.ones(shape, dtype=self.dtype, device=self.device)


def shard_range(total: int, rank: int, size: int) -> Tuple[int, int]:
    per = total // size
    return rank * per, (rank + 1) * per


class AttentionWeights:
    def __init__(self):
        self.qkv_w = self.qkv_b = self.o_w = self.q_norm = self.k_norm = None
        self.qkv_s = self.o_s = None            # fp8 weights: fp32 scale of every output channel [N] (None: bf16 weight)


class MlpWeights:
    def __init__(self):
        self.gate_up_w = self.down_w = None     # dense: this rank's shard, or the whole MLP when it is replicated
        self.gate_up_tp = self.down_tp = None   # replicated MLP: this rank's slice of the same tensors (views)
        self.gate_up_s = self.down_s = None     # fp8 weights: fp32 scale of every output channel
        self.router_w = None                    # MoE: [E, H]
        self.w13 = self.w2 = None               # MoE: [E_local, 2I, H], [E_local, H, I]
        self.is_moe = False
        self.interleaved = False                # gate/up rows re-ordered for the fused SwiGLU GEMM epilogue


class LayerWeights:
    def __init__(self):
        self.input_norm = self.post_norm = None
        self.attn = AttentionWeights()
        self.mlp = MlpWeights()


@register_model("qwen2", "qwen3", "qwen3_moe", "llama", "mistral")
class QwenForCausalLM:
    def __init__(self, args: ModelArgs, comm: Optional[Comm] = None, device="cpu", dtype: Optional[torch.dtype] = None):
        self.args = args
        self.comm = comm or Comm()
        self.device = torch.device(device)
        self.dtype = dtype or _DT[args.dtype]
        tp = self.comm.tp_size
        self.n_q = args.n_heads // tp
        # kv heads are replicated when there are fewer of them than TP ranks (qwen2_attention.cpp:57-65)
        self.n_kv = max(1, args.n_kv_heads // tp)
        self.head_dim = args.head_dim
        self.scale = args.head_dim ** -0.5
        self.layers: List[LayerWeights] = [LayerWeights() for _ in range(args.n_layers)]
        self.embed = self.final_norm = self.lm_head = None
        self.cos_sin = ref.scaled_cos_sin_cache(args, args.head_dim, dtype=torch.float32, device=self.device)
        self.expert_load = None      # [n_moe_layers, E] int64 histogram, filled when EPLB statistics are on
        self.moe_impl = None         # set by the engine for expert-parallel execution
        self.eplb = None             # EplbExecutor when expert-parallel load balancing is on (runtime/eplb.py)
        self.router_logit_bias = None  # [E] fp32 added to every layer's router logits (skewed-load experiments; None: off)
        self.layer_hook = None       # callable(layer index), run right after a layer's attention (its KV is written by then)
        self.capture_layers = None   # layers whose input an EAGLE-3 draft reads; `forward` leaves them in `aux_hidden`
        self.aux_hidden = None       # [T, len(capture_layers) * H] of the last forward

    # ------------------------------------------------------------------ weights
    def kv_cache_shapes(self, num_blocks: int, block_size: int):
        shp = (num_blocks, block_size, self.n_kv, self.head_dim)
        return [(shp, shp) for _ in range(self.args.n_layers)]

    def _kv_head_range(self) -> Tuple[int, int]:
        a, tp, r = self.args, self.comm.tp_size, self.comm.tp_rank
        if a.n_kv_heads >= tp:
            return shard_range(a.n_kv_heads, r, tp)
        h = r * a.n_kv_heads // tp
        return h, h + 1

    def init_random(self, seed: int = 0, std: float = 0.02):
        a, c = self.args, self.comm
        wi = WeightInit(seed, std, self.dtype, self.device)
        D, H = a.head_dim, a.hidden_size
        tp, r = c.tp_size, c.tp_rank
        self.embed = wi.normal("model.embed_tokens.weight", (a.vocab_size, H))
        self.final_norm = wi.ones((H,))
        if a.tie_word_embeddings:
            full_head = self.embed
            self.lm_head = full_head if tp == 1 else full_head[slice(*shard_range(a.vocab_size, r, tp))].contiguous()
        else:
            self.lm_head = wi.normal("lm_head.weight", (a.vocab_size, H), rows=shard_range(a.vocab_size, r, tp))
        q0, q1 = shard_range(a.n_heads, r, tp)
        k0, k1 = self._kv_head_range()
        for i, L in enumerate(self.layers):
            p = f"model.layers.{i}."
            L.input_norm, L.post_norm = wi.ones((H,)), wi.ones((H,))
            L.mlp.interleaved = False
            qw = wi.normal(p + "self_attn.q_proj.weight", (a.n_heads * D, H), rows=(q0 * D, q1 * D))
            kw = wi.normal(p + "self_attn.k_proj.weight", (a.n_kv_heads * D, H), rows=(k0 * D, k1 * D))
            vw = wi.normal(p + "self_attn.v_proj.weight", (a.n_kv_heads * D, H), rows=(k0 * D, k1 * D))
            L.attn.qkv_w = torch.cat([qw, kw, vw], 0)
            if a.attention_bias:
                qb = wi.normal(p + "self_attn.q_proj.bias", (a.n_heads * D,), rows=(q0 * D, q1 * D))
                kb = wi.normal(p + "self_attn.k_proj.bias", (a.n_kv_heads * D,), rows=(k0 * D, k1 * D))
                vb = wi.normal(p + "self_attn.v_proj.bias", (a.n_kv_heads * D,), rows=(k0 * D, k1 * D))
                L.attn.qkv_b = torch.cat([qb, kb, vb], 0)
            L.attn.o_w = wi.normal(p + "self_attn.o_proj.weight", (H, a.n_heads * D), cols=(q0 * D, q1 * D))
            if a.qk_norm:
                L.attn.q_norm, L.attn.k_norm = wi.ones((D,)), wi.ones((D,))
            if a.is_moe_layer(i):
                self._init_moe_random(L, wi, p)
            else:
                I = a.intermediate_size
                i0, i1 = (0, I) if c.cfg.mlp_replicated else shard_range(I, r, tp)
                g = wi.normal(p + "mlp.gate_proj.weight", (I, H), rows=(i0, i1))
                u = wi.normal(p + "mlp.up_proj.weight", (I, H), rows=(i0, i1))
                L.mlp.gate_up_w = torch.cat([g, u], 0)
                L.mlp.down_w = wi.normal(p + "mlp.down_proj.weight", (H, I), cols=(i0, i1))
        return self

    def _local_experts(self) -> Tuple[int, int]:
        return shard_range(self.args.n_routed_experts, *self.comm.cfg.expert_shard())

    def _init_moe_random(self, L: LayerWeights, wi: WeightInit, p: str):
        a = self.args
        H, I = a.hidden_size, a.moe_intermediate_size
        L.mlp.is_moe = True
        L.mlp.router_w = wi.normal(p + "mlp.gate.weight", (a.n_routed_experts, H))
        e0, e1 = self._local_experts()
        w13, w2 = [], []
        for e in range(e0, e1):
            g = wi.normal(p + f"mlp.experts.{e}.gate_proj.weight", (I, H))
            u = wi.normal(p + f"mlp.experts.{e}.up_proj.weight", (I, H))
            w13.append(torch.cat([g, u], 0))
            w2.append(wi.normal(p + f"mlp.experts.{e}.down_proj.weight", (H, I)))
        L.mlp.w13, L.mlp.w2 = torch.stack(w13), torch.stack(w2)

    def load_weights(self, ckpt) -> "QwenForCausalLM":
        """`ckpt` is a CheckpointReader over HF safetensors with the standard Qwen names.  Linear weights stored as fp8
        e4m3 with a per-tensor or per-output-channel `weight_scale` (the reference's w8a8 fp8 mode,
        layers/common/linear.cpp:65-99,134-179) stay fp8 on a CUDA device and run through the fp8 GEMM with per-token
        activation scales; fused shards (q / k / v, gate / up) keep their own scales as per-channel vectors, so nothing is
        re-quantised.  Block-scaled fp8 weights (`weight_scale_inv`) and fp8 on the CPU are dequantised to the model dtype."""
        from ..utils.safetensors_io import DequantizingReader
        raw = ckpt
        ckpt = DequantizingReader(ckpt)
        a, c = self.args, self.comm
        D, H = a.head_dim, a.hidden_size
        tp, r = c.tp_size, c.tp_rank
        dev = lambda t: t.to(self.device, self.dtype).contiguous()
        import os
        keep_fp8 = (self.device.type == "cuda" and self.dtype == torch.bfloat16 and not a.n_routed_experts and
                    os.environ.get("XLLM_FP8_LINEAR", "1") != "0")

        def lin(name, rows=None, cols=None):
            """(weight, per-channel scale or None) of HF tensor `name`, cut to rows [r0, r1) / columns [c0, c1)."""
            t = raw.get(name)
            if (keep_fp8 and t.dtype == torch.float8_e4m3fn and raw.has(name[:-len("weight")] + "weight_scale")
                    and t.shape[1] % 16 == 0):
                sc = raw.get(name[:-len("weight")] + "weight_scale").float().reshape(-1)
                if sc.numel() not in (1, t.shape[0]):
                    raise ValueError(f"{name}: weight_scale of {sc.numel()} values is neither per tensor nor per channel")
                sc = sc.expand(t.shape[0]) if sc.numel() == 1 else sc
                if rows is not None:
                    t, sc = t[rows[0]:rows[1]], sc[rows[0]:rows[1]]
                if cols is not None:
                    t = t[:, cols[0]:cols[1]]
                return t.contiguous().to(self.device), sc.contiguous().to(self.device)
            w = ckpt.get(name)
            if rows is not None:
                w = w[rows[0]:rows[1]]
            if cols is not None:
                w = w[:, cols[0]:cols[1]]
            return dev(w), None

        def fuse(parts):
            """Row-wise concatenation of (weight, scale) pairs; a bf16 part next to fp8 parts is not expected."""
            ws, ss = [p[0] for p in parts], [p[1] for p in parts]
            if all(x is None for x in ss):
                return torch.cat(ws, 0), None
            if any(x is None for x in ss):          # shards quantised in different ways: the fused weight is unquantised
                ws = [w if sc is None else (w.float() * sc[:, None]).to(self.dtype) for w, sc in zip(ws, ss)]
                return torch.cat(ws, 0), None
            return torch.cat(ws, 0), torch.cat(ss, 0)
        self.embed = dev(ckpt.get("model.embed_tokens.weight"))
        self.final_norm = dev(ckpt.get("model.norm.weight"))
        v0, v1 = shard_range(a.vocab_size, r, tp)
        if a.tie_word_embeddings or not ckpt.has("lm_head.weight"):
            self.lm_head = self.embed if tp == 1 else self.embed[v0:v1].contiguous()
        else:
            self.lm_head = dev(ckpt.get("lm_head.weight")[v0:v1])
        q0, q1 = shard_range(a.n_heads, r, tp)
        k0, k1 = self._kv_head_range()
        for i, L in enumerate(self.layers):
            p = f"model.layers.{i}."
            L.input_norm = dev(ckpt.get(p + "input_layernorm.weight"))
            L.post_norm = dev(ckpt.get(p + "post_attention_layernorm.weight"))
            L.attn.qkv_w, L.attn.qkv_s = fuse([lin(p + "self_attn.q_proj.weight", rows=(q0 * D, q1 * D)),
                                               lin(p + "self_attn.k_proj.weight", rows=(k0 * D, k1 * D)),
                                               lin(p + "self_attn.v_proj.weight", rows=(k0 * D, k1 * D))])
            if ckpt.has(p + "self_attn.q_proj.bias"):
                qb = ckpt.get(p + "self_attn.q_proj.bias")[q0 * D:q1 * D]
                kb = ckpt.get(p + "self_attn.k_proj.bias")[k0 * D:k1 * D]
                vb = ckpt.get(p + "self_attn.v_proj.bias")[k0 * D:k1 * D]
                L.attn.qkv_b = dev(torch.cat([qb, kb, vb], 0))
            L.attn.o_w, L.attn.o_s = lin(p + "self_attn.o_proj.weight", cols=(q0 * D, q1 * D))
            if a.qk_norm:
                L.attn.q_norm = dev(ckpt.get(p + "self_attn.q_norm.weight"))
                L.attn.k_norm = dev(ckpt.get(p + "self_attn.k_norm.weight"))
            if a.is_moe_layer(i):
                L.mlp.is_moe = True
                L.mlp.router_w = dev(ckpt.get(p + "mlp.gate.weight"))
                e0, e1 = self._local_experts()
                w13 = [torch.cat([ckpt.get(p + f"mlp.experts.{e}.gate_proj.weight"),
                                  ckpt.get(p + f"mlp.experts.{e}.up_proj.weight")], 0) for e in range(e0, e1)]
                w2 = [ckpt.get(p + f"mlp.experts.{e}.down_proj.weight") for e in range(e0, e1)]
                L.mlp.w13, L.mlp.w2 = dev(torch.stack(w13)), dev(torch.stack(w2))
            else:
                I = a.intermediate_size
                i0, i1 = (0, I) if c.cfg.mlp_replicated else shard_range(I, r, tp)
                L.mlp.gate_up_w, L.mlp.gate_up_s = fuse([lin(p + "mlp.gate_proj.weight", rows=(i0, i1)),
                                                         lin(p + "mlp.up_proj.weight", rows=(i0, i1))])
                L.mlp.down_w, L.mlp.down_s = lin(p + "mlp.down_proj.weight", cols=(i0, i1))
        return self

    def finalize_weights(self) -> "QwenForCausalLM":
        """Device-specific weight layout, applied once after loading: on CUDA the gate/up rows of every MLP are
        interleaved in groups of 16 so that the GEMM epilogue can apply SwiGLU on the accumulator tile."""
        self.fp8_linears = any(L.attn.qkv_s is not None for L in self.layers)
        if self.device.type != "cuda" or self.dtype != torch.bfloat16:
            return self
        from ..ops import cuda_ops, moe_cuda
        for L in self.layers:
            if L.mlp.interleaved:
                continue
            if L.mlp.is_moe:
                if (L.mlp.w13.shape[1] // 2) % 16 == 0:
                    moe_cuda.interleave_w13(L.mlp.w13)
                    L.mlp.interleaved = True
            elif L.mlp.gate_up_w is not None and (L.mlp.gate_up_w.shape[0] // 2) % 16 == 0:
                if L.mlp.gate_up_s is not None:     # fp8: the same row permutation for the bytes and for their scales
                    L.mlp.gate_up_w = cuda_ops.interleave_gate_up(L.mlp.gate_up_w.view(torch.uint8)).view(torch.float8_e4m3fn)
                    L.mlp.gate_up_s = cuda_ops.interleave_gate_up(L.mlp.gate_up_s.view(-1, 1)).view(-1).contiguous()
                else:
                    L.mlp.gate_up_w = cuda_ops.interleave_gate_up(L.mlp.gate_up_w)
                L.mlp.interleaved = True
        if self.comm.cfg.mlp_replicated:
            # this rank's slice of the whole MLP, for steps too short to pay for streaming all of it: gate / up rows are
            # interleaved in groups of 16, so the slice of both is one contiguous row range; down_proj is cut by columns
            tp, r = self.comm.tp_size, self.comm.tp_rank
            for L in self.layers:
                if L.mlp.is_moe or L.mlp.gate_up_w is None:
                    continue
                assert L.mlp.interleaved, "a replicated MLP needs the interleaved gate / up layout"
                i0, i1 = shard_range(self.args.intermediate_size, r, tp)
                L.mlp.gate_up_tp = L.mlp.gate_up_w[2 * i0:2 * i1]
                L.mlp.down_tp = L.mlp.down_w[:, i0:i1]
        return self

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """HF-named tensors of a single-rank model (used to write test checkpoints)."""
        a, D = self.args, self.args.head_dim
        assert self.comm.tp_size == 1 and self.comm.ep_size <= 1
        assert not any(L.mlp.interleaved for L in self.layers), "state_dict() must be taken before finalize_weights()"
        sd = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.final_norm}
        if not a.tie_word_embeddings:
            sd["lm_head.weight"] = self.lm_head
        for i, L in enumerate(self.layers):
            p = f"model.layers.{i}."
            sd[p + "input_layernorm.weight"] = L.input_norm
            sd[p + "post_attention_layernorm.weight"] = L.post_norm
            q, k, v = L.attn.qkv_w.split([a.n_heads * D, a.n_kv_heads * D, a.n_kv_heads * D], 0)
            sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"] = q, k, v
            if L.attn.qkv_b is not None:
                qb, kb, vb = L.attn.qkv_b.split([a.n_heads * D, a.n_kv_heads * D, a.n_kv_heads * D], 0)
                sd[p + "self_attn.q_proj.bias"], sd[p + "self_attn.k_proj.bias"], sd[p + "self_attn.v_proj.bias"] = qb, kb, vb
            sd[p + "self_attn.o_proj.weight"] = L.attn.o_w
            if a.qk_norm:
                sd[p + "self_attn.q_norm.weight"], sd[p + "self_attn.k_norm.weight"] = L.attn.q_norm, L.attn.k_norm
            if L.mlp.is_moe:
                sd[p + "mlp.gate.weight"] = L.mlp.router_w
                I = a.moe_intermediate_size
                for e in range(L.mlp.w13.shape[0]):
                    sd[p + f"mlp.experts.{e}.gate_proj.weight"] = L.mlp.w13[e, :I]
                    sd[p + f"mlp.experts.{e}.up_proj.weight"] = L.mlp.w13[e, I:]
                    sd[p + f"mlp.experts.{e}.down_proj.weight"] = L.mlp.w2[e]
            else:
                I = a.intermediate_size
                sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = L.mlp.gate_up_w[:I], L.mlp.gate_up_w[I:]
                sd[p + "mlp.down_proj.weight"] = L.mlp.down_w
        return {k: v.contiguous() for k, v in sd.items()}

    # ------------------------------------------------------------------ forward
    def _attention(self, L: LayerWeights, h: torch.Tensor, inp, kv) -> torch.Tensor:
        a = self.args
        qkv = ops.linear(h, L.attn.qkv_w, L.attn.qkv_b)
        q = ops.rope_qknorm_kvwrite(qkv, inp.positions, inp.slots, self.cos_sin, L.attn.q_norm, L.attn.k_norm,
                                    a.rms_norm_eps, kv[0], kv[1], self.n_q, self.n_kv, self.head_dim)
        return ops.paged_attention(q.view(-1, self.n_q, self.head_dim), kv[0], kv[1], inp, self.scale, a.sliding_window)

    def _moe(self, L: LayerWeights, h: torch.Tensor, layer_idx: int) -> torch.Tensor:
        """Returns this rank's partial MoE output (before the cross-rank reduction)."""
        a = self.args
        logits = ops.linear(h, L.mlp.router_w)
        if self.router_logit_bias is not None:
            logits = (logits.float() + self.router_logit_bias).to(logits.dtype)
        w, ids = ops.moe_router(logits, a.num_experts_per_tok, "softmax", a.norm_topk_prob)
        if self.expert_load is not None:
            self.expert_load[self._moe_index(layer_idx)].scatter_add_(
                0, ids.reshape(-1).long(), torch.ones(ids.numel(), dtype=torch.int64, device=ids.device))
        e0, _ = self._local_experts()
        if self.eplb is not None:                  # logical expert ids -> physical slots (replicas share the tokens)
            ids = self.eplb.route(self._moe_index(layer_idx), ids)
            e0 = self.eplb.expert_offset
        if self.moe_impl is not None:
            return self.moe_impl(h, L.mlp, w, ids, layer_idx)
        return ops.moe_experts(h, L.mlp.w13, L.mlp.w2, w, ids, e0, L.mlp.interleaved)

    def _moe_index(self, layer_idx: int) -> int:
        return sum(1 for j in range(layer_idx) if self.args.is_moe_layer(j))

    def _forward_fp8(self, x: torch.Tensor, inp, kv_caches) -> torch.Tensor:
        """Layers whose linear weights are fp8 (per-channel scales): every GEMM input is quantised per token, behind the
        RMSNorm that produces it (one kernel) or on its own (attention output, MLP activation); GEMM outputs, the residual
        stream, attention and the KV cache stay bf16.  Under tensor parallelism the partial sums meet in an NCCL
        all-reduce."""
        a, c = self.args, self.comm
        eps = a.rms_norm_eps
        n = len(self.layers)
        residual = x
        xq, xs = ops.rms_norm_quant_fp8(x, self.layers[0].input_norm, eps)
        h = None
        for i, L in enumerate(self.layers):
            kv = kv_caches[i]
            qkv = ops.linear_fp8_scaled(xq, xs, L.attn.qkv_w, L.attn.qkv_s, bias=L.attn.qkv_b)
            q = ops.rope_qknorm_kvwrite(qkv, inp.positions, inp.slots, self.cos_sin, L.attn.q_norm, L.attn.k_norm, eps, kv[0], kv[1],
                                        self.n_q, self.n_kv, self.head_dim)
            attn = ops.paged_attention(q.view(-1, self.n_q, self.head_dim), kv[0], kv[1], inp, self.scale, a.sliding_window)
            if self.layer_hook is not None:
                self.layer_hook(i)
            aq, as_ = ops.quant_rows_fp8(attn)
            y = c.all_reduce(ops.linear_fp8_scaled(aq, as_, L.attn.o_w, L.attn.o_s))
            xq, xs, residual = ops.add_rms_norm_quant_fp8(y, residual, L.post_norm, eps)
            if L.mlp.interleaved or not x.is_cuda:
                act = ops.linear_fp8_scaled(xq, xs, L.mlp.gate_up_w, L.mlp.gate_up_s, swiglu=True)
            else:
                act = ops.silu_and_mul(ops.linear_fp8_scaled(xq, xs, L.mlp.gate_up_w, L.mlp.gate_up_s))
            aq, as_ = ops.quant_rows_fp8(act)
            y = c.all_reduce(ops.linear_fp8_scaled(aq, as_, L.mlp.down_w, L.mlp.down_s))
            if i + 1 < n:
                xq, xs, residual = ops.add_rms_norm_quant_fp8(y, residual, self.layers[i + 1].input_norm, eps)
            else:
                h, residual = ops.add_rms_norm(y, residual, self.final_norm, eps)
        return h

    def forward(self, inp, kv_caches) -> torch.Tensor:
        """Returns the final-normed hidden states [T, H]."""
        a, c = self.args, self.comm
        x = ops.embedding(inp.tokens, self.embed)
        if getattr(self, "fp8_linears", False):
            return self._forward_fp8(x, inp, kv_caches)
        residual = c.init_residual(x)
        h = ops.rms_norm(x, self.layers[0].input_norm, a.rms_norm_eps)
        n = len(self.layers)
        # Long steps with a replicated MLP: attention is tensor parallel, the MLP runs on this rank's rows only.  Per layer
        # one reduce-scatter (after o_proj) and one all-gather (before the next qkv) instead of two of each.
        ft = c.fused_tp
        by_rows = (c.cfg.mlp_replicated and ft is not None and x.is_cuda and ft.mode == "nvls" and
                   x.shape[0] >= ft.mlp_rows_min_tokens)
        aux = []
        if self.capture_layers and ft is not None and x.is_cuda:
            raise RuntimeError("capturing layer inputs needs the whole residual stream on every rank: use "
                               "--communication_backend nccl with an EAGLE-3 draft under tensor parallelism")
        for i, L in enumerate(self.layers):
            if self.capture_layers and i in self.capture_layers:
                aux.append(residual)                 # the input of layer i (sum of everything before it)
            attn = self._attention(L, h, inp, kv_caches[i])
            if self.layer_hook is not None:
                self.layer_hook(i)
            next_norm = self.layers[i + 1].input_norm if i + 1 < n else self.final_norm
            if by_rows and not L.mlp.is_moe:
                h_mine, residual = ft.row_linear_reduce_norm(attn, L.attn.o_w, residual, L.post_norm, a.rms_norm_eps)
                act = ops.gate_up_swiglu(h_mine, L.mlp.gate_up_w, L.mlp.interleaved)
                y = ops.linear(act, L.mlp.down_w)
                h, residual = ft.add_norm_gather(y, x.shape[0], residual, next_norm, a.rms_norm_eps)
                continue
            h, residual = c.row_linear_add_rms_norm(attn, L.attn.o_w, residual, L.post_norm, a.rms_norm_eps)
            if L.mlp.is_moe:
                y = self._moe(L, h, i)
                partial_over_tp = self.moe_impl is None and c.tp_size > 1 and (
                    (c.ep_size == 1 and c.cfg.expert_shard()[1] > 1) or (c.ep_size == c.tp_size and c.dp_size == 1))
                if partial_over_tp:
                    # the experts are dealt out over exactly the TP ranks: their partial sums meet in the TP reduction
                    h, residual = c.partial_add_rms_norm(y, residual, next_norm, a.rms_norm_eps)
                    continue
                if c.ep_size > 1 and self.moe_impl is None:
                    y = c.all_reduce(y, group=c.ep_group)     # expert-parallel level 1 (fused_moe_base.cpp:101-136)
                if residual.shape[0] != y.shape[0]:
                    # complete MoE output beside a row-sharded residual stream (fused TP): each rank adds its own rows
                    if ft.mode == "nvls":
                        shard, rows = ft.shard_of(y.shape[0])
                        h, residual = ft.add_norm_gather(y[c.tp_rank * shard:c.tp_rank * shard + rows].contiguous(), y.shape[0],
                                                         residual, next_norm, a.rms_norm_eps)
                    else:
                        h, residual = c.partial_add_rms_norm(y if c.tp_rank == 0 else torch.zeros_like(y), residual, next_norm,
                                                             a.rms_norm_eps)
                else:
                    h, residual = ops.add_rms_norm(y, residual, next_norm, a.rms_norm_eps)
            else:
                gate_up, down = (L.mlp.gate_up_tp, L.mlp.down_tp) if L.mlp.gate_up_tp is not None else (L.mlp.gate_up_w, L.mlp.down_w)
                act = ops.gate_up_swiglu(h, gate_up, L.mlp.interleaved)
                h, residual = c.row_linear_add_rms_norm(act, down, residual, next_norm, a.rms_norm_eps)
        if aux:
            self.aux_hidden = torch.cat(aux, -1)
        return h

    def logits(self, hidden: torch.Tensor, sample_idx: torch.Tensor, gather: bool = True) -> torch.Tensor:
        """lm_head on the selected rows; vocab shards are gathered across TP ranks (linear.cpp:335-337)."""
        sel = hidden.index_select(0, sample_idx.long()) if sample_idx is not None else hidden
        lg = ops.linear(sel, self.lm_head)
        if self.comm.tp_size > 1 and gather:
            lg = self.comm.all_gather(lg, dim=-1)      # gather=False: this rank's vocabulary shard (greedy fast path)
        return lg

    def pooled_embedding(self, hidden: torch.Tensor, sample_idx: torch.Tensor) -> torch.Tensor:
        """Last-token pooling + L2 normalisation (embedding task; qwen3.h:238-247)."""
        e = hidden.index_select(0, sample_idx.long()).float()
        return torch.nn.functional.normalize(e, dim=-1)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.embed); add(self.lm_head); add(self.final_norm)
        for L in self.layers:
            for t in (L.input_norm, L.post_norm, L.attn.qkv_w, L.attn.qkv_b, L.attn.o_w, L.attn.q_norm, L.attn.k_norm,
                      L.mlp.gate_up_w, L.mlp.down_w, L.mlp.router_w, L.mlp.w13, L.mlp.w2, L.attn.qkv_s, L.attn.o_s,
                      L.mlp.gate_up_s, L.mlp.down_s):
                add(t)
        return total
