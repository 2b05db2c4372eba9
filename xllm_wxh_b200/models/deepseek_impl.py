"""DeepSeek-V2/V3 style decoder (MLA attention + MoE with shared experts) and its MTP draft model.

Behaviour follows the reference's MLU model path, which is the only place the reference implements these
architectures (xllm/models/llm/deepseek_v2.h, deepseek_v3.h:42-101, deepseek_mtp.h, mtp_model_base.h:28-245;
layers/mlu/deepseek_v2_attention.cpp:46-51,134-138,184-240,406-496; layers/mlu/moe_gate.cpp:56-72; fused_moe.cpp:147-175):

* MLA in absorbed form: `q = q_b(norm(q_a(x)))` split into nope / rope parts, `q_lat = q_nope . W_kc`; one 576-wide cache
  row per token `[norm(latent) | rope(k_pe)]`; attention over the latent with scale `(nope + rope)^-0.5 * mscale^2`;
  `out = (attn . W_vc) -> o_proj`.  RoPE is interleaved (GPT-J pairing) with YaRN frequency scaling.
* Router: sigmoid scores, selection on `score + e_score_correction_bias`, group-limited (n_group / topk_group), weights =
  un-biased scores of the selected experts, renormalised, times `routed_scaling_factor`; plus always-on shared experts.
* The first `first_k_dense_replace` layers use a dense SwiGLU MLP.
* Checkpoints may be bf16 or fp8 e4m3 with 128x128 block scales (`weight_scale_inv`), which the reference parses but
  cannot run (hf_model_loader.cpp:377-381); here block-scaled weights stay fp8 and run through the block-scaled GEMM.
* DeepSeek-V3.2 (`deepseek_v32`): a lightning indexer per layer (models/indexer.py) keeps `index_topk` keys per query; the
  attention then reads only those cache rows.  While every sequence of a step is that short the dense kernel runs.
* MTP draft model (`deepseek_v3_mtp`): `h' = eh_proj(cat(enorm(embed(tok)), hnorm(h_prev)))`, one decoder block, a
  shared-head norm, and the target's embedding / lm_head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..ops import reference as ref
from ..parallel.comm import Comm
from .args import ModelArgs
from .indexer import LightningIndexer
from .qwen import WeightInit, shard_range
from .registry import register_model

_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


class QLinear:
    """A weight matrix [N, K] that is either plain (bf16 / fp32) or fp8 e4m3 with 128x128 block scales."""
    __slots__ = ("w", "scale")

    def __init__(self, w: torch.Tensor, scale: Optional[torch.Tensor] = None):
        self.w, self.scale = w, scale

    @property
    def is_fp8(self) -> bool:
        return self.scale is not None

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.scale is None:
            return ops.linear(x, self.w)
        return ops.linear_fp8_block(x, self.w, self.scale)

    def dequant(self, dtype) -> torch.Tensor:
        if self.scale is None:
            return self.w
        return ref.dequant_weight_128x128(self.w, self.scale).to(dtype)

    def nbytes(self) -> int:
        n = self.w.numel() * self.w.element_size()
        return n + (self.scale.numel() * 4 if self.scale is not None else 0)


def _maybe_quant(w: torch.Tensor, fp8: bool) -> QLinear:
    if not fp8:
        return QLinear(w)
    q, s = ref.quant_weight_128x128(w)
    return QLinear(q, s)


class DsLayer:
    def __init__(self):
        self.input_norm = self.post_norm = None
        self.q_a = self.q_a_norm = self.q_b = self.q_proj = None
        self.kv_a = self.kv_a_norm = None
        self.w_kc = self.w_vc = None             # [Hh, nope, kv_lora], [Hh, v, kv_lora]  (from kv_b_proj, kept in model dtype)
        self.o = None
        # mlp
        self.is_moe = False
        self.gate_up = self.down = None          # dense or shared experts (QLinear)
        self.router_w = self.router_bias = None
        self.w13 = self.w2 = None                # [E_local, 2I, H], [E_local, H, I]
        self.w13_scale = self.w2_scale = None    # fp8 block scales [E_local, 2I/128, H/128], [E_local, H/128, I/128]
        self.shared_gate_up = self.shared_down = None
        self.interleaved = False
        self.indexer = None                      # LightningIndexer (DeepSeek-V3.2)


@register_model("deepseek_v2", "deepseek_v3", "deepseek_v32")
class DeepseekForCausalLM:
    is_mtp = False
    kv_replicated_over_tp = True      # the latent cache (and the index-key cache) is the same on every TP rank

    def __init__(self, args: ModelArgs, comm: Optional[Comm] = None, device="cpu", dtype: Optional[torch.dtype] = None):
        self.args = args
        self.comm = comm or Comm()
        self.device = torch.device(device)
        self.dtype = dtype or _DT[args.dtype]
        tp = self.comm.tp_size
        self.n_heads = args.n_heads // tp
        self.nope, self.rope, self.vdim, self.kv_lora = args.qk_nope_head_dim, args.qk_rope_head_dim, args.v_head_dim, args.kv_lora_rank
        self.fp8 = args.quant.block_scaled
        # DeepSeek-V3.2: each query attends to the `index_topk` keys that the layer's lightning indexer ranks highest
        # (models/indexer.py; the reference's MLU indexer, xllm/core/layers/mlu/indexer.h:64)
        self.indexer_on = args.index_topk > 0 and args.index_n_heads > 0
        if args.model_type == "deepseek_v32" and not self.indexer_on:
            raise ValueError("deepseek_v32 needs index_topk and index_n_heads in its configuration (the lightning indexer); "
                             "without them the checkpoint is a deepseek_v3 one")
        if self.indexer_on and args.q_lora_rank <= 0:
            raise ValueError("the lightning indexer reads the low-rank query latent: q_lora_rank must be set")
        self.layers: List[DsLayer] = [DsLayer() for _ in range(self._num_layers())]
        if self.indexer_on:
            for L in self.layers:
                L.indexer = LightningIndexer(args, self.device, self.dtype)
        self.embed = self.final_norm = self.lm_head = None
        # YaRN: blended frequencies, cos/sin scaled by mscale / mscale_all_dim ratio; softmax scale by mscale_all_dim^2
        mscale = 1.0
        self.softmax_scale = (self.nope + self.rope) ** -0.5
        inv_freq = None
        if args.rope_scaling_type == "yarn":
            inv_freq = ref.yarn_inv_freq(self.rope, args.rope_theta, args.rope_scaling_factor, args.rope_original_max_position,
                                         args.rope_beta_fast, args.rope_beta_slow)
            m_all = ref.yarn_mscale(args.rope_scaling_factor, args.rope_mscale_all_dim) if args.rope_mscale_all_dim else 1.0
            mscale = ref.yarn_mscale(args.rope_scaling_factor, args.rope_mscale) / m_all
            self.softmax_scale *= m_all * m_all
        self.cos_sin = ref.build_cos_sin_cache(self.rope, args.max_position_embeddings, args.rope_theta, dtype=torch.float32,
                                               device=self.device, inv_freq=inv_freq, mscale=mscale)
        self.expert_load = None
        self.moe_impl = None
        self.layer_hook = None

    def _num_layers(self) -> int:
        return self.args.n_layers

    # ------------------------------------------------------------------ shapes
    def kv_cache_shapes(self, num_blocks: int, block_size: int):
        """Per layer: the latent cache, and with a lightning indexer its index-key cache behind it."""
        per = ((num_blocks, block_size, self.kv_lora + self.rope),)
        if self.indexer_on:
            per += ((num_blocks, block_size, self.args.index_head_dim),)
        return [per for _ in range(len(self.layers))]

    def _local_experts(self) -> Tuple[int, int]:
        return shard_range(self.args.n_routed_experts, *self.comm.cfg.expert_shard())

    def _layer_index(self, i: int) -> int:
        """Index used in weight names and in the dense / MoE rule."""
        return i

    # ------------------------------------------------------------------ random init
    def init_random(self, seed: int = 0, std: float = 0.02):
        a, c = self.args, self.comm
        wi = WeightInit(seed, std, self.dtype, self.device)
        H, tp, r = a.hidden_size, c.tp_size, c.tp_rank
        if not self.is_mtp or self.embed is None:
            self.embed = wi.normal("model.embed_tokens.weight", (a.vocab_size, H))
            self.lm_head = wi.normal("lm_head.weight", (a.vocab_size, H), rows=shard_range(a.vocab_size, r, tp))
        self.final_norm = wi.ones((H,))
        h0, h1 = shard_range(a.n_heads, r, tp)
        qk = self.nope + self.rope
        for i, L in enumerate(self.layers):
            p = f"model.layers.{self._layer_index(i)}."
            self._init_layer_random(L, wi, p, self._layer_index(i), h0, h1, qk)
        self._init_extra_random(wi)
        return self

    def _init_extra_random(self, wi: WeightInit):
        pass

    def _init_layer_random(self, L: DsLayer, wi: WeightInit, p: str, layer_idx: int, h0: int, h1: int, qk: int):
        a, c = self.args, self.comm
        H, tp, r = a.hidden_size, c.tp_size, c.tp_rank
        L.input_norm, L.post_norm = wi.ones((H,)), wi.ones((H,))
        if a.q_lora_rank > 0:
            L.q_a = _maybe_quant(wi.normal(p + "self_attn.q_a_proj.weight", (a.q_lora_rank, H)), self.fp8)
            L.q_a_norm = wi.ones((a.q_lora_rank,))
            L.q_b = _maybe_quant(wi.normal(p + "self_attn.q_b_proj.weight", (a.n_heads * qk, a.q_lora_rank), rows=(h0 * qk, h1 * qk)), self.fp8)
        else:
            L.q_proj = _maybe_quant(wi.normal(p + "self_attn.q_proj.weight", (a.n_heads * qk, H), rows=(h0 * qk, h1 * qk)), self.fp8)
        L.kv_a = _maybe_quant(wi.normal(p + "self_attn.kv_a_proj_with_mqa.weight", (self.kv_lora + self.rope, H)), self.fp8)
        L.kv_a_norm = wi.ones((self.kv_lora,))
        per = self.nope + self.vdim
        kvb = wi.normal(p + "self_attn.kv_b_proj.weight", (a.n_heads * per, self.kv_lora), rows=(h0 * per, h1 * per))
        self._set_kv_b(L, kvb)
        L.o = _maybe_quant(wi.normal(p + "self_attn.o_proj.weight", (H, a.n_heads * self.vdim), cols=(h0 * self.vdim, h1 * self.vdim)), self.fp8)
        if L.indexer is not None:
            L.indexer.init_random(wi, p + "self_attn.indexer.", a.q_lora_rank, H)
        if a.is_moe_layer(layer_idx):
            L.is_moe = True
            L.router_w = wi.normal(p + "mlp.gate.weight", (a.n_routed_experts, H), dtype=torch.float32 if self.device.type == "cpu" else None)
            if a.topk_method == "noaux_tc":
                L.router_bias = wi.normal(p + "mlp.gate.e_score_correction_bias", (a.n_routed_experts,), dtype=torch.float32)
            I = a.moe_intermediate_size
            e0, e1 = self._local_experts()
            w13, w2 = [], []
            for e in range(e0, e1):
                g = wi.normal(p + f"mlp.experts.{e}.gate_proj.weight", (I, H))
                u = wi.normal(p + f"mlp.experts.{e}.up_proj.weight", (I, H))
                w13.append(torch.cat([g, u], 0))
                w2.append(wi.normal(p + f"mlp.experts.{e}.down_proj.weight", (H, I)))
            self._set_experts(L, torch.stack(w13), torch.stack(w2))
            if a.n_shared_experts > 0:
                Is = I * a.n_shared_experts
                s0, s1 = shard_range(Is, r, tp)
                g = wi.normal(p + "mlp.shared_experts.gate_proj.weight", (Is, H), rows=(s0, s1))
                u = wi.normal(p + "mlp.shared_experts.up_proj.weight", (Is, H), rows=(s0, s1))
                L.shared_gate_up = _maybe_quant(torch.cat([g, u], 0), self.fp8)
                L.shared_down = _maybe_quant(wi.normal(p + "mlp.shared_experts.down_proj.weight", (H, Is), cols=(s0, s1)), self.fp8)
        else:
            I = a.intermediate_size
            i0, i1 = shard_range(I, r, tp)
            g = wi.normal(p + "mlp.gate_proj.weight", (I, H), rows=(i0, i1))
            u = wi.normal(p + "mlp.up_proj.weight", (I, H), rows=(i0, i1))
            L.gate_up = _maybe_quant(torch.cat([g, u], 0), self.fp8)
            L.down = _maybe_quant(wi.normal(p + "mlp.down_proj.weight", (H, I), cols=(i0, i1)), self.fp8)

    def _set_kv_b(self, L: DsLayer, kvb: torch.Tensor):
        per = self.nope + self.vdim
        w = kvb.view(-1, per, self.kv_lora)
        L.w_kc = w[:, :self.nope, :].contiguous()                  # [Hh, nope, c]
        L.w_vc = w[:, self.nope:, :].contiguous()                  # [Hh, v, c]

    def _set_experts(self, L: DsLayer, w13: torch.Tensor, w2: torch.Tensor):
        if not self.fp8:
            L.w13, L.w2 = w13, w2
            return
        q13, s13, q2, s2 = [], [], [], []
        for e in range(w13.shape[0]):
            q, s = ref.quant_weight_128x128(w13[e]); q13.append(q); s13.append(s)
            q, s = ref.quant_weight_128x128(w2[e]); q2.append(q); s2.append(s)
        L.w13, L.w13_scale = torch.stack(q13), torch.stack(s13)
        L.w2, L.w2_scale = torch.stack(q2), torch.stack(s2)

    # ------------------------------------------------------------------ checkpoint loading
    def _get_linear(self, ckpt, name: str, rows=None, cols=None) -> QLinear:
        """HF tensor `name` (+ `name[:-6] + 'weight_scale_inv'` for fp8 block-scaled checkpoints), sharded."""
        w = ckpt.get(name)
        sname = name.replace(".weight", ".weight_scale_inv")
        if w.dtype == torch.float8_e4m3fn and ckpt.has(sname):
            s = ckpt.get(sname).float()
            if rows is not None:
                assert rows[0] % 128 == 0
                w, s = w[rows[0]:rows[1]], s[rows[0] // 128:(rows[1] + 127) // 128]
            if cols is not None:
                assert cols[0] % 128 == 0
                w, s = w[:, cols[0]:cols[1]], s[:, cols[0] // 128:(cols[1] + 127) // 128]
            if self.fp8:
                return QLinear(w.contiguous().to(self.device), s.contiguous().to(self.device))
            return QLinear(ref.dequant_weight_128x128(w, s).to(self.device, self.dtype))
        if rows is not None:
            w = w[rows[0]:rows[1]]
        if cols is not None:
            w = w[:, cols[0]:cols[1]]
        w = w.to(self.device, self.dtype).contiguous()
        return _maybe_quant(w, self.fp8)

    def _get_dense(self, ckpt, name: str) -> torch.Tensor:
        """HF tensor `name` in the model dtype on the device; an fp8 block-scaled one is dequantised."""
        w = ckpt.get(name)
        sname = name.replace(".weight", ".weight_scale_inv")
        if w.dtype == torch.float8_e4m3fn and ckpt.has(sname):
            w = ref.dequant_weight_128x128(w, ckpt.get(sname).float())
        return w.to(self.device, self.dtype).contiguous()

    def load_weights(self, ckpt, prefix_layers: str = "model.layers."):
        a, c = self.args, self.comm
        H, tp, r = a.hidden_size, c.tp_size, c.tp_rank
        dev = lambda t: t.to(self.device, self.dtype).contiguous()
        if ckpt.has("model.embed_tokens.weight"):
            self.embed = dev(ckpt.get("model.embed_tokens.weight"))
        v0, v1 = shard_range(a.vocab_size, r, tp)
        if ckpt.has("lm_head.weight"):
            self.lm_head = dev(ckpt.get("lm_head.weight")[v0:v1])
        if ckpt.has("model.norm.weight"):
            self.final_norm = dev(ckpt.get("model.norm.weight"))
        h0, h1 = shard_range(a.n_heads, r, tp)
        qk = self.nope + self.rope
        per = self.nope + self.vdim
        for i, L in enumerate(self.layers):
            li = self._layer_index(i)
            p = f"{prefix_layers}{li}."
            L.input_norm = dev(ckpt.get(p + "input_layernorm.weight"))
            L.post_norm = dev(ckpt.get(p + "post_attention_layernorm.weight"))
            if a.q_lora_rank > 0:
                L.q_a = self._get_linear(ckpt, p + "self_attn.q_a_proj.weight")
                L.q_a_norm = dev(ckpt.get(p + "self_attn.q_a_layernorm.weight"))
                L.q_b = self._get_linear(ckpt, p + "self_attn.q_b_proj.weight", rows=(h0 * qk, h1 * qk))
            else:
                L.q_proj = self._get_linear(ckpt, p + "self_attn.q_proj.weight", rows=(h0 * qk, h1 * qk))
            L.kv_a = self._get_linear(ckpt, p + "self_attn.kv_a_proj_with_mqa.weight")
            L.kv_a_norm = dev(ckpt.get(p + "self_attn.kv_a_layernorm.weight"))
            kvb = self._get_linear(ckpt, p + "self_attn.kv_b_proj.weight", rows=(h0 * per, h1 * per))
            self._set_kv_b(L, kvb.dequant(self.dtype))
            L.o = self._get_linear(ckpt, p + "self_attn.o_proj.weight", cols=(h0 * self.vdim, h1 * self.vdim))
            if L.indexer is not None:
                L.indexer.load(ckpt, p + "self_attn.indexer.", lambda n: self._get_dense(ckpt, n))
            if a.is_moe_layer(li):
                L.is_moe = True
                L.router_w = ckpt.get(p + "mlp.gate.weight").to(self.device, torch.float32 if self.device.type == "cpu" else self.dtype)
                if ckpt.has(p + "mlp.gate.e_score_correction_bias"):
                    L.router_bias = ckpt.get(p + "mlp.gate.e_score_correction_bias").to(self.device, torch.float32)
                e0, e1 = self._local_experts()
                w13 = torch.stack([torch.cat([self._get_linear(ckpt, p + f"mlp.experts.{e}.gate_proj.weight").dequant(self.dtype),
                                              self._get_linear(ckpt, p + f"mlp.experts.{e}.up_proj.weight").dequant(self.dtype)], 0)
                                   for e in range(e0, e1)])
                w2 = torch.stack([self._get_linear(ckpt, p + f"mlp.experts.{e}.down_proj.weight").dequant(self.dtype)
                                  for e in range(e0, e1)])
                self._set_experts(L, w13, w2)
                if ckpt.has(p + "mlp.shared_experts.gate_proj.weight"):
                    Is = a.moe_intermediate_size * a.n_shared_experts
                    s0, s1 = shard_range(Is, r, tp)
                    g = self._get_linear(ckpt, p + "mlp.shared_experts.gate_proj.weight", rows=(s0, s1)).dequant(self.dtype)
                    u = self._get_linear(ckpt, p + "mlp.shared_experts.up_proj.weight", rows=(s0, s1)).dequant(self.dtype)
                    L.shared_gate_up = _maybe_quant(torch.cat([g, u], 0), self.fp8)
                    L.shared_down = self._get_linear(ckpt, p + "mlp.shared_experts.down_proj.weight", cols=(s0, s1))
            else:
                I = a.intermediate_size
                i0, i1 = shard_range(I, r, tp)
                g = self._get_linear(ckpt, p + "mlp.gate_proj.weight", rows=(i0, i1)).dequant(self.dtype)
                u = self._get_linear(ckpt, p + "mlp.up_proj.weight", rows=(i0, i1)).dequant(self.dtype)
                L.gate_up = _maybe_quant(torch.cat([g, u], 0), self.fp8)
                L.down = self._get_linear(ckpt, p + "mlp.down_proj.weight", cols=(i0, i1))
        self._load_extra(ckpt)
        return self

    def _load_extra(self, ckpt):
        pass

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """HF-named tensors of a single-rank, unquantised model (used to write test checkpoints)."""
        a = self.args
        assert self.comm.tp_size == 1 and self.comm.ep_size <= 1 and not self.fp8
        sd = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.final_norm, "lm_head.weight": self.lm_head}
        for i, L in enumerate(self.layers):
            p = f"model.layers.{self._layer_index(i)}."
            sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = L.input_norm, L.post_norm
            if L.q_a is not None:
                sd[p + "self_attn.q_a_proj.weight"], sd[p + "self_attn.q_a_layernorm.weight"] = L.q_a.w, L.q_a_norm
                sd[p + "self_attn.q_b_proj.weight"] = L.q_b.w
            else:
                sd[p + "self_attn.q_proj.weight"] = L.q_proj.w
            sd[p + "self_attn.kv_a_proj_with_mqa.weight"], sd[p + "self_attn.kv_a_layernorm.weight"] = L.kv_a.w, L.kv_a_norm
            sd[p + "self_attn.kv_b_proj.weight"] = torch.cat([L.w_kc, L.w_vc], 1).reshape(-1, self.kv_lora)
            sd[p + "self_attn.o_proj.weight"] = L.o.w
            if L.indexer is not None:
                sd.update(L.indexer.state(p + "self_attn.indexer."))
            if L.is_moe:
                I = a.moe_intermediate_size
                sd[p + "mlp.gate.weight"] = L.router_w
                if L.router_bias is not None:
                    sd[p + "mlp.gate.e_score_correction_bias"] = L.router_bias
                for e in range(L.w13.shape[0]):
                    sd[p + f"mlp.experts.{e}.gate_proj.weight"], sd[p + f"mlp.experts.{e}.up_proj.weight"] = L.w13[e, :I], L.w13[e, I:]
                    sd[p + f"mlp.experts.{e}.down_proj.weight"] = L.w2[e]
                if L.shared_gate_up is not None:
                    Is = L.shared_gate_up.w.shape[0] // 2
                    sd[p + "mlp.shared_experts.gate_proj.weight"] = L.shared_gate_up.w[:Is]
                    sd[p + "mlp.shared_experts.up_proj.weight"] = L.shared_gate_up.w[Is:]
                    sd[p + "mlp.shared_experts.down_proj.weight"] = L.shared_down.w
            else:
                I = L.gate_up.w.shape[0] // 2
                sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = L.gate_up.w[:I], L.gate_up.w[I:]
                sd[p + "mlp.down_proj.weight"] = L.down.w
        return {k: v.contiguous() for k, v in sd.items() if v is not None}

    # ------------------------------------------------------------------ forward
    def _attention(self, L: DsLayer, h: torch.Tensor, inp, kv) -> torch.Tensor:
        a = self.args
        T = h.shape[0]
        q_in = None
        if L.q_a is not None:
            q_in = ops.rms_norm(L.q_a(h), L.q_a_norm, a.rms_norm_eps)
            q = L.q_b(q_in)
        else:
            q = L.q_proj(h)
        q = q.view(T, self.n_heads, self.nope + self.rope)
        kv_a = L.kv_a(h)                                                        # [T, c + rope]
        kept = None
        if L.indexer is not None:
            L.indexer.write_keys(h, inp.positions, inp.slots, self.cos_sin, kv[1])
            if L.indexer.wanted(inp, kv[0].shape[1]):
                kept = L.indexer.select(*L.indexer.queries(h, q_in, inp.positions, self.cos_sin), kv[1], inp)
        # latent norm + interleaved RoPE on q_pe / k_pe + cache write, then absorb W_kc into q
        q_lat, q_pe = ops.mla_prepare(q, kv_a, inp.positions, inp.slots, self.cos_sin, L.kv_a_norm, a.rms_norm_eps, kv[0],
                                      L.w_kc, self.nope, self.rope, self.kv_lora)
        if kept is None:
            o_lat = ops.mla_attention(q_lat, q_pe, kv[0], inp, self.softmax_scale, self.kv_lora)    # [T, Hh, c]
        else:
            o_lat = ops.mla_attention_sparse(q_lat, q_pe, kv[0], kept[0], kept[1], self.softmax_scale, self.kv_lora)
        o = ops.mla_v_up(o_lat, L.w_vc)                                                          # [T, Hh * v]
        return o

    def _mlp_partial(self, L: DsLayer, h: torch.Tensor, layer_idx: int) -> torch.Tensor:
        """MoE layers: routed + shared output of this rank (partial under TP / EP level 1)."""
        a = self.args
        logits = ops.linear(h.to(L.router_w.dtype), L.router_w)
        grouped = a.topk_method == "noaux_tc" or a.n_group > 1
        w, ids = ops.moe_router(logits, a.num_experts_per_tok, a.scoring_func, a.norm_topk_prob, L.router_bias,
                                a.n_group if grouped else 1, a.topk_group if grouped else 1, a.routed_scaling_factor)
        if self.expert_load is not None:
            self.expert_load[self._moe_index(layer_idx)].scatter_add_(
                0, ids.reshape(-1).long(), torch.ones(ids.numel(), dtype=torch.int64, device=ids.device))
        shared = None
        if L.shared_gate_up is not None:
            shared = L.shared_down(ops.silu_and_mul(L.shared_gate_up(h)))
        eplb = getattr(self, "eplb", None)
        if eplb is not None:                       # logical expert ids -> physical slots (replicas share the tokens)
            ids = eplb.route(self._moe_index(layer_idx), ids)
        if self.moe_impl is not None:
            y = self.moe_impl(h, L, w, ids, layer_idx)
            # moe_impl returns the complete routed output; the shared expert is partial under TP
            if shared is not None:
                y = y + (self.comm.all_reduce(shared) if self.comm.tp_size > 1 else shared)
            return y
        e0, _ = self._local_experts()
        if eplb is not None:
            e0 = eplb.expert_offset
        y = ops.moe_experts_q(h, L, w, ids, e0)
        return y + shared if shared is not None else y

    def _moe_index(self, layer_idx: int) -> int:
        return sum(1 for j in range(layer_idx) if self.args.is_moe_layer(j))

    def _decoder_stack(self, x: torch.Tensor, inp, kv_caches, final_norm: torch.Tensor) -> torch.Tensor:
        """Under tensor parallelism every row-parallel output (o_proj, dense MLP, routed + shared experts) goes through
        the fused reduce + residual + RMSNorm + all-gather of `Comm` (the reference reduces after o_proj and after the MLP
        with NCCL and normalises apart: deepseek_v2_decoder_layer_impl.cpp, linear.cpp:822-825); the residual stream is
        then this rank's row shard.  With a fused expert-parallel exchange the MoE output is already complete, and the
        plain path below is used."""
        a, c = self.args, self.comm
        fused = c.tp_size > 1 and c.fused_tp is not None and x.is_cuda and self.moe_impl is None and c.ep_size == 1
        residual = c.init_residual(x) if fused else x
        h = ops.rms_norm(x, self.layers[0].input_norm, a.rms_norm_eps)
        n = len(self.layers)

        def reduce_norm(y, lin, act, norm_w):
            """`y` partial result, or (`lin`, `act`): the bf16 row-parallel linear that produces it."""
            if fused:
                if y is None and not lin.is_fp8:
                    return c.row_linear_add_rms_norm(act, lin.w, residual, norm_w, a.rms_norm_eps)
                return c.partial_add_rms_norm(lin(act) if y is None else y, residual, norm_w, a.rms_norm_eps)
            y = lin(act) if y is None else y
            if c.tp_size > 1:
                y = c.all_reduce(y)
            return ops.add_rms_norm(y, residual, norm_w, a.rms_norm_eps)

        for i, L in enumerate(self.layers):
            attn = self._attention(L, h, inp, kv_caches[i])
            if self.layer_hook is not None:
                self.layer_hook(i)              # the layer's KV is in the cache: a disaggregated prefill pushes it now
            h, residual = reduce_norm(None, L.o, attn, L.post_norm)
            next_norm = self.layers[i + 1].input_norm if i + 1 < n else final_norm
            if L.is_moe:
                y = self._mlp_partial(L, h, self._layer_index(i))
                if fused:
                    h, residual = reduce_norm(y, None, None, next_norm)
                    continue
                if self.moe_impl is None and (c.tp_size > 1 or c.ep_size > 1):
                    y = c.all_reduce(y, group=c.world_group if c.ep_size > 1 else c.tp_group)
                h, residual = ops.add_rms_norm(y, residual, next_norm, a.rms_norm_eps)
            else:
                h, residual = reduce_norm(None, L.down, ops.silu_and_mul(L.gate_up(h)), next_norm)
        return h

    def forward(self, inp, kv_caches) -> torch.Tensor:
        x = ops.embedding(inp.tokens, self.embed)
        return self._decoder_stack(x, inp, kv_caches, self.final_norm)

    def logits(self, hidden: torch.Tensor, sample_idx: torch.Tensor, gather: bool = True) -> torch.Tensor:
        sel = hidden.index_select(0, sample_idx.long()) if sample_idx is not None else hidden
        lg = ops.linear(sel, self.lm_head)
        if self.comm.tp_size > 1 and gather:
            lg = self.comm.all_gather(lg, dim=-1)      # gather=False: this rank's vocabulary shard (greedy fast path)
        return lg

    def pooled_embedding(self, hidden, sample_idx):
        return torch.nn.functional.normalize(hidden.index_select(0, sample_idx.long()).float(), dim=-1)

    def weight_bytes(self) -> int:
        total = 0
        for t in (self.embed, self.lm_head, self.final_norm):
            total += t.numel() * t.element_size() if t is not None else 0
        for L in self.layers:
            for q in (L.q_a, L.q_b, L.q_proj, L.kv_a, L.o, L.gate_up, L.down, L.shared_gate_up, L.shared_down):
                total += q.nbytes() if q is not None else 0
            for t in (L.w_kc, L.w_vc, L.w13, L.w2, L.w13_scale, L.w2_scale, L.router_w):
                total += t.numel() * t.element_size() if t is not None else 0
            total += L.indexer.nbytes() if L.indexer is not None else 0
        return total


class _ExportedMtpView:
    """Reads a draft directory written by the MTP export tool (tools/export_mtp.py of the reference, :170-183) through
    the names of the full checkpoint: the block is `model.layers.0.*` there, and `enorm / hnorm / eh_proj / embed_tokens /
    shared_head.*` sit directly under `model.`."""
    MODEL_LEVEL = ("embed_tokens", "shared_head", "enorm", "hnorm", "eh_proj")

    def __init__(self, ckpt, layer: int):
        self.ckpt, self.prefix = ckpt, f"model.layers.{layer}."

    def _map(self, name: str) -> str:
        if not name.startswith(self.prefix):
            return name
        rest = name[len(self.prefix):]
        return ("model." if any(s in rest for s in self.MODEL_LEVEL) else "model.layers.0.") + rest

    def has(self, name: str) -> bool:
        return self.ckpt.has(self._map(name))

    def get(self, name: str):
        return self.ckpt.get(self._map(name))

    def get_or_none(self, name: str):
        return self.ckpt.get_or_none(self._map(name))

    def keys(self):
        return self.ckpt.keys()


@register_model("deepseek_v3_mtp", "deepseek_mtp", "deepseek_v32_mtp")
class DeepseekMTP(DeepseekForCausalLM):
    """One MTP module: predicts token t+2 from the target's hidden state at t and the embedding of token t+1.
    The decoder block is layer `n_layers + k` of the original checkpoint (mtp_model_base.h:51-84,205-218)."""
    is_mtp = True

    def __init__(self, args: ModelArgs, comm=None, device="cpu", dtype=None, target: Optional[DeepseekForCausalLM] = None):
        self.target = target
        super().__init__(args, comm, device, dtype)
        self.enorm = self.hnorm = self.eh_proj = self.shared_head_norm = None
        if target is not None:
            self.embed, self.lm_head = target.embed, target.lm_head

    def _num_layers(self) -> int:
        return 1

    def _layer_index(self, i: int) -> int:
        return self.args.n_layers + i

    def _init_extra_random(self, wi: WeightInit):
        H = self.args.hidden_size
        p = f"model.layers.{self.args.n_layers}."
        self.enorm, self.hnorm, self.shared_head_norm = wi.ones((H,)), wi.ones((H,)), wi.ones((H,))
        self.eh_proj = QLinear(wi.normal(p + "eh_proj.weight", (H, 2 * H)))
        if self.target is not None:
            self.embed, self.lm_head = self.target.embed, self.target.lm_head

    def load_weights(self, ckpt, prefix_layers: str = "model.layers."):
        if ckpt.has("model.enorm.weight") and not ckpt.has(f"model.layers.{self.args.n_layers}.enorm.weight"):
            ckpt = _ExportedMtpView(ckpt, self.args.n_layers)      # an exported draft directory
        return super().load_weights(ckpt, prefix_layers)

    def _load_extra(self, ckpt):
        p = f"model.layers.{self.args.n_layers}."
        dev = lambda t: t.to(self.device, self.dtype).contiguous()
        self.enorm, self.hnorm = dev(ckpt.get(p + "enorm.weight")), dev(ckpt.get(p + "hnorm.weight"))
        self.eh_proj = QLinear(dev(ckpt.get(p + "eh_proj.weight")))
        self.shared_head_norm = dev(ckpt.get(p + "shared_head.norm.weight"))
        if ckpt.has(p + "embed_tokens.weight") and self.embed is None:
            self.embed = dev(ckpt.get(p + "embed_tokens.weight"))
        if ckpt.has(p + "shared_head.head.weight") and self.lm_head is None:
            self.lm_head = dev(ckpt.get(p + "shared_head.head.weight"))

    def forward_mtp(self, inp, kv_caches, prev_hidden: torch.Tensor) -> torch.Tensor:
        """`inp.tokens` are the tokens following the positions of `prev_hidden` (shifted by one)."""
        a = self.args
        e = ops.embedding(inp.tokens, self.embed)
        e = torch.where((inp.positions == 0)[:, None], torch.zeros_like(e), e)       # position 0 has no predecessor state
        x = self.eh_proj(torch.cat([ops.rms_norm(e, self.enorm, a.rms_norm_eps),
                                    ops.rms_norm(prev_hidden, self.hnorm, a.rms_norm_eps)], dim=-1))
        return self._decoder_stack(x, inp, kv_caches, self.shared_head_norm)

    def forward(self, inp, kv_caches) -> torch.Tensor:
        raise RuntimeError("the MTP module needs the target's hidden states: call forward_mtp")
