"""Model hyper-parameters parsed from a HF `config.json`.

Covers the architectures the reference registers for text generation on its CUDA/MLU builds:
qwen2, qwen3 (xllm/models/llm/qwen2.h:30-123, qwen3.h:30-283), qwen3_moe (qwen3_moe.h:30-279),
deepseek_v2/v3/v32 (deepseek_v2.h, deepseek_v3.h:42-101) and the exported MTP draft model
`deepseek_v3_mtp` (deepseek_mtp.h, mtp_model_base.h:28-245).  Defaults are those of the
reference's argument loaders.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, List, Optional


@dataclasses.dataclass
class QuantArgs:
    """Quantisation description (reference: hf_model_loader.cpp:57-123, quant_args.h)."""
    method: str = ""                 # "" | "fp8"
    weight_block_size: Optional[List[int]] = None   # [128, 128] for DeepSeek-V3 style checkpoints
    activation_dynamic: bool = True
    fmt: str = "e4m3"

    @property
    def block_scaled(self) -> bool:
        return self.method == "fp8" and self.weight_block_size is not None


@dataclasses.dataclass
class ModelArgs:
    model_type: str = "qwen3"
    dtype: str = "bfloat16"
    vocab_size: int = 151936
    hidden_size: int = 4096
    n_layers: int = 36
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 12288
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = False
    hidden_act: str = "silu"
    bos_token_id: int = -1
    eos_token_id: int = -1
    stop_token_ids: List[int] = dataclasses.field(default_factory=list)
    sliding_window: int = -1
    # MoE
    n_routed_experts: int = 0
    index_topk: int = 0                 # DeepSeek-V3.2: keys per query that the lightning indexer keeps (0: dense attention)
    index_n_heads: int = 0              # heads of the lightning indexer (0: the model has none)
    index_head_dim: int = 128
    index_rope_interleave: bool = False  # pairing of the indexer's RoPE: False = halves (DeepSeek-V3.2), True = even/odd
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    n_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: List[int] = dataclasses.field(default_factory=list)
    first_k_dense_replace: int = 0
    scoring_func: str = "softmax"
    topk_method: str = "greedy"        # "noaux_tc": sigmoid + correction bias + group-limited
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # rope scaling (yarn)
    rope_scaling_type: str = ""
    rope_scaling_factor: float = 1.0
    rope_original_max_position: int = 4096
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    rope_mscale: float = 1.0
    rope_mscale_all_dim: float = 0.0
    rope_low_freq_factor: float = 1.0       # "llama3" scaling
    rope_high_freq_factor: float = 4.0
    rope_attention_factor: float = 0.0      # yarn for dense models: scale of cos / sin (0: 0.1 ln(factor) + 1)
    # MTP
    num_nextn_predict_layers: int = 0
    quant: QuantArgs = dataclasses.field(default_factory=QuantArgs)

    # ------------------------------------------------------------------ derived
    @property
    def is_moe(self) -> bool:
        return self.n_routed_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    def is_moe_layer(self, layer: int) -> bool:
        """qwen3_moe.h `is_moe_layer` rule / DeepSeek `first_k_dense_replace`."""
        if not self.is_moe:
            return False
        if self.model_type.startswith("deepseek"):
            return layer >= self.first_k_dense_replace
        if layer in self.mlp_only_layers:
            return False
        return (layer + 1) % max(self.decoder_sparse_step, 1) == 0

    @property
    def kv_slot_dims(self) -> List[int]:
        """Per-token, per-layer cache width: GQA stores K and V, MLA one latent+rope row."""
        if self.is_mla:
            return [self.kv_lora_rank + self.qk_rope_head_dim]
        return [self.n_kv_heads * self.head_dim, self.n_kv_heads * self.head_dim]

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


def _first(cfg: Dict[str, Any], *names, default=None):
    for n in names:
        if n in cfg and cfg[n] is not None:
            return cfg[n]
    return default


def args_from_hf_config(cfg: Dict[str, Any]) -> ModelArgs:
    mt = _first(cfg, "model_type", "model_name", default="qwen3")
    a = ModelArgs(model_type=mt)
    a.dtype = {"float32": "float32", "float16": "float16"}.get(str(_first(cfg, "torch_dtype", "dtype", default="bfloat16")),
                                                                "bfloat16")
    a.vocab_size = int(_first(cfg, "vocab_size", default=a.vocab_size))
    a.hidden_size = int(_first(cfg, "hidden_size", default=a.hidden_size))
    a.n_layers = int(_first(cfg, "num_hidden_layers", default=a.n_layers))
    a.n_heads = int(_first(cfg, "num_attention_heads", default=a.n_heads))
    a.n_kv_heads = int(_first(cfg, "num_key_value_heads", default=a.n_heads))
    a.head_dim = int(_first(cfg, "head_dim", default=a.hidden_size // a.n_heads))
    a.intermediate_size = int(_first(cfg, "intermediate_size", default=a.intermediate_size))
    a.rms_norm_eps = float(_first(cfg, "rms_norm_eps", default=1e-6))
    a.rope_theta = float(_first(cfg, "rope_theta", default=1e6 if mt.startswith("qwen") else 1e4))
    a.max_position_embeddings = int(_first(cfg, "max_position_embeddings", default=32768))
    a.tie_word_embeddings = bool(_first(cfg, "tie_word_embeddings", default=False))
    a.hidden_act = _first(cfg, "hidden_act", default="silu")
    a.bos_token_id = int(_first(cfg, "bos_token_id", default=-1) or -1)
    eos = _first(cfg, "eos_token_id", default=-1)
    if isinstance(eos, list):
        a.eos_token_id = int(eos[0])
        a.stop_token_ids = [int(e) for e in eos[1:]]
    else:
        a.eos_token_id = int(eos if eos is not None else -1)
    sw = _first(cfg, "sliding_window", default=None)
    a.sliding_window = int(sw) if (sw and cfg.get("use_sliding_window", False)) else -1

    if mt in ("llama", "mistral"):
        # Llama-family decoder (same block as qwen2 without the qkv bias): rms norm, gated silu MLP, grouped-query attention
        a.attention_bias = bool(_first(cfg, "attention_bias", default=False))
        a.qk_norm = False
        if _first(cfg, "mlp_bias", default=False):
            raise ValueError("mlp_bias is not supported")
        if mt == "mistral" and sw:
            a.sliding_window = int(sw)       # Mistral applies its window whenever the config names one
    if not mt.startswith("deepseek"):
        rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or {}
        kind = rs.get("rope_type", rs.get("type", "")) if isinstance(rs, dict) else ""
        if kind in ("llama3", "linear", "yarn"):
            a.rope_scaling_type = kind
            a.rope_scaling_factor = float(rs.get("factor", 1.0))
            a.rope_original_max_position = int(rs.get("original_max_position_embeddings", a.max_position_embeddings))
            a.rope_low_freq_factor = float(rs.get("low_freq_factor", 1.0))
            a.rope_high_freq_factor = float(rs.get("high_freq_factor", 4.0))
            a.rope_beta_fast = float(rs.get("beta_fast", 32))
            a.rope_beta_slow = float(rs.get("beta_slow", 1))
            a.rope_attention_factor = float(rs.get("attention_factor") or 0.0)
        elif kind not in ("", "default"):
            raise ValueError(f"rope scaling '{kind}' is not supported")
        if isinstance(rs, dict) and "rope_theta" in rs and "rope_theta" not in cfg:
            a.rope_theta = float(rs["rope_theta"])
    if mt == "qwen2":
        a.attention_bias = True          # qwen2_attention.cpp:52 — qkv bias always on
        a.qk_norm = False
    elif mt in ("qwen3", "qwen3_moe"):
        a.attention_bias = bool(_first(cfg, "attention_bias", default=False))
        a.qk_norm = True
    if mt == "qwen3_moe":
        a.n_routed_experts = int(_first(cfg, "num_experts", "num_local_experts", default=128))
        a.num_experts_per_tok = int(_first(cfg, "num_experts_per_tok", default=8))
        a.moe_intermediate_size = int(_first(cfg, "moe_intermediate_size", default=768))
        a.norm_topk_prob = bool(_first(cfg, "norm_topk_prob", default=True))
        a.decoder_sparse_step = int(_first(cfg, "decoder_sparse_step", default=1))
        a.mlp_only_layers = list(_first(cfg, "mlp_only_layers", default=[]))
        a.scoring_func = "softmax"
    if mt.startswith("deepseek"):
        a.attention_bias = bool(_first(cfg, "attention_bias", default=False))
        a.n_routed_experts = int(_first(cfg, "n_routed_experts", default=256))
        a.num_experts_per_tok = int(_first(cfg, "num_experts_per_tok", default=8))
        a.moe_intermediate_size = int(_first(cfg, "moe_intermediate_size", default=2048))
        a.n_shared_experts = int(_first(cfg, "n_shared_experts", default=1))
        a.first_k_dense_replace = int(_first(cfg, "first_k_dense_replace", default=3))
        a.norm_topk_prob = bool(_first(cfg, "norm_topk_prob", default=True))
        a.scoring_func = _first(cfg, "scoring_func", default="sigmoid")
        a.topk_method = _first(cfg, "topk_method", default="noaux_tc")
        a.n_group = int(_first(cfg, "n_group", default=8))
        a.topk_group = int(_first(cfg, "topk_group", default=4))
        a.routed_scaling_factor = float(_first(cfg, "routed_scaling_factor", default=2.5))
        # `"q_lora_rank": null` (DeepSeek-V2-Lite) means no low-rank query projection; only a missing key takes the default
        a.q_lora_rank = int(cfg["q_lora_rank"] or 0) if "q_lora_rank" in cfg else 1536
        a.kv_lora_rank = int(_first(cfg, "kv_lora_rank", default=512))
        a.qk_nope_head_dim = int(_first(cfg, "qk_nope_head_dim", default=128))
        a.qk_rope_head_dim = int(_first(cfg, "qk_rope_head_dim", default=64))
        a.v_head_dim = int(_first(cfg, "v_head_dim", default=128))
        a.head_dim = a.qk_nope_head_dim + a.qk_rope_head_dim
        a.num_nextn_predict_layers = int(_first(cfg, "num_nextn_predict_layers", default=0))
        a.index_topk = int(_first(cfg, "index_topk", default=0))     # DeepSeek-V3.2 sparse attention: keys kept per query
        a.index_n_heads = int(_first(cfg, "index_n_heads", default=64 if a.index_topk > 0 else 0))
        a.index_head_dim = int(_first(cfg, "index_head_dim", default=128))
        a.index_rope_interleave = bool(_first(cfg, "indexer_rope_interleave", default=False))
        rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or {}     # newer exports call the block rope_parameters
        if "rope_theta" in rs and "rope_theta" not in cfg:
            a.rope_theta = float(rs["rope_theta"])
        if rs and rs.get("type", rs.get("rope_type", "")) not in ("", "default"):
            a.rope_scaling_type = rs.get("type", rs.get("rope_type", ""))
            a.rope_scaling_factor = float(rs.get("factor", 1.0))
            a.rope_original_max_position = int(rs.get("original_max_position_embeddings", 4096))
            a.rope_beta_fast = float(rs.get("beta_fast", 32))
            a.rope_beta_slow = float(rs.get("beta_slow", 1))
            a.rope_mscale = float(rs.get("mscale", 1.0))
            a.rope_mscale_all_dim = float(rs.get("mscale_all_dim", 0.0))
    qc = cfg.get("quantization_config") or {}
    if qc:
        method = qc.get("quant_method", "")
        if method in ("fp8", "compressed-tensors"):
            a.quant = QuantArgs(method="fp8", weight_block_size=qc.get("weight_block_size"),
                                activation_dynamic=qc.get("activation_scheme", "dynamic") == "dynamic",
                                fmt=qc.get("fmt", "e4m3"))
    return a


def load_model_args(model_dir: str) -> ModelArgs:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    a = args_from_hf_config(cfg)
    gpath = os.path.join(model_dir, "generation_config.json")
    if os.path.exists(gpath):
        with open(gpath) as f:
            g = json.load(f)
        eos = g.get("eos_token_id")
        if isinstance(eos, list):
            a.stop_token_ids = sorted(set(a.stop_token_ids) | {int(e) for e in eos if int(e) != a.eos_token_id})
        elif eos is not None and a.eos_token_id < 0:
            a.eos_token_id = int(eos)
    return a


# Named architectures of the benchmark configurations (random-init, synthetic requests).
def preset(name: str) -> ModelArgs:
    name = name.lower()
    if name in ("tiny-qwen2", "tiny_qwen2"):
        return ModelArgs(model_type="qwen2", dtype="float32", vocab_size=1024, hidden_size=256, n_layers=2, n_heads=4,
                         n_kv_heads=2, head_dim=64, intermediate_size=688, rms_norm_eps=1e-6, rope_theta=1e6,
                         tie_word_embeddings=True, attention_bias=True, qk_norm=False, max_position_embeddings=4096)
    if name in ("qwen3-8b", "qwen3_8b"):
        return ModelArgs(model_type="qwen3", vocab_size=151936, hidden_size=4096, n_layers=36, n_heads=32, n_kv_heads=8,
                         head_dim=128, intermediate_size=12288, qk_norm=True, rope_theta=1e6, max_position_embeddings=40960)
    if name in ("qwen2.5-72b", "qwen2_5_72b"):
        return ModelArgs(model_type="qwen2", vocab_size=152064, hidden_size=8192, n_layers=80, n_heads=64, n_kv_heads=8,
                         head_dim=128, intermediate_size=29568, attention_bias=True, qk_norm=False, rope_theta=1e6,
                         max_position_embeddings=32768)
    if name in ("qwen3-30b-a3b", "qwen3_30b_a3b"):
        return ModelArgs(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, n_layers=48, n_heads=32, n_kv_heads=4,
                         head_dim=128, intermediate_size=6144, qk_norm=True, n_routed_experts=128, num_experts_per_tok=8,
                         moe_intermediate_size=768, norm_topk_prob=True, rope_theta=1e6, max_position_embeddings=40960)
    if name in ("deepseek-v3", "deepseek_v3"):
        return ModelArgs(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, n_layers=61, n_heads=128,
                         n_kv_heads=128, head_dim=192, intermediate_size=18432, n_routed_experts=256, num_experts_per_tok=8,
                         moe_intermediate_size=2048, n_shared_experts=1, first_k_dense_replace=3, scoring_func="sigmoid",
                         topk_method="noaux_tc", n_group=8, topk_group=4, routed_scaling_factor=2.5, q_lora_rank=1536,
                         kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, rope_theta=1e4,
                         rope_scaling_type="yarn", rope_scaling_factor=40.0, rope_original_max_position=4096,
                         rope_mscale=1.0, rope_mscale_all_dim=1.0, max_position_embeddings=163840,
                         num_nextn_predict_layers=1,
                         quant=QuantArgs(method="fp8", weight_block_size=[128, 128]))
    raise KeyError(name)
