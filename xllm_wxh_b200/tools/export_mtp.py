"""Export the multi-token-prediction (MTP) block of a DeepSeek-V3 / R1 / V3.2 style checkpoint as a draft model directory.

Same job and output layout as the reference's tools/export_mtp.py (:155-217): the decoder block stored as layer
`num_hidden_layers` of the full checkpoint becomes layer 0 of a one-layer model, its MTP-specific tensors
(`enorm`, `hnorm`, `eh_proj`, `embed_tokens`, `shared_head.*`) move to the model level, fp8 128x128 block-scaled weights
are dequantised to bf16, `config.json` is rewritten (`num_hidden_layers = 1`, `model_type = <type>_mtp`,
`first_k_dense_replace = 0`, no `quantization_config`) and every other file of the directory is copied.

    python -m xllm_wxh_b200.tools.export_mtp --input-dir /path/to/DeepSeek-V3 --output-dir /path/to/DeepSeek-V3-mtp

The result is what `--draft_model` expects; the engine also accepts the full checkpoint directory as a draft model and
then reads the same block in place.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict, Optional

import torch

from ..utils.safetensors_io import CheckpointReader, save_safetensors

MODEL_LEVEL = ("embed_tokens", "shared_head", "enorm", "hnorm", "eh_proj")
MTP_TYPES = {"deepseek_v3": ("deepseek_v3_mtp", "DeepseekMTPForCausalLM"),
             "deepseek_v32": ("deepseek_v32_mtp", "DeepseekV32MtpForCausalLM"),
             "glm4_moe": ("glm4_moe_mtp", "Glm4MoeMtpForCausalLM")}


def detect_model_type(cfg: Dict) -> str:
    mt = str(cfg.get("model_type", "")).lower()
    archs = [str(a).lower() for a in cfg.get("architectures") or []]
    if "deepseek" in mt or any("deepseek" in a for a in archs):
        return "deepseek_v32" if any(k in cfg for k in ("index_head_dim", "index_n_heads", "index_topk")) else "deepseek_v3"
    if "glm4" in mt or any("glm4" in a for a in archs):
        return "glm4_moe" if int(cfg.get("n_routed_experts") or 0) > 0 else "glm4"
    if mt:
        return mt
    raise ValueError("unable to detect the model type from config.json")


def block_dequant(w8: torch.Tensor, scale: torch.Tensor, block=(128, 128)) -> torch.Tensor:
    """fp8 weight [N, K] x one fp32 scale per 128x128 block -> bf16."""
    n, k = w8.shape
    bn, bk = block
    assert scale.shape == ((n + bn - 1) // bn, (k + bk - 1) // bk), (scale.shape, w8.shape)
    s = scale.float().repeat_interleave(bn, 0)[:n].repeat_interleave(bk, 1)[:, :k]
    return (w8.float() * s).to(torch.bfloat16)


def mtp_key(key: str, layer: int) -> Optional[str]:
    """Name of a tensor of the full checkpoint inside the exported draft model (None: not part of the MTP block)."""
    prefix = f"model.layers.{layer}"
    if not key.startswith(prefix + "."):
        return None
    if any(s in key for s in MODEL_LEVEL):
        return "model" + key[len(prefix):]
    return "model.layers.0" + key[len(prefix):]


def export(input_dir: str, output_dir: str, model_type: Optional[str] = None) -> Dict[str, torch.Tensor]:
    with open(os.path.join(input_dir, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    mt = (model_type or detect_model_type(cfg)).lower()
    if mt not in MTP_TYPES:
        raise ValueError(f"unsupported model type for MTP export: {mt}")
    if "num_nextn_predict_layers" not in cfg:
        raise ValueError("config.json has no 'num_nextn_predict_layers': this model has no MTP block")
    if int(cfg["num_nextn_predict_layers"]) != 1:
        raise ValueError(f"only one MTP layer is supported, found {cfg['num_nextn_predict_layers']}")
    layer = int(cfg["num_hidden_layers"])
    os.makedirs(output_dir, exist_ok=True)
    for name in os.listdir(input_dir):
        src = os.path.join(input_dir, name)
        if os.path.isfile(src) and not name.endswith(".safetensors"):
            shutil.copy2(src, os.path.join(output_dir, name))
    new_cfg = dict(cfg)
    new_cfg.update(num_hidden_layers=1, architectures=[MTP_TYPES[mt][1]], model_type=MTP_TYPES[mt][0], quantization_config="")
    if mt.startswith("deepseek"):
        new_cfg["first_k_dense_replace"] = 0
    with open(os.path.join(output_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(new_cfg, f, indent=2, ensure_ascii=False, sort_keys=True)
    ck = CheckpointReader(input_dir)
    raw: Dict[str, torch.Tensor] = {}
    for key in ck.keys():
        nk = mtp_key(key, layer)
        if nk is not None:
            raw[nk] = ck.get(key)
    if not raw:
        raise ValueError(f"no MTP parameters found at layer {layer}")
    params: Dict[str, torch.Tensor] = {}
    for key, t in raw.items():
        if key.endswith("weight_scale_inv"):
            continue
        sk = key[:-len("weight")] + "weight_scale_inv" if key.endswith(".weight") else None
        if sk is not None and sk in raw and mt.startswith("deepseek"):
            params[key] = block_dequant(t, raw[sk])
        else:
            params[key] = t
    save_safetensors(os.path.join(output_dir, "mtp_layer_parameters.safetensors"), params)
    with open(os.path.join(output_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {k: "mtp_layer_parameters.safetensors" for k in params}}, f, indent=4)
    return params


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="export the MTP block of a checkpoint as a draft model directory")
    ap.add_argument("--input-dir", required=True, help="HuggingFace model directory")
    ap.add_argument("--output-dir", required=True, help="draft model directory to create")
    ap.add_argument("--model-type", default=None, help="deepseek_v3 (V3, R1) | deepseek_v32 | glm4_moe; detected when omitted")
    ns = ap.parse_args(argv)
    params = export(ns.input_dir, ns.output_dir, ns.model_type)
    print(f"exported {len(params)} tensors to {ns.output_dir}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
