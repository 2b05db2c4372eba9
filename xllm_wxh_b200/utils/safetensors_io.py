"""HF checkpoint access: a directory of `*.safetensors` files read through the C++ mmap reader, plus a
small writer used by tests and by the MTP export tool.

Reference: xllm/core/framework/hf_model_loader.cpp (file enumeration), state_dict/state_dict.cpp:122-262
(zero-copy tensors, prefix views, sharded loads)."""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

from .. import _core

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
    "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class CheckpointReader:
    """All tensors of a model directory; tensors are zero-copy views into the mapped files."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {model_dir}")
        self.files = [_core.SafeTensorsFile(os.path.join(model_dir, f)) for f in files]
        self.index: Dict[str, int] = {}
        for i, f in enumerate(self.files):
            for k in f.keys():
                self.index[k] = i
        self.total_bytes = sum(f.data_size for f in self.files)

    def keys(self) -> List[str]:
        return list(self.index.keys())

    def has(self, name: str) -> bool:
        return name in self.index

    def get(self, name: str) -> torch.Tensor:
        f = self.files[self.index[name]]
        info = f.info(name)
        raw = f.view(name)                     # numpy uint8, keeps the file alive
        t = torch.from_numpy(raw)
        dt = _DTYPES[info.dtype]
        return t.view(dt).reshape(list(info.shape)) if info.shape else t.view(dt).reshape(())

    def get_or_none(self, name: str) -> Optional[torch.Tensor]:
        return self.get(name) if name in self.index else None

    def items(self, prefix: str = "") -> Iterator[Tuple[str, torch.Tensor]]:
        for k in self.index:
            if k.startswith(prefix):
                yield k, self.get(k)


class DequantizingReader:
    """View of a checkpoint in which fp8 weights come back dequantised (bf16): `X.weight` stored as e4m3 with either
    `X.weight_scale_inv` (one fp32 scale per 128 x 128 block, the DeepSeek-V3 / Qwen3-FP8 layout) or `X.weight_scale`
    (per tensor or per output channel, the reference's w8a8 fp8 mode: layers/common/linear.cpp:65-99,134-179, where fused
    shards are re-quantised to a common scale; dequantising first needs no common scale).  Models whose GEMMs run in bf16
    load fp8 checkpoints through it; `input_scale` tensors (static activation scales) are not needed then."""

    def __init__(self, ckpt, block=(128, 128)):
        self.ckpt, self.block = ckpt, block

    def has(self, name: str) -> bool:
        return self.ckpt.has(name)

    def keys(self):
        return self.ckpt.keys()

    def get_or_none(self, name: str):
        return self.get(name) if self.ckpt.has(name) else None

    def get(self, name: str) -> torch.Tensor:
        t = self.ckpt.get(name)
        if t.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2) or not name.endswith(".weight"):
            return t
        base = name[:-len("weight")]
        if self.ckpt.has(base + "weight_scale_inv"):
            s = self.ckpt.get(base + "weight_scale_inv").float()
            bn, bk = self.block
            n, k = t.shape
            if s.shape != ((n + bn - 1) // bn, (k + bk - 1) // bk):
                raise ValueError(f"{name}: block scales {tuple(s.shape)} do not fit a {tuple(t.shape)} weight")
            s = s.repeat_interleave(bn, 0)[:n].repeat_interleave(bk, 1)[:, :k]
            return (t.float() * s).to(torch.bfloat16)
        if self.ckpt.has(base + "weight_scale"):
            s = self.ckpt.get(base + "weight_scale").float()
            if s.numel() == 1:
                s = s.reshape(())
            elif s.numel() == t.shape[0]:
                s = s.reshape(-1, 1)
            else:
                raise ValueError(f"{name}: weight_scale of shape {tuple(s.shape)} is neither per tensor nor per channel")
            return (t.float() * s).to(torch.bfloat16)
        raise ValueError(f"{name} is fp8 but the checkpoint has neither weight_scale_inv nor weight_scale for it")


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        b = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
