"""MoE on the GPU: router kernel, expert sort, grouped tcgen05 GEMMs, weighted combine.

Single-rank flow (the expert-parallel flows in `parallel/fused_ep.py` reuse the same pieces):
    router -> sort expanded (token, slot) pairs by expert (+ 128-row tile table) -> gather rows
           -> grouped GEMM w13 (+SwiGLU epilogue when the weights are interleaved) -> grouped GEMM w2 -> combine.
Everything the grouped GEMM needs about the routing (tile table, tile count) stays on the device, so the sequence can be
captured in a CUDA graph.

Reference flow: FusedMoE on MLU (xllm/core/layers/mlu/fused_moe.cpp:349-455: gate -> gen_idx -> expand -> group_gemm ->
act -> group_gemm -> combine).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import cuda_ops
from .cuda_ops import _check, _ptr, _stream, c_float, c_int, c_void_p, lib


def moe_router(logits: torch.Tensor, top_k: int, scoring: str = "softmax", renorm: bool = True,
               bias: Optional[torch.Tensor] = None, n_group: int = 1, topk_group: int = 1, route_scale: float = 1.0,
               load_hist: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    T, E = logits.shape
    assert logits.is_contiguous() and logits.dtype in (torch.float32, torch.bfloat16)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    _check(lib().xl_moe_router(_ptr(logits), c_int(0 if logits.dtype == torch.float32 else 1), _ptr(bias), _ptr(w), _ptr(ids),
                               _ptr(load_hist), c_int(T), c_int(E), c_int(top_k), c_int(int(scoring == "sigmoid")),
                               c_int(int(renorm)), c_int(n_group), c_int(topk_group), c_float(route_scale), _stream()),
           "xl_moe_router")
    cuda_ops.launch_count += 1
    return w, ids


class SortedRouting:
    """Device-side result of the expert sort for `n` (token, slot) pairs."""
    __slots__ = ("work", "sorted_src", "dst_of", "E_local", "max_tiles", "n")

    def __init__(self, work, sorted_src, dst_of, E_local, max_tiles, n):
        self.work, self.sorted_src, self.dst_of, self.E_local, self.max_tiles, self.n = work, sorted_src, dst_of, E_local, max_tiles, n

    @property
    def counts(self): return self.work[:self.E_local]
    @property
    def offsets(self): return self.work[self.E_local:2 * self.E_local + 1]
    @property
    def total_rows(self): return self.work[2 * self.E_local:2 * self.E_local + 1]
    @property
    def num_m_tiles(self): return self.work[3 * self.E_local + 1:3 * self.E_local + 2]
    @property
    def tile_expert(self): return self.work[3 * self.E_local + 2:3 * self.E_local + 2 + self.max_tiles]
    @property
    def tile_row0(self): return self.work[3 * self.E_local + 2 + self.max_tiles:3 * self.E_local + 2 + 2 * self.max_tiles]
    @property
    def tile_row_end(self): return self.work[3 * self.E_local + 2 + 2 * self.max_tiles:3 * self.E_local + 2 + 3 * self.max_tiles]


def moe_sort(ids: torch.Tensor, expert_offset: int, E_local: int, max_rows: Optional[int] = None) -> SortedRouting:
    """`max_rows` bounds how many of the `ids` can be local experts (default: all of them); it sizes the tile table."""
    n = ids.numel()
    rows = n if max_rows is None else min(n, max_rows)
    max_tiles = (rows + 127) // 128 + E_local
    work = torch.empty(3 * E_local + 3 * max_tiles + 8, dtype=torch.int32, device=ids.device)
    sorted_src = torch.empty(max(rows, 1), dtype=torch.int32, device=ids.device)
    dst_of = torch.empty(max(n, 1), dtype=torch.int32, device=ids.device)
    _check(lib().xl_moe_sort(_ptr(ids), c_int(n), c_int(expert_offset), c_int(E_local), _ptr(work), c_int(max_tiles),
                             _ptr(sorted_src), _ptr(dst_of), _stream()), "xl_moe_sort")
    cuda_ops.launch_count += 3
    return SortedRouting(work, sorted_src, dst_of, E_local, max_tiles, rows)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, r, swiglu: bool = False, out: Optional[torch.Tensor] = None,
                 c_rows_per_expert: int = 0, c_col_stride: int = 0) -> torch.Tensor:
    """a [R_cap, K] rows sorted by expert; w [E_local, N, K]; returns [R_cap, N] (or [R_cap, N/2] with the SwiGLU epilogue).
    `r` provides the device-side tile table (`tile_expert`, `tile_row0`, `tile_row_end`, `num_m_tiles`, `max_tiles`).
    With `out` given, row `row - expert * c_rows_per_expert` / column offset `expert * c_col_stride` place each tile."""
    R_cap, K = a.shape
    E, N, K2 = w.shape
    assert K == K2 and w.is_contiguous() and a.stride(-1) == 1
    if out is None:
        out = torch.empty((R_cap, N // 2 if swiglu else N), dtype=torch.bfloat16, device=a.device)
    _check(lib().xl_grouped_gemm_bf16(_ptr(a), _ptr(w), _ptr(out), c_int(R_cap), c_int(N), c_int(K), c_int(a.stride(0)),
                                      c_int(out.stride(0)), c_int(E), _ptr(r.tile_expert), _ptr(r.tile_row0), _ptr(r.tile_row_end),
                                      _ptr(r.num_m_tiles), c_int(r.max_tiles), c_int(int(swiglu)), c_int(c_rows_per_expert),
                                      c_int(c_col_stride), _stream()),
           "xl_grouped_gemm_bf16")
    cuda_ops.launch_count += 1
    return out


def gather_rows(x: torch.Tensor, r: SortedRouting, k: int) -> torch.Tensor:
    T, H = x.shape
    out = torch.empty((max(r.n, 1), H), dtype=x.dtype, device=x.device)
    _check(lib().xl_moe_gather_rows(_ptr(x), _ptr(r.sorted_src), _ptr(r.total_rows), _ptr(out), c_int(H), c_int(k),
                                    c_int(x.stride(0)), c_int(r.n), _stream()), "xl_moe_gather_rows")
    cuda_ops.launch_count += 1
    return out


def combine(y: torch.Tensor, r: SortedRouting, weights: torch.Tensor, T: int, add: Optional[torch.Tensor] = None) -> torch.Tensor:
    H = y.shape[1]
    k = weights.shape[1]
    out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
    _check(lib().xl_moe_combine(_ptr(y), _ptr(r.dst_of), _ptr(weights), _ptr(add), _ptr(out), c_int(T), c_int(H), c_int(k),
                                _stream()), "xl_moe_combine")
    cuda_ops.launch_count += 1
    return out


def interleave_w13(w13: torch.Tensor) -> torch.Tensor:
    """[E, 2I, H] (gate rows then up rows per expert) -> per expert rows interleaved in groups of 16, in place."""
    E, I2, H = w13.shape
    I = I2 // 2
    assert I % 16 == 0
    for e in range(E):
        w13[e].copy_(cuda_ops.interleave_gate_up(w13[e]))
    return w13


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor,
                expert_offset: int = 0, interleaved: bool = False, add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sum_k w_k * expert_k(x) over the experts held locally ([expert_offset, expert_offset + E_local))."""
    T, H = x.shape
    k = ids.shape[1]
    r = moe_sort(ids, expert_offset, w13.shape[0])
    xs = gather_rows(x, r, k)
    if interleaved:
        h = grouped_gemm(xs, w13, r, swiglu=True)
    else:
        h = cuda_ops.silu_and_mul(grouped_gemm(xs, w13, r))
    y = grouped_gemm(h, w2, r)
    return combine(y, r, weights, T, add)
