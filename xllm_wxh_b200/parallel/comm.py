"""Parallel context of one rank: tensor/expert/data-parallel group layout and the collectives the
model code calls.

Group layout follows the reference (xllm/core/framework/parallel_state/collective_communicator.cpp:
119-219, process_group.cpp:31-77): world = dp_size x tp_size with TP ranks contiguous; the MoE
expert-parallel group spans the world (ep_size ranks, strided when moe_tp > 1).

Three implementations exist for the row-parallel "GEMM -> reduce -> +residual -> RMSNorm" step:
  * tp_size == 1: plain kernels;
  * `nccl`: GEMM, NCCL all-reduce, add+RMSNorm kernel (what the reference does: linear.cpp:822-825) —
    kept as the baseline and as the oracle;
  * `fused`: the sm_100a kernels in `parallel/fused_tp.py` that push partial tiles to the owner rank over
    NVLink from inside the GEMM epilogue and reduce + normalise + all-gather in one pass.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops


@dataclasses.dataclass
class ParallelConfig:
    world_size: int = 1
    rank: int = 0
    dp_size: int = 1
    ep_size: int = 1
    tp_mode: str = "fused"          # fused | nccl
    ep_mode: str = "fused"          # fused (all-to-all kernels) | nccl | allreduce (EP level 1)
    mlp_replicated: bool = False    # every TP rank holds the whole dense MLP (row-sharded MLP for long steps)
    moe_experts_over_tp: bool = False  # no expert-parallel group: the routed experts are dealt out over the TP ranks

    @property
    def tp_size(self) -> int:
        return self.world_size // self.dp_size

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def dp_rank(self) -> int:
        return self.rank // self.tp_size

    @property
    def ep_rank(self) -> int:
        return self.rank % self.ep_size if self.ep_size > 1 else 0

    def expert_shard(self) -> Tuple[int, int]:
        """(index, count) of this rank's share of the routed experts: its place in the expert-parallel group, else (when
        `moe_experts_over_tp`) in the tensor-parallel group, whose reduction then also sums the experts' outputs."""
        if self.ep_size > 1:
            return self.ep_rank, self.ep_size
        if self.moe_experts_over_tp and self.tp_size > 1:
            return self.tp_rank, self.tp_size
        return 0, 1


class Comm:
    """Single-rank default: every collective is the identity."""

    def __init__(self, cfg: Optional[ParallelConfig] = None):
        self.cfg = cfg or ParallelConfig()
        self.tp_group = None
        self.dp_group = None
        self.ep_group = None
        self.world_group = None
        self.fused_tp = None
        self.fused_ep = None

    # --- layout
    @property
    def tp_size(self): return self.cfg.tp_size
    @property
    def tp_rank(self): return self.cfg.tp_rank
    @property
    def ep_size(self): return self.cfg.ep_size
    @property
    def ep_rank(self): return self.cfg.ep_rank
    @property
    def dp_size(self): return self.cfg.dp_size
    @property
    def dp_rank(self): return self.cfg.dp_rank
    @property
    def rank(self): return self.cfg.rank
    @property
    def world_size(self): return self.cfg.world_size

    # --- collectives (reference: parallel_state.cpp:89-263)
    def all_reduce(self, x: torch.Tensor, group=None) -> torch.Tensor:
        g = group if group is not None else self.tp_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        dist.all_reduce(x, group=g)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1, group=None) -> torch.Tensor:
        g = group if group is not None else self.tp_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        n = dist.get_world_size(g)
        flat = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x.contiguous(), group=g)
        if dim == 0:
            return flat
        out = flat.view((n,) + tuple(x.shape))
        return torch.cat(list(out.unbind(0)), dim=dim)

    def reduce_scatter(self, x: torch.Tensor, group=None) -> torch.Tensor:
        """Row-wise reduce-scatter with padding to a multiple of the group size (parallel_state.cpp:188-240)."""
        g = group if group is not None else self.tp_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        n = dist.get_world_size(g)
        T = x.shape[0]
        pad = (-T) % n
        if pad:
            x = torch.cat([x, x.new_zeros((pad,) + tuple(x.shape[1:]))], 0)
        out = x.new_empty((x.shape[0] // n,) + tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out, x.contiguous(), group=g)
        return out

    def gather_tokens(self, x: torch.Tensor, counts: List[int], group=None) -> torch.Tensor:
        """Variable-length all-gather: pad to max, gather, compact (parallel_state.cpp:104-125)."""
        g = group if group is not None else self.dp_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        m = max(counts)
        xp = x
        if x.shape[0] < m:
            xp = torch.cat([x, x.new_zeros((m - x.shape[0],) + tuple(x.shape[1:]))], 0)
        flat = torch.empty((len(counts) * m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, xp.contiguous(), group=g)
        out = flat.view((len(counts), m) + tuple(x.shape[1:]))
        return torch.cat([out[i, :c] for i, c in enumerate(counts)], 0)

    # --- the row-parallel hot step (K1 of the kernel plan)
    def row_linear_add_rms_norm(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor,
                                eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """y = all_reduce(x @ w.T); residual' = y + residual; return (RMSNorm(residual'), residual')."""
        if self.tp_size == 1:
            y = ops.linear(x, w)
            return ops.add_rms_norm(y, residual, norm_w, eps)
        if self.fused_tp is not None and x.is_cuda:
            return self.fused_tp.row_linear_add_rms_norm(x, w, residual, norm_w, eps)
        y = ops.linear(x, w)
        y = self.all_reduce(y)
        return ops.add_rms_norm(y, residual, norm_w, eps)

    def partial_add_rms_norm(self, y: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor,
                             eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """`y`: this rank's partial sum of a row-parallel step (any producer).  Same result as
        `row_linear_add_rms_norm` from the GEMM output on."""
        if self.tp_size > 1:
            ft = self.fused_tp
            if ft is not None and y.is_cuda and ft.mode != "push" and y.dtype == torch.bfloat16:
                return ft.partial_add_rms_norm(y, residual, norm_w, eps)
            y = self.all_reduce(y)
        return ops.add_rms_norm(y, residual, norm_w, eps)

    def init_residual(self, x: torch.Tensor) -> torch.Tensor:
        """Residual stream at the first layer.  The fused TP path keeps only this rank's row shard of it."""
        if self.tp_size > 1 and self.fused_tp is not None and x.is_cuda:
            return self.fused_tp.init_residual(x)
        return x

    def row_linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        y = ops.linear(x, w)
        return self.all_reduce(y) if self.tp_size > 1 else y

    def barrier(self):
        if self.world_group is not None:
            dist.barrier(group=self.world_group)


def init_comm(cfg: ParallelConfig, device: torch.device) -> Comm:
    """Create the process groups on an already-initialised default group."""
    c = Comm(cfg)
    if cfg.world_size == 1:
        return c
    assert dist.is_initialized(), "torch.distributed must be initialised before init_comm"
    c.world_group = dist.group.WORLD
    tp, dp = cfg.tp_size, cfg.dp_size
    # every rank must create every group, in the same order
    for d in range(dp):
        ranks = list(range(d * tp, (d + 1) * tp))
        g = dist.new_group(ranks) if tp > 1 and dp > 1 else (dist.group.WORLD if tp > 1 else None)
        if cfg.dp_rank == d:
            c.tp_group = g
    if dp > 1:
        for t in range(tp):
            ranks = list(range(t, cfg.world_size, tp))
            g = dist.new_group(ranks) if tp > 1 else dist.group.WORLD
            if cfg.tp_rank == t:
                c.dp_group = g
    if cfg.ep_size > 1:
        c.ep_group = dist.group.WORLD if cfg.ep_size == cfg.world_size else dist.new_group(list(range(cfg.ep_size)))
    return c
