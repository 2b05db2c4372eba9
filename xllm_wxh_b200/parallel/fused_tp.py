"""Fused tensor-parallel row-parallel step over NVLink peer memory.

    y = x @ W_shard^T            (partials of every rank)
    residual' = sum_ranks(y) + residual ;  h = RMSNorm(residual')

implemented as two kernels that carry the collective themselves (no NCCL call on this path):
  1. `xl_gemm_bf16_publish`   : tcgen05 GEMM into this rank's peer-mapped partial buffer; its last CTA publishes a
                                completion flag to every rank (`xl_gemm_bf16_rs_push` is the older variant whose
                                epilogue stores each row into the owner's receive buffer);
  2. `xl_tp_pull_reduce_norm_gather`: the owner fetches the partials of its rows from all ranks with coalesced peer
                                loads (reduce-scatter), adds its residual shard, normalises, and stores the
                                normalised rows into every rank's activation buffer (all-gather by peer stores).
The residual stream stays sharded by rows across the TP group.  Buffers are `cudaMalloc`ed once and shared with
`cudaIpc*` handles exchanged through `torch.distributed`.

This replaces the reference's `RowParallelLinear` all-reduce + `fused_add_rms_norm` pair
(xllm/core/layers/common/linear.cpp:822-825, kernels/cuda/norm.cu:78-172).
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

import torch
import torch.distributed as dist

from ..ops import cuda_ops
from ..ops.cuda_ops import _check, _ptr, _stream, c_int, c_void_p, lib


class _CudaBuffer:
    """A raw device allocation exposed to torch through `__cuda_array_interface__`."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}

    def tensor(self, device) -> torch.Tensor:
        return torch.as_tensor(self, device=device)


class SymmetricBuffer:
    """Same-size allocation on every rank of `group_ranks`, each rank holding pointers to all of them."""

    def __init__(self, nbytes: int, rank: int, group_ranks: List[int], device: torch.device):
        L = lib()
        L.xl_dev_malloc.restype = ctypes.c_void_p
        L.xl_ipc_open_handle.restype = ctypes.c_void_p
        self.nbytes = nbytes
        self.local_ptr = L.xl_dev_malloc(ctypes.c_long(nbytes))
        if not self.local_ptr:
            raise RuntimeError(f"cudaMalloc of {nbytes} bytes failed")
        handle = (ctypes.c_char * 64)()
        if L.xl_ipc_get_handle(c_void_p(self.local_ptr), handle) != 64:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        gathered: List[bytes] = [b""] * dist.get_world_size()
        dist.all_gather_object(gathered, (rank, bytes(handle)))
        by_rank = {r: h for r, h in gathered}
        self.ptrs: List[int] = []
        for r in group_ranks:
            if r == rank:
                self.ptrs.append(self.local_ptr)
            else:
                p = L.xl_ipc_open_handle((ctypes.c_char * 64).from_buffer_copy(by_rank[r][:64]))
                if not p:
                    raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {r} (peer access unavailable?)")
                self.ptrs.append(p)
        self.local = _CudaBuffer(self.local_ptr, nbytes).tensor(device)
        self.ptr_array = (ctypes.c_void_p * len(self.ptrs))(*self.ptrs)

    def offset_array(self, byte_offset: int):
        return (ctypes.c_void_p * len(self.ptrs))(*[p + byte_offset for p in self.ptrs])


class FusedTP:
    def __init__(self, comm, hidden: int, max_tokens: int, device: torch.device, timeout_s: float = 2.0, mode: str = "pull"):
        self.comm, self.H, self.device = comm, hidden, device
        self.tp, self.rank = comm.tp_size, comm.tp_rank
        group = list(range(comm.dp_rank * self.tp, (comm.dp_rank + 1) * self.tp))
        self.T_cap = max_tokens
        self.shard_cap = (max_tokens + self.tp - 1) // self.tp
        es = 2
        self.mode = mode                    # "pull": partials stay local and owners fetch them; "push": epilogue peer stores
        if mode == "push":
            self.recv = SymmetricBuffer(self.tp * self.shard_cap * hidden * es, comm.rank, group, device)
        else:
            self.partial = SymmetricBuffer(self.T_cap * hidden * es, comm.rank, group, device)
            self.partial_t = self.partial.local.view(torch.bfloat16).view(self.T_cap, hidden)
        self.gathered = SymmetricBuffer(self.T_cap * hidden * es, comm.rank, group, device)
        self.sync = SymmetricBuffer(256 * 4, comm.rank, group, device)   # ints: [0:8) gemm flags, 16/17 counters, 18 epoch, [32:48) gather arrival counters [parity][rank]
        self.flags_in = self.sync.offset_array(0)
        self.gather_flags = self.sync.offset_array(32 * 4)
        self.done_gemm = c_void_p(self.sync.local_ptr + 16 * 4)
        self.done_reduce = c_void_p(self.sync.local_ptr + 17 * 4)
        self.epoch = c_void_p(self.sync.local_ptr + 18 * 4)
        self.gathered_t = self.gathered.local.view(torch.bfloat16).view(self.T_cap, hidden)
        self.timeout_s = timeout_s
        dist.barrier()

    def shard_of(self, T: int) -> Tuple[int, int]:
        shard = (T + self.tp - 1) // self.tp
        rows = max(0, min(shard, T - self.rank * shard))
        return shard, rows

    def init_residual(self, x: torch.Tensor) -> torch.Tensor:
        shard, rows = self.shard_of(x.shape[0])
        return x[self.rank * shard:self.rank * shard + rows].contiguous()

    def row_linear_add_rms_norm(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor,
                                eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
        T, K = x.shape
        H = w.shape[0]
        assert H == self.H and T <= self.T_cap and x.dtype == torch.bfloat16
        if x.stride(-1) != 1:
            x = x.contiguous()
        shard, rows = self.shard_of(T)
        L = lib()
        res_out = torch.empty((rows, H), dtype=torch.bfloat16, device=x.device)
        if self.mode == "push":
            _check(L.xl_gemm_bf16_rs_push(_ptr(x), _ptr(w), c_int(T), c_int(H), c_int(K), c_int(x.stride(0)), c_int(w.stride(0)),
                                          self.recv.ptr_array, self.flags_in, self.done_gemm, self.epoch, c_int(self.tp),
                                          c_int(self.rank), c_int(shard), c_int(self.shard_cap), _stream()), "xl_gemm_bf16_rs_push")
            _check(L.xl_tp_reduce_norm_gather(c_void_p(self.recv.local_ptr), _ptr(residual), _ptr(res_out), _ptr(norm_w),
                                              self.gathered.ptr_array, c_void_p(self.sync.local_ptr), self.gather_flags,
                                              self.done_reduce, self.epoch, c_int(self.tp), c_int(self.rank), c_int(shard),
                                              c_int(self.shard_cap), c_int(rows), c_int(T), c_int(H), ctypes.c_float(eps),
                                              ctypes.c_double(self.timeout_s), _stream()), "xl_tp_reduce_norm_gather")
        else:
            _check(L.xl_gemm_bf16_publish(_ptr(x), _ptr(w), c_void_p(self.partial.local_ptr), c_int(T), c_int(H), c_int(K),
                                          c_int(x.stride(0)), c_int(w.stride(0)), c_int(H), self.flags_in, self.done_gemm,
                                          self.epoch, c_int(self.tp), c_int(self.rank), _stream()), "xl_gemm_bf16_publish")
            _check(L.xl_tp_pull_reduce_norm_gather(self.partial.ptr_array, _ptr(residual), _ptr(res_out), _ptr(norm_w),
                                                   self.gathered.ptr_array, c_void_p(self.sync.local_ptr), self.gather_flags,
                                                   self.done_reduce, self.epoch, c_int(self.tp), c_int(self.rank), c_int(shard),
                                                   c_int(rows), c_int(T), c_int(H), ctypes.c_float(eps),
                                                   ctypes.c_double(self.timeout_s), _stream()), "xl_tp_pull_reduce_norm_gather")
        cuda_ops.launch_count += 2
        return self.gathered_t[:T], res_out


def attach(engine) -> None:
    """Give the engine's Comm a FusedTP when tensor parallelism is on and the fused backend is selected."""
    comm = engine.comm
    if comm.tp_size not in (2, 4, 8) or comm.cfg.tp_mode != "fused":
        return          # other group sizes use the NCCL path
    import os
    comm.fused_tp = FusedTP(comm, engine.args.hidden_size, engine.opt.max_tokens_per_batch + 16, engine.device,
                            mode=os.environ.get("XLLM_TP_FUSED_MODE", "pull"))
