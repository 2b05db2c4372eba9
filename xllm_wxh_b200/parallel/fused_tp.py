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


class MulticastBuffer:
    """Same-size allocation on every rank of a process group, bound to one NVLink multicast object: `ptrs` are the plain
    (unicast) addresses of every rank's copy as mapped into this process, `mc_ptr` is the multicast address, on which
    `multimem.ld_reduce` reads the sum over all copies and `multimem.st` writes all of them (the NVSwitch does the work).
    Allocation, handle exchange and mapping are torch's symmetric-memory allocator; the kernels are this package's."""

    def __init__(self, nbytes: int, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem
        self.nbytes = nbytes
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, group=group.group_name if group is not None else dist.group.WORLD.group_name)
        self.mc_ptr = int(self.handle.multicast_ptr or 0)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.local_ptr = self.local.data_ptr()
        self.ptr_array = (ctypes.c_void_p * len(self.ptrs))(*self.ptrs)

    def offset_array(self, byte_offset: int):
        return (ctypes.c_void_p * len(self.ptrs))(*[p + byte_offset for p in self.ptrs])


def nvls_wanted() -> bool:
    """`XLLM_TP_NVLS=0` keeps the fused paths on plain peer loads and stores (tests in which a rank exits on purpose run
    that way: a rank that dies while its memory is bound to a multicast object disturbs the other GPUs)."""
    import os
    return os.environ.get("XLLM_TP_NVLS", "1") != "0" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"


class FusedTP:
    def __init__(self, comm, hidden: int, max_tokens: int, device: torch.device, timeout_s: float = 2.0, mode: str = "pull"):
        self.comm, self.H, self.device = comm, hidden, device
        self.tp, self.rank = comm.tp_size, comm.tp_rank
        group = list(range(comm.dp_rank * self.tp, (comm.dp_rank + 1) * self.tp))
        self.T_cap = max_tokens
        self.shard_cap = (max_tokens + self.tp - 1) // self.tp
        es = 2
        # steps of at least this many rows run a replicated MLP on each rank's own rows (about 96 rows per rank)
        self.mlp_rows_min_tokens = int(__import__("os").environ.get("XLLM_TP_MLP_ROWS_MIN_TOKENS", str(96 * self.tp)))
        self.launches = 0                   # fused reduce steps issued (tests read it)
        self.mode = mode                    # "nvls": in-switch reduction and broadcast; "pull": partials stay local and owners fetch them; "push": epilogue peer stores
        self.timeout_s = timeout_s
        if mode == "nvls":
            try:
                if self._init_nvls(comm, hidden, device):
                    return
            except Exception as e:          # no multicast support for this group: plain peer memory instead
                import sys
                sys.stderr.write(f"fused TP: NVLS unavailable ({e!r}); using peer loads\n")
            self.mode = mode = "pull"
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
        dist.barrier()

    def _init_nvls(self, comm, hidden: int, device: torch.device) -> bool:
        """One multicast-bound allocation: [partial results | gathered activations | flags]."""
        row_bytes = hidden * 2
        data = ((self.T_cap * row_bytes + 1023) // 1024) * 1024
        buf = MulticastBuffer(2 * data + 4096, comm.tp_group, device)
        ok = torch.tensor([1 if buf.mc_ptr else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=comm.tp_group)
        if int(ok.item()) == 0:
            return False
        self.mc = buf
        self.partial_ptr, self.mc_partial = buf.local_ptr, buf.mc_ptr
        self.mc_gathered = buf.mc_ptr + data
        self.gathered_t = buf.local[data:data + self.T_cap * row_bytes].view(torch.bfloat16).view(self.T_cap, hidden)
        sync0 = 2 * data                     # ints: [0:8) gemm flags, 16/17 counters, 18 epoch, [32:48) gather arrival counters
        self.flags_in = buf.offset_array(sync0)
        self.flags_local = c_void_p(buf.local_ptr + sync0)
        self.gather_flags = buf.offset_array(sync0 + 32 * 4)
        self.done_gemm = c_void_p(buf.local_ptr + sync0 + 16 * 4)
        self.done_reduce = c_void_p(buf.local_ptr + sync0 + 17 * 4)
        self.epoch = c_void_p(buf.local_ptr + sync0 + 18 * 4)
        # second set of words for the all-gather that runs apart from a reduction (`add_norm_gather`)
        self.gather2_flags = buf.offset_array(sync0 + (64 + 32) * 4)
        self.done_gather2 = c_void_p(buf.local_ptr + sync0 + (64 + 17) * 4)
        self.epoch_gather2 = c_void_p(buf.local_ptr + sync0 + (64 + 18) * 4)
        torch.cuda.synchronize(device)
        dist.barrier(group=comm.tp_group)
        return True

    def shard_of(self, T: int) -> Tuple[int, int]:
        shard = (T + self.tp - 1) // self.tp
        rows = max(0, min(shard, T - self.rank * shard))
        return shard, rows

    def init_residual(self, x: torch.Tensor) -> torch.Tensor:
        shard, rows = self.shard_of(x.shape[0])
        return x[self.rank * shard:self.rank * shard + rows].contiguous()

    def gemm(self, x: torch.Tensor, w: torch.Tensor) -> None:
        """Row-parallel GEMM of this rank into its peer-visible partial buffer; the last CTA publishes the step's epoch to
        every rank ("nvls" and "pull" modes)."""
        T, K = x.shape
        H = w.shape[0]
        assert H == self.H and T <= self.T_cap and x.dtype == torch.bfloat16 and self.mode in ("nvls", "pull")
        if x.stride(-1) != 1:
            x = x.contiguous()
        dst = self.partial_ptr if self.mode == "nvls" else self.partial.local_ptr
        _check(lib().xl_gemm_bf16_publish(_ptr(x), _ptr(w), c_void_p(dst), c_int(T), c_int(H), c_int(K), c_int(x.stride(0)),
                                          c_int(w.stride(0)), c_int(H), self.flags_in, self.done_gemm, self.epoch, c_int(self.tp),
                                          c_int(self.rank), _stream()), "xl_gemm_bf16_publish")
        cuda_ops.launch_count += 1

    def reduce(self, T: int, residual: torch.Tensor, res_out: torch.Tensor, norm_w: torch.Tensor, eps: float) -> torch.Tensor:
        """Reduce-scatter of the partial results + residual + RMSNorm + all-gather; returns the normalised activation
        [T, H] (a view of this rank's gathered buffer).  `res_out` may be `residual` itself."""
        H = self.H
        shard, rows = self.shard_of(T)
        L = lib()
        self.launches += 1
        if self.mode == "nvls":
            _check(L.xl_tp_nvls_reduce_norm_gather(c_void_p(self.mc_partial), _ptr(residual), _ptr(res_out), _ptr(norm_w),
                                                   c_void_p(self.mc_gathered), self.flags_local, self.gather_flags,
                                                   self.done_reduce, self.epoch, c_int(self.tp), c_int(self.rank), c_int(shard),
                                                   c_int(rows), c_int(T), c_int(H), ctypes.c_float(eps),
                                                   ctypes.c_double(self.timeout_s), _stream()), "xl_tp_nvls_reduce_norm_gather")
        else:
            _check(L.xl_tp_pull_reduce_norm_gather(self.partial.ptr_array, _ptr(residual), _ptr(res_out), _ptr(norm_w),
                                                   self.gathered.ptr_array, c_void_p(self.sync.local_ptr), self.gather_flags,
                                                   self.done_reduce, self.epoch, c_int(self.tp), c_int(self.rank), c_int(shard),
                                                   c_int(rows), c_int(T), c_int(H), ctypes.c_float(eps),
                                                   ctypes.c_double(self.timeout_s), _stream()), "xl_tp_pull_reduce_norm_gather")
        cuda_ops.launch_count += 1
        return self.gathered_t[:T]

    def row_linear_reduce_norm(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor,
                               eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """Row-parallel GEMM + reduce-scatter + residual + RMSNorm without the all-gather: returns the normalised rows
        this rank owns [rows, H] and its residual shard (NVLS mode)."""
        assert self.mode == "nvls"
        T = x.shape[0]
        H = self.H
        shard, rows = self.shard_of(T)
        self.gemm(x, w)
        out = torch.empty((rows, H), dtype=torch.bfloat16, device=x.device)
        res_out = torch.empty((rows, H), dtype=torch.bfloat16, device=x.device)
        _check(lib().xl_tp_nvls_reduce_norm(c_void_p(self.mc_partial), _ptr(residual), _ptr(res_out), _ptr(norm_w), _ptr(out),
                                            self.flags_local, self.done_reduce, self.epoch, c_int(self.tp), c_int(self.rank),
                                            c_int(shard), c_int(rows), c_int(T), c_int(H), ctypes.c_float(eps),
                                            ctypes.c_double(self.timeout_s), _stream()), "xl_tp_nvls_reduce_norm")
        cuda_ops.launch_count += 1
        return out, res_out

    def add_norm_gather(self, y: torch.Tensor, T: int, residual: torch.Tensor, norm_w: torch.Tensor,
                        eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """`y` [rows, H]: rows of a T-row step that this rank computed whole.  residual' = y + residual; the normalised
        rows go to every rank (all-gather through the multicast address).  Returns ([T, H], residual')."""
        assert self.mode == "nvls"
        H = self.H
        shard, rows = self.shard_of(T)
        assert y.shape[0] == rows and y.is_contiguous()
        res_out = torch.empty((rows, H), dtype=torch.bfloat16, device=y.device)
        _check(lib().xl_tp_nvls_norm_gather(_ptr(y), _ptr(residual), _ptr(res_out), _ptr(norm_w), c_void_p(self.mc_gathered),
                                            self.gather2_flags, self.done_gather2, self.epoch_gather2, c_int(self.tp),
                                            c_int(self.rank), c_int(shard), c_int(rows), c_int(T), c_int(H), ctypes.c_float(eps),
                                            ctypes.c_double(self.timeout_s), _stream()), "xl_tp_nvls_norm_gather")
        cuda_ops.launch_count += 1
        return self.gathered_t[:T], res_out

    def partial_add_rms_norm(self, y: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor,
                             eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """`y` [T, H]: this rank's partial result of a row-parallel step computed by any kernel (fp8 GEMM, routed experts).
        Publishes it and runs the fused reduce + residual + RMSNorm + all-gather; same return as `row_linear_add_rms_norm`."""
        T, H = y.shape
        assert H == self.H and T <= self.T_cap and y.dtype == torch.bfloat16 and self.mode in ("nvls", "pull")
        if y.stride(-1) != 1:
            y = y.contiguous()
        shard, rows = self.shard_of(T)
        dst = self.partial_ptr if self.mode == "nvls" else self.partial.local_ptr
        _check(lib().xl_tp_publish_rows(_ptr(y), c_int(y.stride(0)), c_void_p(dst), c_int(T), c_int(H), self.flags_in,
                                        self.done_gemm, self.epoch, c_int(self.tp), c_int(self.rank), _stream()),
               "xl_tp_publish_rows")
        cuda_ops.launch_count += 1
        res_out = torch.empty((rows, H), dtype=torch.bfloat16, device=y.device)
        return self.reduce(T, residual, res_out, norm_w, eps), res_out

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
        if self.mode != "push":
            self.gemm(x, w)
            return self.reduce(T, residual, res_out, norm_w, eps), res_out
        _check(L.xl_gemm_bf16_rs_push(_ptr(x), _ptr(w), c_int(T), c_int(H), c_int(K), c_int(x.stride(0)), c_int(w.stride(0)),
                                      self.recv.ptr_array, self.flags_in, self.done_gemm, self.epoch, c_int(self.tp),
                                      c_int(self.rank), c_int(shard), c_int(self.shard_cap), _stream()), "xl_gemm_bf16_rs_push")
        _check(L.xl_tp_reduce_norm_gather(c_void_p(self.recv.local_ptr), _ptr(residual), _ptr(res_out), _ptr(norm_w),
                                          self.gathered.ptr_array, c_void_p(self.sync.local_ptr), self.gather_flags,
                                          self.done_reduce, self.epoch, c_int(self.tp), c_int(self.rank), c_int(shard),
                                          c_int(self.shard_cap), c_int(rows), c_int(T), c_int(H), ctypes.c_float(eps),
                                          ctypes.c_double(self.timeout_s), _stream()), "xl_tp_reduce_norm_gather")
        cuda_ops.launch_count += 2
        return self.gathered_t[:T], res_out


def attach(engine) -> None:
    """Give the engine's Comm a FusedTP when tensor parallelism is on and the fused backend is selected."""
    comm = engine.comm
    if comm.tp_size not in (2, 4, 8) or comm.cfg.tp_mode != "fused":
        return          # other group sizes use the NCCL path
    import os
    # measured on B200s: with two ranks the switch reduction moves as many bytes as peer loads and is a little slower
    # (15.7 against 15.4 ms per bench step); from four ranks on it wins (10.9 against 11.4 ms)
    mode = os.environ.get("XLLM_TP_FUSED_MODE", "nvls" if nvls_wanted() and comm.tp_size >= 4 else "pull")
    comm.fused_tp = FusedTP(comm, engine.args.hidden_size, engine.opt.max_tokens_per_batch + 16, engine.device, mode=mode)
