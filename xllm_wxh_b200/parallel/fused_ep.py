"""Expert parallelism: token dispatch / combine between the ranks that hold the experts.

Two implementations behind the same call `moe(h, mlp_weights, topk_weights, topk_ids, layer) -> [T, H]`:

* `FusedEP` (`--expert_parallel_degree 2`): the all-to-all is carried by our own kernels over NVLink peer memory
  (`csrc/cuda/ep_fused.cu`): rows are stored straight into the destination rank's receive buffer, sorted there by
  expert, run through the grouped tcgen05 GEMMs, and every output row is stored back into its source rank's return
  slot, where the top-k weighted sum reads local memory only.  No NCCL call on this path.
* `GatherEP` (default, the reference's "level 1", xllm/core/layers/common/dp_utils.cpp:109-205,
  fused_moe_base.cpp:101-136): all-gather the tokens of every attention-DP rank, compute the local experts on all of
  them, all-reduce, slice this rank's rows back.  Kept as the NCCL baseline and as the oracle for the fused path.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import cuda_ops, moe_cuda
from ..ops.cuda_ops import _check, _ptr, _stream, c_int, c_void_p, lib
from .fused_tp import SymmetricBuffer


class GatherEP:
    def __init__(self, comm, expert_offset: int):
        self.comm, self.e0 = comm, expert_offset
        self.dp_token_counts: Optional[List[int]] = None      # set per step by the worker

    def __call__(self, h, mlp, w, ids, layer_idx):
        from .. import ops
        c = self.comm
        counts = self.dp_token_counts
        if c.dp_size > 1 and counts is not None:
            g = c.world_group
            hh = c.gather_tokens(h, counts, group=g)
            ww = c.gather_tokens(w, counts, group=g)
            ii = c.gather_tokens(ids, counts, group=g)
            y = ops.moe_experts(hh, mlp.w13, mlp.w2, ww, ii, self.e0, mlp.interleaved)
            y = c.all_reduce(y, group=g)
            start = sum(counts[:c.dp_rank])
            return y[start:start + counts[c.dp_rank]]
        y = ops.moe_experts(h, mlp.w13, mlp.w2, w, ids, self.e0, mlp.interleaved)
        return c.all_reduce(y, group=c.ep_group)


class FusedEP:
    def __init__(self, comm, hidden: int, n_experts: int, top_k: int, max_tokens: int, device: torch.device,
                 timeout_s: float = 2.0):
        self.comm, self.H, self.k, self.device = comm, hidden, top_k, device
        self.R, self.rank = comm.ep_size, comm.ep_rank
        assert self.R == comm.world_size, "the fused all-to-all spans the whole world"
        self.E_local = n_experts // self.R
        self.T_cap = max_tokens
        self.per_token = min(top_k, self.E_local)
        self.cap = max_tokens * self.per_token                    # rows one source may send to one destination
        self.slots_cap = max_tokens * top_k
        group = list(range(self.R))
        self.recv_x = SymmetricBuffer(self.R * self.cap * hidden * 2, comm.rank, group, device)
        self.recv_meta = SymmetricBuffer(self.R * self.cap * 8, comm.rank, group, device)
        self.ret_y = SymmetricBuffer(self.slots_cap * hidden * 2, comm.rank, group, device)
        self.sync = SymmetricBuffer(256 * 4, comm.rank, group, device)   # ints: count[0:8) disp[8:16) ret[16:24) cursor[24:32) done[32:36) epoch[36]
        self.recv_count = self.sync.offset_array(0)
        self.disp_flags = self.sync.offset_array(8 * 4)
        self.ret_flags = self.sync.offset_array(16 * 4)
        base = self.sync.local_ptr
        self.send_cursor, self.done, self.epoch = c_void_p(base + 24 * 4), c_void_p(base + 32 * 4), c_void_p(base + 36 * 4)
        self.recv_x_t = self.recv_x.local.view(torch.bfloat16).view(self.R * self.cap, hidden)
        self.ret_y_t = self.ret_y.local.view(torch.bfloat16).view(self.slots_cap, hidden)
        self.timeout = ctypes.c_double(timeout_s)
        self.dp_token_counts: Optional[List[int]] = None
        self._identity = torch.arange(self.slots_cap, dtype=torch.int32, device=device)
        dist.barrier()

    def _peer_args(self):
        return (self.recv_x.ptr_array, self.recv_meta.ptr_array, self.recv_count, self.disp_flags, self.ret_y.ptr_array,
                self.ret_flags, self.send_cursor, self.done, self.epoch, c_int(self.R), c_int(self.rank), c_int(self.cap),
                c_int(self.H), c_int(self.E_local), self.timeout)

    def __call__(self, h, mlp, w, ids, layer_idx, add: Optional[torch.Tensor] = None):
        T, H = h.shape
        assert T <= self.T_cap and H == self.H
        L = lib()
        if h.stride(-1) != 1:
            h = h.contiguous()
        _check(L.xl_ep_dispatch_send(*self._peer_args(), _ptr(h), _ptr(ids), c_int(T), c_int(self.k), c_int(h.stride(0)),
                                     _stream()), "xl_ep_dispatch_send")
        n = self.R * self.cap
        ids_flat = torch.empty(n, dtype=torch.int32, device=h.device)
        base = self.sync.local_ptr
        _check(L.xl_ep_recv_prepare(c_void_p(self.recv_meta.local_ptr), c_void_p(base), c_void_p(base + 8 * 4), self.epoch,
                                    c_int(self.R), c_int(self.rank), c_int(self.cap), self.timeout, _ptr(ids_flat), _stream()),
               "xl_ep_recv_prepare")
        counts = self.dp_token_counts
        rows_bound = (sum(counts) if counts else self.R * self.T_cap) * self.per_token
        r = moe_cuda.moe_sort(ids_flat, 0, self.E_local, max_rows=max(rows_bound, 1))
        xs = moe_cuda.gather_rows(self.recv_x_t, r, 1)
        if mlp.interleaved:
            hmid = moe_cuda.grouped_gemm(xs, mlp.w13, r, swiglu=True)
        else:
            hmid = cuda_ops.silu_and_mul(moe_cuda.grouped_gemm(xs, mlp.w13, r))
        y = moe_cuda.grouped_gemm(hmid, mlp.w2, r)
        _check(L.xl_ep_return_send(*self._peer_args(), _ptr(y), _ptr(r.sorted_src), _ptr(r.total_rows),
                                   c_void_p(self.recv_meta.local_ptr), c_int(max(rows_bound, 1)), _stream()), "xl_ep_return_send")
        _check(L.xl_ep_combine_wait(c_void_p(base + 16 * 4), self.epoch, c_int(self.R), self.timeout, _stream()),
               "xl_ep_combine_wait")
        cuda_ops.launch_count += 4
        out = torch.empty((T, H), dtype=torch.bfloat16, device=h.device)
        _check(L.xl_moe_combine(_ptr(self.ret_y_t), _ptr(self._identity), _ptr(w), _ptr(add), _ptr(out), c_int(T), c_int(H),
                                c_int(self.k), _stream()), "xl_moe_combine")
        cuda_ops.launch_count += 1
        return out


def attach(engine) -> None:
    """Install the expert-parallel MoE implementation on the engine's model."""
    comm, model, args = engine.comm, engine.worker.model, engine.args
    if comm.ep_size <= 1 or not args.is_moe:
        return
    e0 = comm.ep_rank * (args.n_routed_experts // comm.ep_size)
    if comm.cfg.ep_mode == "fused" and engine.device.type == "cuda":
        model.moe_impl = FusedEP(comm, args.hidden_size, args.n_routed_experts, args.num_experts_per_tok,
                                 engine.opt.max_tokens_per_batch + 16, engine.device)
    else:
        model.moe_impl = GatherEP(comm, e0)
