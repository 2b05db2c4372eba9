"""Expert parallelism: token dispatch / combine between the ranks that hold the experts.

Two implementations behind the same call `moe(h, mlp_weights, topk_weights, topk_ids, layer) -> [T, H]`:

* `FusedEP` (`--expert_parallel_degree 2`): the all-to-all is carried by our own kernels over NVLink peer memory
  (`csrc/cuda/ep_fused.cu`): the ranks first exchange their per-expert row counts, so that every row is stored
  straight into its final, expert-major place in the destination rank's receive buffer (as bf16, or quantised to
  e4m3 with 1x128 scales on the way); the grouped tcgen05 GEMMs read that buffer, and every output row is stored
  back into its source rank's return slot, where the top-k weighted sum reads local memory only.  No NCCL call, no
  sort and no gather on this path.
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
            # Every rank pads its rows to the largest count (padding rows route to no expert), so the collectives and all
            # shapes depend on that one number only: CUDA graphs of a rank stay valid whatever the other ranks hold, as
            # long as the maximum is the same.
            g = c.world_group
            m, T = max(counts), h.shape[0]

            def padded(x, fill):
                if T == m:
                    return x.contiguous()
                out = x.new_full((m,) + tuple(x.shape[1:]), fill)
                out[:T] = x
                return out
            R, me = len(counts), c.dp_rank
            assert R == c.world_size, "the gather spans the world: attention DP x EP without tensor parallelism"
            hh = torch.empty((R * m,) + tuple(h.shape[1:]), dtype=h.dtype, device=h.device)
            ww = torch.empty((R * m,) + tuple(w.shape[1:]), dtype=w.dtype, device=w.device)
            ii = torch.empty((R * m,) + tuple(ids.shape[1:]), dtype=ids.dtype, device=ids.device)
            dist.all_gather_into_tensor(hh, padded(h, 0), group=g)
            dist.all_gather_into_tensor(ww, padded(w, 0), group=g)
            dist.all_gather_into_tensor(ii, padded(ids, -1), group=g)
            y = ops.moe_experts(hh, mlp.w13, mlp.w2, ww, ii, self.e0, mlp.interleaved)
            y = c.all_reduce(y, group=g)
            return y[me * m:me * m + T]
        y = ops.moe_experts(h, mlp.w13, mlp.w2, w, ids, self.e0, mlp.interleaved)
        return c.all_reduce(y, group=c.ep_group)


class _XlEpArgs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("recv_x", "recv_scale", "recv_meta", "counts_all", "count_flags", "data_flags", "ret_y",
                                                "ret_flags", "hist", "base", "fill", "abort_flag", "done_counter", "epoch", "total_rows",
                                                "num_m_tiles", "tile_expert", "tile_row0", "tile_row_end")] + \
               [(n, ctypes.c_int) for n in ("max_tiles", "R", "rank", "rows_cap", "H", "E_local", "fp8")] + [("timeout_s", ctypes.c_double)]


class _TileTable:
    """The grouped GEMMs' view of what the dispatch kernel computed for this rank's receive buffer."""

    def __init__(self, work: torch.Tensor, max_tiles: int):
        self.work, self.max_tiles = work, max_tiles
        self.total_rows, self.num_m_tiles = work[0:1], work[1:2]
        self.tile_expert = work[8:8 + max_tiles]
        self.tile_row0 = work[8 + max_tiles:8 + 2 * max_tiles]
        self.tile_row_end = work[8 + 2 * max_tiles:8 + 3 * max_tiles]


class FusedEP:
    """Five launches per MoE layer with bf16 experts: dispatch (count, layout exchange, send, arrival wait), grouped GEMM
    w13 + SwiGLU, grouped GEMM w2, return, combine (wait + weighted sum); with fp8 block-scaled experts the rows travel as
    e4m3 + 1x128 scales and one activation-quantisation kernel sits between the two GEMMs."""

    def __init__(self, comm, hidden: int, n_experts: int, top_k: int, max_tokens: int, device: torch.device,
                 timeout_s: float = 2.0, fp8: bool = False):
        self.comm, self.H, self.k, self.device, self.fp8 = comm, hidden, top_k, device, fp8
        self.R, self.rank = comm.ep_size, comm.ep_rank
        assert self.R == comm.world_size, "the fused all-to-all spans the whole world"
        assert hidden % 128 == 0
        self.E_local = n_experts // self.R
        self.T_cap = max_tokens
        self.per_token = min(top_k, self.E_local)
        self.rows_cap = self.R * max_tokens * self.per_token      # rows one rank can receive (every source, every slot)
        self.slots_cap = max_tokens * top_k
        group = list(range(self.R))
        es = 1 if fp8 else 2
        self.recv_x = SymmetricBuffer(self.rows_cap * hidden * es, comm.rank, group, device)
        self.recv_scale = SymmetricBuffer(self.rows_cap * (hidden // 128) * 4, comm.rank, group, device) if fp8 else None
        self.recv_meta = SymmetricBuffer(self.rows_cap * 8, comm.rank, group, device)
        self.ret_y = SymmetricBuffer(self.slots_cap * hidden * 2, comm.rank, group, device)
        RE = self.R * self.E_local
        # ints: [0:8) count flags, [8:16) data flags, [16:24) return flags, then the count tables of every rank (two parities)
        self.sync = SymmetricBuffer((64 + 2 * self.R * RE) * 4, comm.rank, group, device)
        self.max_tiles = (self.rows_cap + 127) // 128 + self.E_local
        # local scratch: hist / base / fill [RE each], abort, done[4], epoch, then the tile table
        self.local = torch.zeros(3 * RE + 16, dtype=torch.int32, device=device)
        self.work = torch.zeros(8 + 3 * self.max_tiles, dtype=torch.int32, device=device)
        self.table = _TileTable(self.work, self.max_tiles)
        lp, wp = self.local.data_ptr(), self.work.data_ptr()
        a = _XlEpArgs()
        self._keep = [self.recv_x.ptr_array, self.recv_meta.ptr_array, self.ret_y.ptr_array, self.sync.offset_array(64 * 4),
                      self.sync.offset_array(0), self.sync.offset_array(8 * 4), self.sync.offset_array(16 * 4),
                      self.recv_scale.ptr_array if fp8 else None]
        cast = lambda arr: ctypes.cast(arr, ctypes.c_void_p) if arr is not None else None
        a.recv_x, a.recv_meta, a.ret_y, a.counts_all = cast(self._keep[0]), cast(self._keep[1]), cast(self._keep[2]), cast(self._keep[3])
        a.count_flags, a.data_flags, a.ret_flags, a.recv_scale = cast(self._keep[4]), cast(self._keep[5]), cast(self._keep[6]), cast(self._keep[7])
        a.hist, a.base, a.fill = lp, lp + RE * 4, lp + 2 * RE * 4
        a.abort_flag, a.done_counter, a.epoch = lp + 3 * RE * 4, lp + (3 * RE + 4) * 4, lp + (3 * RE + 8) * 4
        a.total_rows, a.num_m_tiles = wp, wp + 4
        a.tile_expert, a.tile_row0, a.tile_row_end = wp + 8 * 4, wp + (8 + self.max_tiles) * 4, wp + (8 + 2 * self.max_tiles) * 4
        a.max_tiles, a.R, a.rank, a.rows_cap, a.H, a.E_local, a.fp8 = self.max_tiles, self.R, self.rank, self.rows_cap, hidden, self.E_local, int(fp8)
        a.timeout_s = timeout_s
        self.args = a
        self.recv_x_t = (self.recv_x.local.view(torch.float8_e4m3fn) if fp8 else self.recv_x.local.view(torch.bfloat16)).view(self.rows_cap, hidden)
        self.recv_scale_t = self.recv_scale.local.view(torch.float32).view(self.rows_cap, hidden // 128) if fp8 else None
        self.ret_y_t = self.ret_y.local.view(torch.bfloat16).view(self.slots_cap, hidden)
        self.dp_token_counts: Optional[List[int]] = None
        dist.barrier()

    def _rows_bound(self) -> int:
        """Upper bound of the rows this rank can receive in the step: every rank's token count is at most the largest
        one, which is the only number of the other ranks that shapes (and CUDA graphs) depend on."""
        counts = self.dp_token_counts
        return max(1, min(self.rows_cap, (self.R * max(counts) if counts else self.R * self.T_cap) * self.per_token))

    def dispatch(self, h: torch.Tensor, ids: torch.Tensor) -> None:
        T = h.shape[0]
        assert T <= self.T_cap and h.shape[1] == self.H and ids.dtype == torch.int32 and ids.is_contiguous()
        if h.stride(-1) != 1:
            h = h.contiguous()
        _check(lib().xl_ep_dispatch(ctypes.byref(self.args), _ptr(h), _ptr(ids), c_int(T), c_int(self.k), c_int(h.stride(0)), _stream()),
               "xl_ep_dispatch")
        cuda_ops.launch_count += 1

    def experts(self, mlp, rows: int) -> torch.Tensor:
        """The two grouped GEMMs over the received rows (expert-major, dense); returns y [rows, H]."""
        t = self.table
        if not self.fp8:
            xs = self.recv_x_t[:rows]
            if mlp.interleaved:
                hmid = moe_cuda.grouped_gemm(xs, mlp.w13, t, swiglu=True)
            else:
                hmid = cuda_ops.silu_and_mul(moe_cuda.grouped_gemm(xs, mlp.w13, t))
            return moe_cuda.grouped_gemm(hmid, mlp.w2, t)
        L = lib()
        E, I2, H = mlp.w13.shape
        xq, xsc = self.recv_x_t[:rows], self.recv_scale_t[:rows]
        hmid = torch.empty((rows, I2), dtype=torch.bfloat16, device=self.device)
        _check(L.xl_grouped_gemm_fp8_block(_ptr(xq), _ptr(mlp.w13), _ptr(hmid), _ptr(xsc), _ptr(mlp.w13_scale), c_int(rows), c_int(I2),
                                           c_int(H), c_int(hmid.stride(0)), c_int(E), _ptr(t.tile_expert), _ptr(t.tile_row0),
                                           _ptr(t.tile_row_end), _ptr(t.num_m_tiles), c_int(t.max_tiles), _stream()),
               "xl_grouped_gemm_fp8_block(w13)")
        hq, hsc = cuda_ops.quant_act_1x128(hmid, gated=True, rows_dev=t.total_rows)
        y = torch.empty((rows, H), dtype=torch.bfloat16, device=self.device)
        _check(L.xl_grouped_gemm_fp8_block(_ptr(hq), _ptr(mlp.w2), _ptr(y), _ptr(hsc), _ptr(mlp.w2_scale), c_int(rows), c_int(H),
                                           c_int(I2 // 2), c_int(y.stride(0)), c_int(E), _ptr(t.tile_expert), _ptr(t.tile_row0),
                                           _ptr(t.tile_row_end), _ptr(t.num_m_tiles), c_int(t.max_tiles), _stream()),
               "xl_grouped_gemm_fp8_block(w2)")
        cuda_ops.launch_count += 2
        return y

    def __call__(self, h, mlp, w, ids, layer_idx, add: Optional[torch.Tensor] = None):
        T, H = h.shape
        ids = ids.contiguous()
        self.dispatch(h, ids)
        rows = self._rows_bound()
        y = self.experts(mlp, rows)
        L = lib()
        _check(L.xl_ep_return(ctypes.byref(self.args), _ptr(y), c_int(y.stride(0)), c_int(rows), _stream()), "xl_ep_return")
        out = torch.empty((T, H), dtype=torch.bfloat16, device=h.device)
        _check(L.xl_ep_combine(ctypes.byref(self.args), _ptr(ids), _ptr(w.contiguous()), _ptr(add), _ptr(out), c_int(T), c_int(self.k),
                               _stream()), "xl_ep_combine")
        cuda_ops.launch_count += 2
        return out


def attach(engine) -> None:
    """Install the expert-parallel MoE implementation on the engine's model."""
    comm, model, args = engine.comm, engine.worker.model, engine.args
    if comm.ep_size <= 1 or not args.is_moe:
        return
    e0 = comm.ep_rank * (args.n_routed_experts // comm.ep_size)
    if comm.cfg.ep_mode == "fused" and engine.device.type == "cuda":
        fp8 = bool(getattr(getattr(args, "quant", None), "block_scaled", False))
        n_slots = args.n_routed_experts + (engine.opt.redundant_experts_num * comm.ep_size if engine.opt.enable_eplb else 0)
        model.moe_impl = FusedEP(comm, args.hidden_size, n_slots, args.num_experts_per_tok,
                                 engine.opt.max_tokens_per_batch + 16, engine.device, fp8=fp8)
    else:
        model.moe_impl = GatherEP(comm, e0)
