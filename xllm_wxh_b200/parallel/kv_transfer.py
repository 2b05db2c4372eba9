"""KV-cache transfer between a prefill and a decode instance.

`KVTransfer.push(pairs)` copies the listed (source block -> destination block) pairs of every cache tensor of this
rank into the cache of the matching rank of the linked decode instance.

* `LocalCopyTransfer`  : both instances live in this process (tests, CPU, single-process GPU set-ups): tensor copies.
* `NvlinkPushTransfer` : the decode rank's cache tensors are mapped through CUDA IPC and written by the push kernel
                         (`csrc/cuda/kv_transfer.cu`) with peer stores; per-tensor ready flags are published to the
                         decode GPU for layer-pipelined consumers.  With `pull=True` the roles swap (PULL mode): the
                         object lives on the decode rank, maps the prefill rank's cache and the same kernel reads the
                         blocks over NVLink with peer loads.

* `MultiTransfer`      : one source rank serving several destination ranks (instances of different TP degree whose
                         ranks all hold the same cache, i.e. the MLA latent cache; `plan_links` says who serves whom).

Reference roles: KVCacheTransfer::push_kv_blocks / merge_kv_blocks (xllm/core/framework/kv_cache/kv_cache_transfer.cpp:86-140:
source TP rank -> destination workers when the degrees differ); the reference's implementations exist for Ascend only.
Both sides must use the same block size; caches sharded by KV head need the same TP degree as well.
"""
from __future__ import annotations

import base64
import ctypes
from typing import Dict, List, Sequence, Tuple

import torch


def plan_links(src_tp: int, dst_tp: int, src_rank: int) -> List[int]:
    """Destination TP ranks that source TP rank `src_rank` writes to when every rank of an instance holds the same cache.
    Equal degrees: rank r -> rank r.  A wider destination: r -> r, r + src_tp, r + 2 src_tp, ... (the stride rule of the
    reference's merge_kv_blocks).  A narrower destination: the first dst_tp source ranks serve one rank each and the others
    none (the reference lets the surplus ranks write the same rows a second time)."""
    if src_tp <= 0 or dst_tp <= 0 or not 0 <= src_rank < src_tp:
        raise ValueError(f"bad link plan: src_tp={src_tp} dst_tp={dst_tp} src_rank={src_rank}")
    if src_rank >= dst_tp:
        return []
    return list(range(src_rank, dst_tp, src_tp))


def plan_source(src_tp: int, dst_tp: int, dst_rank: int) -> int:
    """PULL mode: the source TP rank that destination rank `dst_rank` reads (the inverse of `plan_links`)."""
    if src_tp <= 0 or dst_tp <= 0 or not 0 <= dst_rank < dst_tp:
        raise ValueError(f"bad link plan: src_tp={src_tp} dst_tp={dst_tp} dst_rank={dst_rank}")
    return dst_rank % src_tp


class MultiTransfer:
    """Several transfers driven as one: a source rank that serves more than one destination rank (or none)."""

    def __init__(self, transfers):
        self.transfers = list(transfers)

    @property
    def bytes_moved(self) -> int:
        return sum(t.bytes_moved for t in self.transfers)

    def push(self, pairs, layer: int = -1):
        for t in self.transfers:
            t.push(pairs, layer)

    def push_layer_async(self, pairs, layer: int):
        for t in self.transfers:
            t.push_layer_async(pairs, layer)

    def join(self):
        for t in self.transfers:
            t.join()

    def wait(self):
        for t in self.transfers:
            t.wait()


class LocalCopyTransfer:
    def __init__(self, src_caches, dst_caches):
        self.src, self.dst = src_caches, dst_caches
        self.bytes_moved = 0

    def push(self, pairs: Sequence[Tuple[int, int]], layer: int = -1):
        """`layer` >= 0: only that layer's tensors (layer-by-layer push under the forward pass)."""
        if not pairs:
            return
        s = torch.tensor([p[0] for p in pairs], dtype=torch.long, device=self.src[0][0].device)
        d = torch.tensor([p[1] for p in pairs], dtype=torch.long, device=self.dst[0][0].device)
        layers = list(zip(self.src, self.dst)) if layer < 0 else [(self.src[layer], self.dst[layer])]
        for ls, ld in layers:
            for ts, td in zip(ls, ld):
                blk = ts.index_select(0, s)
                td.index_copy_(0, d, blk.to(td.device))
                self.bytes_moved += blk.numel() * blk.element_size()

    def push_layer_async(self, pairs: Sequence[Tuple[int, int]], layer: int):
        self.push(pairs, layer)

    def join(self):
        pass

    def wait(self):
        for layer in self.dst:
            if layer[0].is_cuda:
                torch.cuda.synchronize(layer[0].device)


def export_cache_handles(kv_caches) -> List[Dict]:
    """IPC descriptions of this rank's cache tensors (decode side): one entry per tensor in layer order."""
    from ..ops.cuda_ops import c_void_p, lib
    out = []
    for layer in kv_caches:
        for t in layer:
            if getattr(t, "_xl_own_alloc", False):
                # allocated with cudaMalloc by this library (Worker.allocate_kv_cache(ipc=True)): plain runtime handle
                buf = (ctypes.c_char * 64)()
                if lib().xl_ipc_get_handle(c_void_p(t.data_ptr()), buf) != 64:
                    raise RuntimeError("cudaIpcGetMemHandle failed for a KV-cache tensor")
                handle, offset = bytes(buf), 0
            else:
                _, handle, _, offset, *_ = t.untyped_storage()._share_cuda_()
                from ..runtime.weight_transfer import runtime_ipc_handle
                handle = runtime_ipc_handle(handle)
                offset = int(offset) + t.storage_offset() * t.element_size()
            out.append({"handle": base64.b64encode(handle).decode(), "offset": int(offset),
                        "nbytes": t.numel() * t.element_size(), "blocks": t.shape[0], "block_bytes": t[0].numel() * t.element_size()})
    return out


def local_peer_handles(kv_caches) -> List[Dict]:
    """Descriptions of cache tensors that live on another GPU of this same process (peer access, no IPC): for
    measurements and single-process set-ups.  `NvlinkPushTransfer` takes them in place of IPC handles."""
    return [{"ptr": t.data_ptr(), "offset": 0, "nbytes": t.numel() * t.element_size(), "blocks": t.shape[0],
             "block_bytes": t[0].numel() * t.element_size()} for layer in kv_caches for t in layer]


class NvlinkPushTransfer:
    def __init__(self, src_caches, peer_handles: List[Dict], device: torch.device, pull: bool = False):
        """`src_caches`: this rank's cache tensors; `peer_handles`: the other instance's.  `pull`: this rank is the
        destination (pairs stay (block of the prefill instance, block of the decode instance))."""
        from ..ops.cuda_ops import lib
        L = lib()
        L.xl_ipc_open_handle.restype = ctypes.c_void_p
        self.device = device
        self.pull = pull
        self.tensors = [t for layer in src_caches for t in layer]
        # tensors of layer i: [layer_first[i], layer_first[i + 1])
        self.layer_first = [0]
        for layer in src_caches:
            self.layer_first.append(self.layer_first[-1] + len(layer))
        self.side = torch.cuda.Stream(device=device)       # layer-by-layer pushes run here, beside the forward pass
        self._pairs_dev = None
        assert len(self.tensors) == len(peer_handles), "prefill and decode instances hold different cache tensors"
        dst_ptrs, opened = [], {}
        for t, h in zip(self.tensors, peer_handles):
            bb = t[0].numel() * t.element_size()
            assert bb == h["block_bytes"], ("block size / head layout differs between the instances (caches sharded by KV head "
                                            "need the same TP degree on both sides)")
            if "ptr" in h:                       # a tensor of this process on a peer GPU
                dst_ptrs.append(h["ptr"])
                continue
            raw = base64.b64decode(h["handle"])
            base = opened.get(raw)
            if base is None:
                base = L.xl_ipc_open_handle((ctypes.c_char * 64).from_buffer_copy(raw[:64]))
                if not base:
                    raise RuntimeError("cudaIpcOpenMemHandle failed for the decode instance's KV cache")
                opened[raw] = base
            dst_ptrs.append(base + h["offset"])
        self.src_blocks = self.tensors[0].shape[0]
        self.dst_blocks = peer_handles[0]["blocks"]
        n = len(self.tensors)
        self.src_ptrs = torch.tensor([t.data_ptr() for t in self.tensors], dtype=torch.int64, device=device)
        self.dst_ptrs = torch.tensor(dst_ptrs, dtype=torch.int64, device=device)
        if pull:
            self.src_ptrs, self.dst_ptrs = self.dst_ptrs, self.src_ptrs
            self.src_blocks, self.dst_blocks = self.dst_blocks, self.src_blocks
        self.block_bytes = torch.tensor([t[0].numel() * t.element_size() for t in self.tensors], dtype=torch.int64, device=device)
        self.done = torch.zeros(n, dtype=torch.int32, device=device)
        self.epoch = 0
        self.bytes_moved = 0

    def push(self, pairs: Sequence[Tuple[int, int]], layer: int = -1):
        """Copy the listed (source block, destination block) pairs of every cache tensor (`layer` < 0) or of one layer's
        tensors into the decode instance's cache, on the current stream."""
        if not pairs:
            return
        from ..ops import cuda_ops
        from ..ops.cuda_ops import _check, _ptr, _stream, c_int, c_long, c_void_p, lib
        if layer <= 0:
            self.epoch += 1
            self._pairs_dev = torch.tensor(list(pairs), dtype=torch.int32, device=self.device).contiguous()
        first, n = (0, len(self.tensors)) if layer < 0 else (self.layer_first[layer], self.layer_first[layer + 1] - self.layer_first[layer])
        off = lambda t, es: c_void_p(t.data_ptr() + first * es)
        _check(lib().xl_kv_push(off(self.src_ptrs, 8), off(self.dst_ptrs, 8), _ptr(self._pairs_dev), off(self.done, 4), c_void_p(0),
                                off(self.block_bytes, 8), c_long(self.src_blocks), c_long(self.dst_blocks), c_int(n),
                                c_int(len(pairs)), c_int(self.epoch), _stream()), "xl_kv_push")
        cuda_ops.launch_count += 1
        if not hasattr(self, "_bytes_per_block"):
            self._bytes_per_block = [int(b) for b in self.block_bytes.tolist()]
        self.bytes_moved += len(pairs) * sum(self._bytes_per_block[first:first + n])

    def push_layer_async(self, pairs: Sequence[Tuple[int, int]], layer: int):
        """Push one layer's blocks on the side stream as soon as the compute stream has written them: the copy over NVLink
        runs beside the rest of the forward pass (the reference synchronises its push per layer the same way,
        llm_worker_impl.cpp:98-113)."""
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            self.push(pairs, layer)

    def join(self):
        """The compute stream waits for the pushes issued so far (before source blocks can be reused)."""
        torch.cuda.current_stream(self.device).wait_stream(self.side)

    def wait(self):
        torch.cuda.synchronize(self.device)
