"""Host-memory tier of the paged KV cache: the data plane.

Role of the reference's HierarchyKVCacheTransfer (xllm/core/framework/kv_cache/hierarchy_kv_cache_transfer.cpp: layer-wise
asynchronous device->host offload and host->device prefetch of KV blocks, `host_blocks_factor`,
global_flags.cpp:439-442).  The bookkeeping (which block lives where, under which prefix key) is done by the C++
scheduler; every step it hands this class two lists of block copies:

    offloads [(device block, host block)]   blocks that entered the device prefix cache and are not on the host yet
    loads    [(host block, device block)]   prefix blocks of a new request that only the host still holds

Layout.  The device cache is one tensor per layer and per K / V, so one logical block is `n_tensors` separate pieces.
The host pool stores a block as ONE contiguous record in pinned memory (all pieces back to back).  A small kernel packs
the pieces of up to `slots` blocks into a device staging area (`xl_kv_pack`), and each block then crosses PCIe as a
single multi-megabyte copy on the copy engines; loads run the same path backwards.  Everything is issued on a side
stream:

    side stream:  wait(forward of the previous step issued) -> pack -> D2H copies ... -> H2D copies -> unpack -> event
    main stream:  wait(event) only when the step has loads; offloads overlap the following forwards, because the
                  scheduler keeps the device blocks referenced for two more steps (and the main stream waits for the
                  offload event of two steps ago before it may reuse them)

On a CPU device (tests) the same copies are plain tensor assignments.

Third tier.  With a shared block store attached (`attach_store`, service/kv_store.py; KVCacheStore in the reference,
kv_cache_store.cpp:89-183) every block that reaches the host pool is also written to the store under its prefix key by a
background thread, straight from its pinned record once the copy from the device has finished; `fill` puts a record
fetched from the store into a host block that the scheduler adopted for it.  A host block whose record is still being
sent is not overwritten: the next copy into it waits for the send.
"""
from __future__ import annotations

import ctypes
import queue
import threading
from collections import deque
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class HostKvTier:
    def __init__(self, kv_caches, num_host_blocks: int, device: torch.device, slots: int = 32):
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        self._slots_wanted = slots
        self.tensors: List[torch.Tensor] = [t for layer in kv_caches for t in layer]
        assert self.tensors, "the KV cache must be allocated before its host tier"
        self.cache_blocks = int(self.tensors[0].shape[0])
        self.block_bytes = [int(t[0].numel() * t.element_size()) for t in self.tensors]
        assert all(b % 16 == 0 for b in self.block_bytes), "cache blocks must be multiples of 16 bytes"
        self.offsets, off = [], 0
        for b in self.block_bytes:
            self.offsets.append(off)
            off += b
        self.stride = off                                        # bytes of one packed block
        self.num_host_blocks = int(num_host_blocks)
        # host block ids start at 1 like device ids (0 is the padding id of the block managers)
        self.pool = torch.empty((self.num_host_blocks + 1, self.stride), dtype=torch.uint8, pin_memory=self.is_cuda)
        self.bytes_offloaded = 0
        self.bytes_loaded = 0
        # third tier (attach_store)
        self.store = None
        self.store_rank, self.store_world, self.store_ns = 0, 1, ""
        self.blocks_put = self.blocks_filled = 0
        self._busy: Dict[int, int] = {}                          # host block -> sends of its record still to finish
        self._busy_cv = threading.Condition()
        self._put_q: "queue.Queue" = queue.Queue()
        self._put_thread: Optional[threading.Thread] = None
        self._last_offload_event = None
        if self.is_cuda:
            self.slots = max(1, min(slots, self.num_host_blocks))
            self.staging = torch.empty((self.slots, self.stride), dtype=torch.uint8, device=self.device)
            self.side = torch.cuda.Stream(self.device)
            self._ptrs = torch.tensor([t.data_ptr() for t in self.tensors], dtype=torch.int64, device=self.device)
            self._bb = torch.tensor(self.block_bytes, dtype=torch.int64, device=self.device)
            self._off = torch.tensor(self.offsets, dtype=torch.int64, device=self.device)
            self._offload_events = deque()                       # one per step that offloaded, oldest first

    # ------------------------------------------------------------------ CUDA path
    def _pack(self, pairs: Sequence[Tuple[int, int]], to_cache: bool):
        from ..ops import cuda_ops
        from ..ops.cuda_ops import _check, _ptr, c_int, c_long, lib
        pt = torch.tensor(list(pairs), dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _check(lib().xl_kv_pack(_ptr(self._ptrs), _ptr(self._bb), _ptr(self._off), _ptr(pt), _ptr(self.staging),
                                c_long(self.stride), c_long(self.cache_blocks), c_long(self.slots), c_int(len(self.tensors)),
                                c_int(len(pairs)), c_int(1 if to_cache else 0), st), "xl_kv_pack")
        cuda_ops.launch_count += 1

    def _run_cuda(self, offloads, loads):
        main = torch.cuda.current_stream(self.device)
        # The scheduler keeps offloaded device blocks referenced for two more steps; the third step after an offload may
        # reuse them, so its forward waits until that copy has read them (one entry per step, None = no offload).
        while len(self._offload_events) > 2:
            ev = self._offload_events.popleft()
            if ev is not None:
                main.wait_event(ev)
        if not offloads:
            self._offload_events.append(None)
        if not offloads and not loads:
            return
        self.side.wait_stream(main)                              # KV written by the steps issued so far
        with torch.cuda.stream(self.side):
            for i in range(0, len(offloads), self.slots):
                chunk = offloads[i:i + self.slots]
                self._pack([(d, j) for j, (d, _) in enumerate(chunk)], to_cache=False)
                for j, (_, h) in enumerate(chunk):
                    self.pool[h].copy_(self.staging[j], non_blocking=True)
            if offloads:
                ev = torch.cuda.Event()
                ev.record(self.side)
                self._offload_events.append(ev)
                self._last_offload_event = ev
            for i in range(0, len(loads), self.slots):
                chunk = loads[i:i + self.slots]
                for j, (h, _) in enumerate(chunk):
                    self.staging[j].copy_(self.pool[h], non_blocking=True)
                self._pack([(d, j) for j, (_, d) in enumerate(chunk)], to_cache=True)
            if loads:
                ev = torch.cuda.Event()
                ev.record(self.side)
                main.wait_event(ev)                              # the forward reads what was just loaded

    # ------------------------------------------------------------------ CPU path (tests)
    def _run_cpu(self, offloads, loads):
        for d, h in offloads:
            rec = self.pool[h]
            for t, off, bb in zip(self.tensors, self.offsets, self.block_bytes):
                rec[off:off + bb] = t[d].contiguous().view(torch.uint8).reshape(-1)
        for h, d in loads:
            rec = self.pool[h]
            for t, off, bb in zip(self.tensors, self.offsets, self.block_bytes):
                t[d] = rec[off:off + bb].view(t.dtype).view(t[d].shape)

    def run(self, offloads: Sequence[Tuple[int, int]], loads: Sequence[Tuple[int, int]],
            put_keys: Sequence[Tuple[int, Tuple[int, int]]] = ()) -> None:
        """Issue the copies of one step: all offloads, then all loads, before the step's forward is enqueued.
        `put_keys`: (host block, prefix key) of the offloaded blocks, for the shared store."""
        for d, h in offloads:
            assert 0 < d < self.cache_blocks and 0 < h <= self.num_host_blocks, (d, h)
        for h, d in loads:
            assert 0 < d < self.cache_blocks and 0 < h <= self.num_host_blocks, (h, d)
        self.bytes_offloaded += len(offloads) * self.stride
        self.bytes_loaded += len(loads) * self.stride
        if self._busy and offloads:
            self._wait_not_busy([h for _, h in offloads])
        if self.is_cuda:
            self._run_cuda(list(offloads), list(loads))
        elif offloads or loads:
            self._run_cpu(offloads, loads)
        if put_keys and self.store is not None:
            with self._busy_cv:
                for h, _ in put_keys:
                    self._busy[h] = self._busy.get(h, 0) + 1
            self._put_q.put((self._last_offload_event if self.is_cuda else None, list(put_keys)))

    # ------------------------------------------------------------------ shared store (third tier)
    def attach_store(self, client, rank: int = 0, world: int = 1, namespace: str = "") -> None:
        self.store, self.store_rank, self.store_world, self.store_ns = client, rank, world, namespace
        if self._put_thread is None:
            self._put_thread = threading.Thread(target=self._put_loop, name="xllm-kv-store-put", daemon=True)
            self._put_thread.start()

    def _wait_not_busy(self, host_blocks: Sequence[int], timeout_s: float = 10.0) -> None:
        with self._busy_cv:
            self._busy_cv.wait_for(lambda: not any(h in self._busy for h in host_blocks), timeout=timeout_s)

    def _put_loop(self):
        from ..service.kv_store import block_key
        while True:
            item = self._put_q.get()
            if item is None:
                return
            ev, pairs = item
            try:
                if ev is not None:
                    ev.synchronize()                             # the records are complete in pinned memory
                keys = [block_key(k, self.store_rank, self.store_world, self.store_ns) for _, k in pairs]
                there = self.store.batch_exist(keys)
                todo = [(key, h) for key, (h, _), t in zip(keys, pairs, there) if not t]
                for i in range(0, len(todo), 8):                  # a few records per message: the socket's time limit is per message
                    part = todo[i:i + 8]
                    views = [memoryview(self.pool[h].numpy()) for _, h in part]
                    self.blocks_put += self.store.batch_put([k for k, _ in part], views)
            except Exception:                                    # the store is an optimisation: never take the engine down
                pass
            finally:
                with self._busy_cv:
                    for h, _ in pairs:
                        n = self._busy.get(h, 0) - 1
                        if n <= 0:
                            self._busy.pop(h, None)
                        else:
                            self._busy[h] = n
                    self._busy_cv.notify_all()
                self._put_q.task_done()

    def flush_store(self) -> None:
        """Wait until every queued block has been sent (tests, shutdown)."""
        if self._put_thread is not None:
            self._put_q.join()

    def fill(self, host_block: int, data) -> None:
        """Put a record fetched from the store into a host block (the scheduler has just adopted it for this content)."""
        assert 0 < host_block <= self.num_host_blocks and len(data) == self.stride, (host_block, len(data), self.stride)
        self._wait_not_busy([host_block])
        if self.is_cuda:
            self.side.synchronize()                              # an earlier load may still be reading the old record
        self.pool[host_block].copy_(torch.frombuffer(data, dtype=torch.uint8))
        self.blocks_filled += 1

    def drain(self):
        if self.is_cuda:
            self.side.synchronize()

    def detach(self):
        """The device cache is about to be released (engine sleep): keep the host pool, drop everything that points into
        device memory."""
        self.drain()
        self.tensors = []
        if self.is_cuda:
            self.staging = self._ptrs = None
            self._offload_events.clear()

    def attach(self, kv_caches):
        """A new device cache of the same geometry replaces the released one (engine wake-up)."""
        self.tensors = [t for layer in kv_caches for t in layer]
        assert [int(t[0].numel() * t.element_size()) for t in self.tensors] == self.block_bytes, "cache geometry changed"
        self.cache_blocks = int(self.tensors[0].shape[0])
        if self.is_cuda:
            self.staging = torch.empty((self.slots, self.stride), dtype=torch.uint8, device=self.device)
            self._ptrs = torch.tensor([t.data_ptr() for t in self.tensors], dtype=torch.int64, device=self.device)
