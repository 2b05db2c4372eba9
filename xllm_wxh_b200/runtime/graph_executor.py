"""CUDA-graph executor for decode steps and, optionally, for steps that carry prefill tokens.

Same contract as the reference's CudaGraphExecutorImpl (xllm/core/runtime/cuda_graph_executor_impl.cpp:
102-183 persistent buffers, 682-842 capture, 844-924 replay, 1387-1407 buckets): one graph per token
bucket {1,2,4,8,16k}, captured lazily on first use and replayed afterwards; inputs live in persistent
device buffers (here: the worker's single packed step buffer, whose section offsets depend only on
the bucket capacities); all graphs share one memory pool so that capture memory is the maximum over
shapes, not the sum (the reference reaches that with a VMM-backed allocator,
platform/shared_vmm_allocator.h:25-80); a failed capture is fatal rather than silently falling back.

Everything shape-dependent that changes per step (sequence lengths, block tables, slots, sampling
indexes, and the split of the batch into decode and prefill sequences) is read by the kernels from
device memory, so no host-side "plan" is needed before replay, and attention is part of the captured
graph (the reference captures prefill piecewise around an eager attention call,
cuda_graph_executor_impl.cpp:1217-1227, kernels/cuda/attention_runner.cpp:28-164).  The number of live
graphs is bounded; the least recently used one is dropped first.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class CudaGraphExecutor:
    def __init__(self, worker):
        self.worker = worker
        self.graphs: Dict[Tuple[int, ...], Tuple[torch.cuda.CUDAGraph, torch.Tensor, torch.Tensor, int]] = {}
        self.pool = torch.cuda.graph_pool_handle() if worker.opt.enable_graph_vmm_pool else None
        self.capture_stream = torch.cuda.Stream(device=worker.device)
        self.max_graphs = 96
        self.capture_after = 2          # a shape with prefill tokens is captured at its second appearance
        self.seen: Dict[Tuple[int, ...], int] = {}
        self.warmed = set()             # kinds of step (decode-only / with prefill) that already ran outside a capture
        self.num_eager_padded = 0
        self.num_captures = 0
        self.num_replays = 0
        self.replayed_kernels = 0       # kernels executed through replays (captured count x replays)

    def invalidate(self):
        """The staging buffer moved: captured graphs point at freed memory."""
        self.graphs.clear()
        return self

    def _key(self, inp) -> Tuple[int, ...]:
        L = inp.layout
        # decode-only steps and steps with prefill tokens launch different attention kernels
        # an expert-parallel MoE layer sizes its exchange (collective shapes, row bounds) by the largest token count among
        # the DP ranks
        counts = getattr(getattr(self.worker.model, "moe_impl", None), "dp_token_counts", None)
        return (L.T_cap, L.B_cap, L.MB_cap, L.S_cap, L.P_cap, int(inp.has_prefill)) + ((max(counts),) if counts else ())

    def run(self, inp, gather_logits: bool = True):
        """`gather_logits=False`: the captured step ends with this rank's vocabulary shard of the logits (no all-gather)."""
        self._gather = gather_logits
        key = self._key(inp) + (int(gather_logits),)
        entry = self.graphs.pop(key, None)
        if entry is None:
            # Shapes with prefill tokens vary a lot (chunk sizes, number of sequences): one that shows up for the
            # first time runs at its padded size without a graph, and is captured only when it comes back.
            seen = self.seen.get(key, 0) + 1
            if len(self.seen) > 4096:
                self.seen.clear()
            self.seen[key] = seen
            # With collectives that cross the DP groups (expert parallelism under attention DP) every rank must run
            # each layer's exchange exactly once per step, whatever its own shape: the extra eager run that `_capture`
            # makes for lazy initialisation would leave this rank one exchange ahead of its peers.  The first step of
            # each kind therefore runs eagerly as the step itself.
            first_of_kind = self._cross_dp() and bool(inp.has_prefill) not in self.warmed
            if (inp.has_prefill and seen < self.capture_after) or first_of_kind:
                w = self.worker
                self.num_eager_padded += 1
                self.warmed.add(bool(inp.has_prefill))
                hidden = w.model.forward(inp, w.kv_caches)
                return hidden, w.model.logits(hidden, inp.sample_idx, self._gather)
            while len(self.graphs) >= self.max_graphs:
                self.graphs.pop(next(iter(self.graphs)))      # dicts keep insertion order: first = least recently used
            entry = self._capture(key, inp)
        self.graphs[key] = entry
        g, hidden, logits, n_kernels = entry
        g.replay()
        self.num_replays += 1
        self.replayed_kernels += n_kernels
        return hidden, logits

    def _cross_dp(self) -> bool:
        c = self.worker.comm
        return c.dp_size > 1 and c.ep_size > 1

    def _capture(self, key, inp):
        w = self.worker
        model, kv = w.model, w.kv_caches
        # one eager run first, once per kind of step: lazy initialisation (kernel attributes, workspaces, handles) must
        # not happen inside a capture
        cur = torch.cuda.current_stream(w.device)
        self.capture_stream.wait_stream(cur)
        if bool(inp.has_prefill) not in self.warmed:
            self.warmed.add(bool(inp.has_prefill))
            with torch.cuda.stream(self.capture_stream):
                hidden = model.forward(inp, kv)
                logits = model.logits(hidden, inp.sample_idx, self._gather)
            cur.wait_stream(self.capture_stream)
        torch.cuda.synchronize(w.device)
        g = torch.cuda.CUDAGraph()
        from ..ops import cuda_ops
        before = cuda_ops.launch_count
        # The garbage collector must not run inside the capture: finalising an unreachable CUDAGraph of an earlier
        # engine destroys its executable graph, which CUDA refuses while a stream is capturing and which
        # invalidates the capture in progress.
        import gc
        gc.collect()
        gc_was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g, pool=self.pool, stream=self.capture_stream):
                hidden = model.forward(inp, kv)
                logits = model.logits(hidden, inp.sample_idx, self._gather)
        except Exception as e:  # fail fast by design
            raise RuntimeError(f"CUDA graph capture failed for bucket {key}: {e}") from e
        finally:
            if gc_was_enabled:
                gc.enable()
        n_kernels = cuda_ops.launch_count - before
        cuda_ops.launch_count = before          # captured launches did not execute; replays are counted separately
        self.graphs[key] = (g, hidden, logits, n_kernels)
        self.num_captures += 1
        return self.graphs[key]
