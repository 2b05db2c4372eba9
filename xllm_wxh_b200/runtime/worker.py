"""Per-device worker: owns the model shard, the paged KV tensors, the staging buffers and the
executors (eager + CUDA graph).

Role of the reference's WorkerImpl / LLMWorkerImpl (xllm/core/runtime/worker_impl.cpp:171-708,
llm_worker_impl.cpp:79-229): `execute()` = host->device copy of the packed step inputs on the
compute stream, placeholder-token patching for schedule overlap (worker_impl.cpp:510-530), model
forward (eager or graph replay), logits of the selected rows, sampling, device->host copy of the
sampled tokens into pinned memory.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import os

import numpy as np
import torch

from .. import _core, ops
from ..config import Options
from ..framework.step_input import StepInput, make_layout, H_NUM_TOKENS, H_NUM_SEQS
from ..models.args import ModelArgs
from ..models.registry import get_model_class
from ..parallel.comm import Comm


def graph_bucket(n: int) -> int:
    """Token buckets of the graph executor: 1, 2, 4, 8, then multiples of 16
    (reference: cuda_graph_executor_impl.cpp:1387-1407)."""
    if n <= 1:
        return 1
    if n <= 2:
        return 2
    if n <= 4:
        return 4
    if n <= 8:
        return 8
    return (n + 15) // 16 * 16


def pow2_bucket(n: int, lo: int = 1) -> int:
    b = lo
    while b < n:
        b *= 2
    return b


@dataclasses.dataclass
class StepResult:
    batch_id: int
    n_sample: int
    width: int
    tokens: torch.Tensor                  # pinned host int32 [S_cap * width]
    logprobs: Optional[torch.Tensor]      # pinned host fp32
    top_vals: Optional[torch.Tensor]
    top_ids: Optional[torch.Tensor]
    event: Optional["torch.cuda.Event"]
    embeddings: Optional[torch.Tensor] = None

    def wait(self):
        if self.event is not None:
            self.event.synchronize()
        return self


class Worker:
    def __init__(self, args: ModelArgs, options: Options, comm: Optional[Comm] = None, device: str = "cpu",
                 model=None):
        self.args, self.opt = args, options
        self.comm = comm or Comm()
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        if self.is_cuda:
            torch.cuda.set_device(self.device)
        dtype = {"auto": None, "bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[options.dtype]
        self.model = model if model is not None else get_model_class(args.model_type)(args, self.comm, self.device, dtype)
        self.kv_caches: List[Tuple[torch.Tensor, ...]] = []
        self.num_blocks = 0
        self.block_size = options.block_size
        self._layouts: Dict[Tuple[int, int, int, int, int], "_core.BatchLayout"] = {}
        self._host: Optional[torch.Tensor] = None
        self._own_host: Optional[torch.Tensor] = None
        self._dev: Optional[torch.Tensor] = None
        self._last_tokens: Optional[torch.Tensor] = None    # device int32: previous step's samples (overlap patching)
        self._graphs = None
        self._result_slots: List[Dict[str, torch.Tensor]] = []
        self._slot_i = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.kernel_launches = 0
        self.sharded_greedy_steps = 0
        self.sharded_sampling_steps = 0          # steps that sampled from per-shard candidates (tensor parallel)
        self.shard_sampling_overflows = 0
        self._shard_sampling_ok = True
        self._shard_over_event = None
        self._shard_over_host = torch.zeros(1, dtype=torch.int32, pin_memory=self.is_cuda)
        # "no", "yes" for the reranker score (defaults: the reference's constants for the Qwen3 vocabulary)
        self.yes_no_ids = (int(getattr(options, "rerank_no_token_id", 2152)), int(getattr(options, "rerank_yes_token_id", 9693)))

    # ------------------------------------------------------------------ memory
    def profile_kv_blocks(self) -> int:
        """How many KV blocks fit (reference: llm_engine.cpp:375-530 estimate_kv_cache_capacity)."""
        if self.opt.num_kv_blocks > 0:
            return self.opt.num_kv_blocks
        per_block = self.kv_bytes_per_block()
        if self.opt.max_cache_size > 0:
            return max(2, int(self.opt.max_cache_size // per_block))
        if self.is_cuda:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = total * self.opt.max_memory_utilization - (total - free)
            # activations of the largest step + graph pools + workspaces
            a = self.args
            act = self.opt.max_tokens_per_batch * (a.hidden_size * 12 + a.intermediate_size // max(1, self.comm.tp_size) * 6 +
                                                   0) * 2
            act += 1024 * a.vocab_size * 4 // max(1, self.comm.tp_size) * 3
            budget -= act + (2 << 30)
            return max(2, int(budget // per_block))
        return 1024

    def kv_bytes_per_block(self) -> int:
        shapes = self.model.kv_cache_shapes(1, self.block_size)
        es = torch.empty((), dtype=self.model.dtype).element_size()
        return sum(int(np.prod(s)) * es for layer in shapes for s in layer)

    def allocate_kv_cache(self, num_blocks: int, ipc: bool = False):
        """`ipc`: allocate every cache tensor with its own cudaMalloc so that it can be exported through CUDA IPC
        (decode side of a disaggregated pair: the prefill instance writes into these tensors over NVLink)."""
        self.num_blocks = num_blocks
        shapes = self.model.kv_cache_shapes(num_blocks, self.block_size)
        if ipc and self.is_cuda:
            import ctypes
            from ..ops.cuda_ops import lib
            from ..parallel.fused_tp import _CudaBuffer
            L = lib()
            L.xl_dev_malloc.restype = ctypes.c_void_p
            es = torch.empty((), dtype=self.model.dtype).element_size()
            caches = []
            for layer in shapes:
                ts = []
                for s in layer:
                    nbytes = int(np.prod(s)) * es
                    ptr = L.xl_dev_malloc(ctypes.c_long(nbytes))
                    if not ptr:
                        raise RuntimeError(f"cudaMalloc of {nbytes} bytes for the KV cache failed")
                    t = _CudaBuffer(ptr, nbytes).tensor(self.device).view(self.model.dtype).view(s)
                    t._xl_own_alloc = True
                    ts.append(t)
                caches.append(tuple(ts))
            self.kv_caches = caches
            return
        self.kv_caches = [tuple(torch.zeros(s, dtype=self.model.dtype, device=self.device) for s in layer) for layer in shapes]

    # ------------------------------------------------------------------ staging
    def layout_for(self, T: int, B: int, MB: int, S: int, P: int) -> "_core.BatchLayout":
        key = (T, B, MB, S, P)
        L = self._layouts.get(key)
        if L is None:
            L = make_layout(T, B, MB, S, P)
            self._layouts[key] = L
        return L

    def _ensure_staging(self, words: int):
        """Device-side step buffer.  It is sized once for the largest message where possible: growing it later
        moves it, which invalidates every captured graph."""
        if not self.is_cuda:
            return
        if self._dev is None or self._dev.numel() < words:
            n = pow2_bucket(words, 1 << 16)
            self._dev = torch.empty(n, dtype=torch.int32, device=self.device)
            if self._graphs is not None:
                self._graphs.invalidate()

    def set_host(self, host_view: torch.Tensor):
        """Packed inputs of the coming step (pinned on CUDA).  On CPU the 'device' buffer is the same memory."""
        self._host = host_view
        if not self.is_cuda:
            self._dev = host_view

    def host_staging(self, words: int) -> torch.Tensor:
        """A private pinned buffer for callers that drive the worker without an engine (tests, tools)."""
        if self._own_host is None or self._own_host.numel() < words:
            self._own_host = torch.zeros(pow2_bucket(words, 1 << 12), dtype=torch.int32, pin_memory=self.is_cuda)
        self._ensure_staging(words)
        self.set_host(self._own_host)
        return self._own_host

    def _result_slot(self, S: int, width: int, top: int) -> Dict[str, torch.Tensor]:
        # a small ring of pinned result buffers so that an overlapped step does not overwrite unread results
        if not self._result_slots:
            self._result_slots = [dict() for _ in range(4)]
        slot = self._result_slots[self._slot_i % 4]
        self._slot_i += 1
        n = S * width
        if "tokens" not in slot or slot["tokens"].numel() < n:
            cap = pow2_bucket(n, 256)
            slot["tokens"] = torch.empty(cap, dtype=torch.int32, pin_memory=self.is_cuda)
            slot["logprobs"] = torch.empty(cap, dtype=torch.float32, pin_memory=self.is_cuda)
        if top > 0 and ("top_vals" not in slot or slot["top_vals"].numel() < n * top):
            cap = pow2_bucket(n * top, 256)
            slot["top_vals"] = torch.empty(cap, dtype=torch.float32, pin_memory=self.is_cuda)
            slot["top_ids"] = torch.empty(cap, dtype=torch.int32, pin_memory=self.is_cuda)
        return slot

    # ------------------------------------------------------------------ execution
    def choose_caps(self, batch_tokens: int, batch_seqs: int, max_blocks: int, sample_rows: int, decode_only: bool,
                    pen_cap: int = 32, graphable: bool = True) -> Tuple[int, int, int, int, int, bool]:
        """Capacities of the packed layout for this step; `padded` tells whether the step runs at the bucket
        size (graph replay) or at its real size (eager).  Decode-only steps use the reference's token buckets;
        steps that contain prefill tokens (when `enable_prefill_piecewise_graph` is on) round the token count up to
        a multiple of 128, which is also the row tile of the GEMM kernels."""
        use_graph = (self.is_cuda and self.opt.enable_graph and graphable and
                     (decode_only or self.opt.enable_prefill_piecewise_graph) and
                     batch_tokens <= self.opt.max_tokens_for_graph_mode)
        if use_graph:
            T = graph_bucket(batch_tokens) if (decode_only or batch_tokens <= 64) else (batch_tokens + 127) // 128 * 128
            B = graph_bucket(batch_seqs)
            S = graph_bucket(sample_rows)
            MB = pow2_bucket(max_blocks, 8)
            return T, max(B, 1), MB, max(S, 1), pow2_bucket(pen_cap, 32), True
        return max(batch_tokens, 1), max(batch_seqs, 1), max(max_blocks, 1), max(sample_rows, 1), pow2_bucket(pen_cap, 32), False

    @torch.inference_mode()
    def execute(self, layout: "_core.BatchLayout", padded: bool, patch_placeholders: bool = False,
                want_embeddings: int = 0) -> StepResult:
        """Run one step whose packed inputs are already in `self._host[:layout.total_words]`.  `want_embeddings`: 0 = sample
        tokens; 1 = return the pooled embedding of every sampling row instead; 2 = return, in the same place, the
        probability of the "yes" token against the "no" token at every sampling row (`self.yes_no_ids`)."""
        L = layout
        host = self._host
        header = host[L.header:L.header + 32].numpy().copy()
        if self.is_cuda:
            self._dev[:L.total_words].copy_(host[:L.total_words], non_blocking=True)
            self.h2d_bytes += L.total_words * 4
        inp = StepInput(self._dev, L, header, padded=padded)
        if patch_placeholders and self._last_tokens is not None:
            # token id -(j+1) stands for "j-th sample of the previous step"
            tok = inp.tokens
            idx = (-tok - 1).clamp_min(0).long().clamp_max(self._last_tokens.numel() - 1)
            tok.copy_(torch.where(tok < 0, self._last_tokens.index_select(0, idx), tok))
        # Tensor-parallel greedy steps keep the logits sharded: every rank takes the maximum of its vocabulary shard and
        # only (value, index) pairs are exchanged, instead of gathering [rows, vocab] logits on every rank.
        tp = self.comm.tp_size
        shardable = (tp > 1 and not want_embeddings and not inp.any_logprobs and not inp.any_penalty and inp.n_spec == 0 and
                     self.args.vocab_size % tp == 0 and os.environ.get("XLLM_TP_GREEDY_SHARDED", "1") != "0")
        # Steps that sample can stay sharded too when every sampling row has a top-k of at most 64: each rank extracts the
        # candidates of its vocabulary slice and only those are exchanged (`_sample_from_shards`).  Opt-in
        # (XLLM_TP_SAMPLE_SHARDED=1): over NVLink the gather of 256 x 151936 logits costs 0.23 ms with the sampler, the
        # candidate exchange 0.59 ms (200 times fewer bytes, but a dozen small launches); it pays on slower links.
        local = shardable and (inp.all_greedy or (self._shard_sampling_ok and 1 <= inp.max_top_k <= self.SHARD_TOPK_MAX and
                                                  os.environ.get("XLLM_TP_SAMPLE_SHARDED", "0") == "1"))
        if padded and self.is_cuda and not getattr(self, "no_graph", False):
            hidden, logits = self._graph_executor().run(inp, gather_logits=not local)
        else:
            hidden = self.model.forward(inp, self.kv_caches)
            logits = None if want_embeddings == 1 else self.model.logits(hidden, inp.sample_idx, not local)
        return self._finish(inp, hidden, logits, want_embeddings, sharded_logits=local)

    def _greedy_from_shards(self, logits: torch.Tensor) -> torch.Tensor:
        """argmax over the whole vocabulary from per-rank shards: ties go to the lowest token id, as a plain argmax."""
        tp, r = self.comm.tp_size, self.comm.tp_rank
        vals, idx = logits.max(dim=-1)
        cand = torch.stack([vals.float(), (idx + r * logits.shape[-1]).int().view(torch.float32)], dim=-1).contiguous()
        allc = self.comm.all_gather(cand, dim=0).view(tp, logits.shape[0], 2)
        best = allc[:, :, 0].argmax(dim=0)                   # first maximum = lowest rank = lowest token id
        ids = allc[:, :, 1].contiguous().view(torch.int32)
        self.sharded_greedy_steps += 1
        return ids.gather(0, best[None, :])[0].contiguous()

    SHARD_TOPK_MAX = 64          # largest top-k a step may ask for and still sample from per-shard candidates
    SHARD_WIDTH = 96             # candidate places per rank and row (top-k plus room for ties at the k-th logit)

    def _sample_from_shards(self, logits: torch.Tensor, inp: StepInput) -> torch.Tensor:
        """Sampling over the whole vocabulary from per-rank shards of the logits.  The k largest logits of a row (and the
        ties at the k-th) are among the k largest of every shard, so each rank contributes at most SHARD_WIDTH (value,
        token id) pairs per row, the ranks exchange those, and the sampler (top-k, top-p, draw in vocabulary order) runs
        on the merged candidates: rank-major order is token-id order, so the draw equals that of the unsharded step.
        A row with more ties than fit raises a flag that is read one step later; from then on the logits are gathered."""
        tp, r = self.comm.tp_size, self.comm.tp_rank
        S, Vs = logits.shape
        W = self.SHARD_WIDTH
        if self._shard_over_event is not None and self._shard_over_event.query():
            if int(self._shard_over_host[0]) != 0:
                self._shard_sampling_ok = False
                self.shard_sampling_overflows += 1
            self._shard_over_event = None
        vals, ids, over = ops.topk_candidates(logits, inp, r * Vs, W)
        packed = torch.cat([vals, ids.view(torch.float32), over.view(torch.float32).expand(S, 1)], dim=-1).contiguous()
        allc = self.comm.all_gather(packed, dim=0).view(tp, S, 2 * W + 1)
        mv = allc[:, :, :W].permute(1, 0, 2).reshape(S, tp * W).contiguous()
        mi = allc[:, :, W:2 * W].contiguous().view(torch.int32).view(tp, S, W).permute(1, 0, 2).reshape(S, tp * W)
        pick, _, _, _ = ops.sample(mv, inp)
        tokens = mi.gather(1, pick.long().clamp_(0, tp * W - 1)[:, None])[:, 0].contiguous()
        if logits.is_cuda:
            any_over = allc[:, 0, 2 * W].contiguous().view(torch.int32).max().reshape(1)
            self._shard_over_host.copy_(any_over, non_blocking=True)
            self._shard_over_event = torch.cuda.Event()
            self._shard_over_event.record()
        elif int(allc[:, 0, 2 * W].contiguous().view(torch.int32).max()) != 0:
            self._shard_sampling_ok = False
            self.shard_sampling_overflows += 1
        self.sharded_sampling_steps += 1
        return tokens

    def _finish(self, inp: StepInput, hidden, logits, want_embeddings: int, sharded_logits: bool = False) -> StepResult:
        S = inp.S
        batch_id = int(np.uint32(inp.header[12])) | (int(np.uint32(inp.header[13])) << 32)
        if want_embeddings == 2:
            # Qwen3-reranker scoring (sampler.cpp:78-90 of the reference): softmax over the logits of "no" and "yes" at
            # the position that would generate the answer; the score is the probability of "yes"
            no_id, yes_id = self.yes_no_ids
            pair = logits[:, [no_id, yes_id]].float()
            score = torch.softmax(pair, dim=-1)[:inp.n_sample, 1:2].cpu()
            return StepResult(batch_id, inp.n_sample, 1, torch.zeros(max(S, 1), dtype=torch.int32), None, None, None, None, score)
        if want_embeddings:
            emb = self.model.pooled_embedding(hidden, inp.sample_idx)[:inp.n_sample].float().cpu()
            return StepResult(batch_id, inp.n_sample, 1, torch.zeros(max(S, 1), dtype=torch.int32), None, None, None, None, emb)
        if sharded_logits:
            tokens = self._greedy_from_shards(logits) if inp.all_greedy else self._sample_from_shards(logits, inp)
            lp, tv, ti = None, None, None
        else:
            tokens, lp, tv, ti = ops.sample(logits, inp)
        self._last_tokens = tokens
        slot = self._result_slot(S, 1, inp.max_top_logprobs if inp.any_logprobs else 0)
        slot["tokens"][:S].copy_(tokens, non_blocking=True)
        self.d2h_bytes += S * 4
        out_lp = out_tv = out_ti = None
        if lp is not None:
            slot["logprobs"][:S].copy_(lp, non_blocking=True)
            out_lp = slot["logprobs"][:S]
            self.d2h_bytes += S * 4
            if tv is not None:
                k = tv.shape[-1]
                slot["top_vals"][:S * k].copy_(tv.reshape(-1), non_blocking=True)
                slot["top_ids"][:S * k].copy_(ti.reshape(-1), non_blocking=True)
                out_tv, out_ti = slot["top_vals"][:S * k].view(S, k), slot["top_ids"][:S * k].view(S, k)
        ev = None
        if self.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
        return StepResult(batch_id, inp.n_sample, 1, slot["tokens"][:S], out_lp, out_tv, out_ti, ev)

    def _graph_executor(self):
        if self._graphs is None:
            from .graph_executor import CudaGraphExecutor
            self._graphs = CudaGraphExecutor(self)
        return self._graphs
