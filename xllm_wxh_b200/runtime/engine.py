"""LLMEngine: scheduler (C++) + rank-local worker + the step protocol between ranks.

Role of the reference's LLMEngine / DistManager / WorkerServer trio
(xllm/core/distributed_runtime/llm_engine.cpp:71-322 init, 375-678 KV sizing, 1014-1150 step;
dist_manager.cpp:144-318; worker_server.cpp:66-242): one process per GPU; rank 0 additionally runs the
scheduler.  Every step rank 0 packs the inputs of each attention-DP group into one pinned message and
publishes it to the other ranks through a shared-memory broadcast channel (the reference uses brpc or
a shared-memory ring, remote_worker.cpp:172-190); all ranks then run the same kernels; the first rank
of every DP group reports the sampled tokens.  Collectives between ranks go through NCCL or the fused
NVLink kernels, never through this control channel.
"""
from __future__ import annotations

import logging
import os
import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _core
from ..config import Options
from ..models.args import ModelArgs, load_model_args, preset
from ..parallel.comm import Comm, ParallelConfig, init_comm
from .worker import StepResult, Worker, pow2_bucket

log = logging.getLogger("xllm.engine")

CTRL_WORDS = 128         # [0:4) command, [4:60) per-DP-rank batch descriptors, [64:72) rows each DP rank runs this step
CMD_STEP, CMD_STOP, CMD_DUMMY, CMD_CALL = 1, 2, 3, 4
_MAX_DP = 8


def resolve_model_args(model: str) -> Tuple[ModelArgs, Optional[str]]:
    """`preset:<name>` -> random-initialised architecture; otherwise a HF model directory."""
    if model.startswith("preset:"):
        return preset(model.split(":", 1)[1]), None
    return load_model_args(model), model


class LLMEngine:
    def __init__(self, options: Options, model_args: Optional[ModelArgs] = None, model=None,
                 rank: Optional[int] = None, world_size: Optional[int] = None):
        self.opt = options.validate()
        devices = self.opt.device_list()
        env_world = int(os.environ.get("WORLD_SIZE", "1"))
        self.world_size = world_size if world_size is not None else (env_world if env_world > 1 else len(devices))
        self.rank = rank if rank is not None else int(os.environ.get("RANK", "0"))
        local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        if model_args is None:
            model_args, self.model_dir = resolve_model_args(self.opt.model)
        else:
            self.model_dir = None
        self.args = model_args
        if self.opt.max_model_len > 0:
            self.args.max_position_embeddings = min(self.args.max_position_embeddings, self.opt.max_model_len)
        first = devices[0]
        if first.startswith("cuda"):
            device = f"cuda:{local_rank}" if (self.world_size > 1 and len(devices) < self.world_size) else devices[min(local_rank, len(devices) - 1)]
        else:
            device = "cpu"
        self.device = torch.device(device)
        self.numa_node = -1
        if self.device.type == "cuda" and self.opt.enable_numa_binding:
            from ..platform import numa
            self.numa_node = numa.bind_rank_to_device(self.device.index or 0)
        pcfg = ParallelConfig(world_size=self.world_size, rank=self.rank, dp_size=self.opt.dp_size,
                              ep_size=self.opt.ep_size if self.opt.ep_size > 1 else 1,
                              tp_mode="nccl" if self.opt.communication_backend == "nccl" else "fused",
                              ep_mode="fused" if self.opt.expert_parallel_degree == 2 else "allreduce")
        pcfg.mlp_replicated = self._want_replicated_mlp(pcfg)
        # EPLB moves experts between the ranks of an expert-parallel group; without such a group its table covers one rank
        pcfg.moe_experts_over_tp = pcfg.ep_size == 1 and pcfg.tp_size > 1 and not self.opt.enable_eplb
        self._init_distributed()
        self.comm = init_comm(pcfg, self.device) if self.world_size > 1 else Comm(pcfg)
        self.worker = Worker(self.args, self.opt, self.comm, device, model=model)
        if model is None:
            self._load_model()
        self._setup_parallel_kernels()
        self.block_size = self.opt.block_size
        nb = self.worker.profile_kv_blocks()
        if self.world_size > 1:
            t = torch.tensor([nb], dtype=torch.int64, device=self.device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
            nb = int(t.item())
        self.num_blocks = nb
        # the cache that another instance maps: the decode side's when KV is pushed, the prefill side's when it is pulled
        mapped_role = "PREFILL" if self.opt.kv_cache_transfer_mode == "PULL" else "DECODE"
        self.worker.allocate_kv_cache(nb, ipc=self.opt.enable_disagg_pd and self.opt.instance_role == mapped_role)
        self.worker._ensure_staging(self._max_message_words() // max(1, self.opt.dp_size))
        # host-memory tier of the prefix cache (every rank keeps the host copy of its own shard of each block)
        self.host_tier = None
        n_host = int(self.opt.host_blocks_factor * (nb - 1)) if self.opt.enable_prefix_cache else 0
        if n_host >= 1:
            from .host_kv_tier import HostKvTier
            self.host_tier = HostKvTier(self.worker.kv_caches, n_host, self.device)
        # shared block store behind the host tier.  Every rank writes its own share of a block through and fetches it
        # back (a share is named by the rank's place in its tensor-parallel group); the prefix keys live in rank 0's
        # scheduler and travel with the step message.
        self.kv_store = None
        self.external_step_lock = None               # set by the master: held while a step is built and run
        self.store_prefetched_blocks = 0
        self._store_put_keys: List = []
        if self.opt.enable_kvcache_store and self.opt.store_master_server_address:
            if self.host_tier is None:
                log.warning("--enable_kvcache_store needs the host tier (--host_blocks_factor); store not used")
            elif self.opt.dp_size > 1 and self.world_size == 1:
                log.warning("attention DP in one process has one cache only; store not used")
            else:
                from ..service.kv_store import KvStoreClient, model_namespace, weights_fingerprint
                name = self.opt.model_id or os.path.basename(os.path.normpath(str(self.opt.model)))
                self._store_fp = weights_fingerprint(self.model_dir, self.opt.random_seed)
                self._store_ns = model_namespace(name, self.args, self.block_size, self.host_tier.stride, self._store_fp,
                                                 self.opt.kv_cache_dtype)
                self.kv_store = KvStoreClient(self.opt.store_master_server_address)
                self.host_tier.attach_store(self.kv_store, self.comm.tp_rank, self.comm.tp_size, self._store_ns)
        self.scheduler: Optional["_core.Scheduler"] = None
        self._chan = None
        self._res_chans: Dict[int, "_core.ShmChannel"] = {}
        self._msg: Optional[torch.Tensor] = None
        self._inflight: List[Tuple[List, Optional[StepResult], List]] = []
        self._setup_channels()
        if self.rank == 0:
            so = _core.SchedulerOptions()
            so.max_tokens_per_batch = self.opt.max_tokens_per_batch
            so.max_seqs_per_batch = self.opt.max_seqs_per_batch
            so.enable_chunked_prefill = self.opt.enable_chunked_prefill
            so.max_tokens_per_chunk_for_prefill = self.opt.max_tokens_per_chunk_for_prefill
            so.prefill_only_batches = self.opt.num_speculative_tokens > 0 or self.opt.enable_prefill_sp
            so.use_zero_evict = self.opt.use_zero_evict
            so.max_decode_token_per_sequence = self.opt.max_decode_token_per_sequence
            so.num_speculative_tokens = self.opt.num_speculative_tokens
            # a multi-step MTP draft writes its own KV up to k - 1 positions past the rows of the step
            if self.opt.num_speculative_tokens > 1 and self.opt.speculative_algorithm.upper() in ("MTP", "EAGLE3"):
                so.spec_extra_slots = self.opt.num_speculative_tokens
            so.prefill_scheduling_memory_usage_threshold = self.opt.prefill_scheduling_memory_usage_threshold
            so.enable_online_preempt_offline = self.opt.enable_online_preempt_offline
            so.priority_strategy = self.opt.priority_strategy
            so.chunked_match_frequency = self.opt.chunked_match_frequency
            so.dp_size = self.opt.dp_size
            so.handoff_after_prefill = self.opt.enable_disagg_pd and self.opt.instance_role == "PREFILL"
            so.host_blocks_factor = self.opt.host_blocks_factor if self.host_tier is not None else 0.0
            so.use_mix_scheduler = self.opt.use_mix_scheduler
            so.enable_latency_aware_schedule = self.opt.enable_latency_aware_schedule
            so.max_global_ttft_ms = float(self.opt.max_global_ttft_ms)
            so.max_global_tpot_ms = float(self.opt.max_global_tpot_ms)
            so.aggressive_coeff = self.opt.aggressive_coeff
            so.starve_threshold = self.opt.starve_threshold
            so.enable_starve_prevent = self.opt.enable_starve_prevent
            self.scheduler = _core.Scheduler(so, nb, self.block_size, self.opt.enable_prefix_cache, self.opt.xxh3_128bits_seed)
        self._tls = threading.local()
        from .sleep import SleepState
        self._sleep_state = SleepState()
        self.bytes_released_by_sleep = 0
        self.step_count = 0
        self.last_step_ms = 0.0
        # host-side phase times of the most recent steps (ms): schedule, pack+publish, kernel issue, wait for results
        self.host_trace: List[Tuple[float, float, float, float]] = []
        self._t_pack = self._t_issue = 0.0
        self.top_logprobs: Dict[Tuple[int, int], List] = {}
        self._marks: Dict[int, object] = {}
        self.kv_transfer = None          # set when linked to a decode instance (parallel/kv_transfer.py)
        self.kv_sources = {}             # PULL mode, decode side: prefill instance index -> its mapped cache
        self.kv_transfer_peers: Dict[int, object] = {}     # further decode instances (link index >= 1)
        self.transfer_pairs_provider = None
        self._pack_hook = None           # callable(engine, msg, layout, offset): edit a packed batch before it is published
        self.pre_execute_hooks = []      # callables(engine, batches) run on rank 0 before a step is published

    # ------------------------------------------------------------------ set-up
    def bind_thread(self):
        """CUDA's current device is per host thread and a new thread starts on device 0: every thread that drives the
        engine (serving loop, control-service handlers, executor threads) binds this rank's device first."""
        if self.device.type == "cuda" and getattr(self._tls, "bound", None) != self.device.index:
            torch.cuda.set_device(self.device)
            self._tls.bound = self.device.index

    def _init_distributed(self):
        if self.world_size <= 1 or torch.distributed.is_initialized():
            return
        addr, port = self.opt.master_node_addr.rsplit(":", 1)
        os.environ.setdefault("MASTER_ADDR", addr)
        os.environ.setdefault("MASTER_PORT", port)
        backend = "nccl" if self.device.type == "cuda" else "gloo"
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        kw = {"device_id": self.device} if backend == "nccl" else {}
        torch.distributed.init_process_group(backend, rank=self.rank, world_size=self.world_size, **kw)

    def _want_replicated_mlp(self, pcfg) -> bool:
        """Whether every tensor-parallel rank keeps the whole dense MLP (`--tp_mlp_mode`).  A step of T rows then runs the
        MLP of T / tp rows per rank with no collective inside it; what it costs is memory (tp times the sharded MLP) and,
        for short steps, weight traffic, so short steps keep using the rank's slice of the same tensors."""
        a, mode = self.args, self.opt.tp_mlp_mode
        tp = pcfg.tp_size
        if tp < 2 or self.device.type != "cuda" or pcfg.tp_mode != "fused" or mode == "tp" or a.n_routed_experts > 0:
            return False
        if a.intermediate_size % (16 * tp) or a.dtype not in ("bfloat16", "auto"):
            return False
        if mode == "rows":
            return True
        # auto: measured at TP 4 on a 1279-row step of Qwen3-8B the row-sharded MLP (320 rows against whole weights: two
        # partly filled 256-row tiles) lost to the sharded one (11.6 against 10.9 ms per step), so it stays opt-in
        return False

    def _load_model(self):
        m = self.worker.model
        if self.model_dir is None:
            m.init_random(self.opt.random_seed)
        else:
            from ..utils.safetensors_io import CheckpointReader
            m.load_weights(CheckpointReader(self.model_dir))
        if hasattr(m, "finalize_weights"):
            m.finalize_weights()

    def _setup_parallel_kernels(self):
        if self.world_size > 1 and self.device.type == "cuda":
            from ..parallel import fused_tp
            fused_tp.attach(self)
        if self.world_size > 1:
            from ..parallel import fused_ep
            fused_ep.attach(self)
        self.eplb = None
        if self.opt.enable_eplb:
            from . import eplb
            eplb.attach(self)

    def _chan_name(self, suffix: str) -> str:
        port = os.environ.get("MASTER_PORT", self.opt.master_node_addr.rsplit(":", 1)[-1])
        return f"/xllm_b200_{os.getuid()}_{port}_{suffix}"

    def _setup_channels(self):
        if self.world_size <= 1:
            return
        cap_words = CTRL_WORDS + self._max_message_words() + self._xfer_words()
        name = self._chan_name("step")
        if self.rank == 0:
            self._chan = _core.ShmChannel(name, cap_words * 4, self.world_size - 1, True)
        torch.distributed.barrier()
        if self.rank != 0:
            self._chan = _core.ShmChannel(name, cap_words * 4, self.world_size - 1, False)
        tp = self.comm.tp_size
        for d in range(1, self.opt.dp_size):
            rname = self._chan_name(f"res{d}")
            if self.rank == 0:
                self._res_chans[d] = _core.ShmChannel(rname, 1 << 22, 1, True)
        torch.distributed.barrier()
        if self.rank != 0 and self.comm.tp_rank == 0 and self.comm.dp_rank > 0:
            self._res_chans[self.comm.dp_rank] = _core.ShmChannel(self._chan_name(f"res{self.comm.dp_rank}"), 1 << 22, 1, False)
        torch.distributed.barrier()

    def _max_message_words(self) -> int:
        o = self.opt
        mb = (self.args.max_position_embeddings + self.block_size - 1) // self.block_size + 1
        L = _core.BatchLayout(o.max_tokens_per_batch + 16, o.max_seqs_per_batch + 16, pow2_bucket(mb, 8),
                              (o.max_seqs_per_batch + 16) * (1 + o.num_speculative_tokens), 1 << 16)
        return L.total_words * max(1, o.dp_size)

    def _xfer_words(self) -> int:
        """Room for the host-tier copy lists of a step: at most one offload and one load per device block and DP rank."""
        if self.host_tier is None:
            return 0
        keys = 4 * self.num_blocks + 1 if self.kv_store is not None else 0      # prefix keys of the offloaded blocks
        return (4 * self.num_blocks + 4 + keys) * max(1, self.opt.dp_size)

    def _ensure_msg(self, words: int):
        need = CTRL_WORDS + words
        if self._msg is None or self._msg.numel() < need:
            n = pow2_bucket(need, 1 << 16)
            old = self._msg
            self._msg = torch.zeros(n, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            if old is not None:
                self._msg[:old.numel()].copy_(old)       # keep what has been packed so far
        return self._msg

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_tokens: Sequence[int], sampling: Optional["_core.SamplingParams"] = None,
                    stop: Optional["_core.StopCriteria"] = None, n: int = 1, best_of: int = 1, priority: int = 0,
                    offline: bool = False, ext_id: str = "", ttft_slo_ms: float = 0.0, tpot_slo_ms: float = 0.0,
                    ttft_weight: int = 1, tpot_weight: int = 1) -> int:
        sp = sampling or _core.SamplingParams()
        st = stop or _core.StopCriteria()
        if st.max_context_len > self.args.max_position_embeddings:
            st.max_context_len = self.args.max_position_embeddings
        if self.kv_store is not None:
            self._store_prefetch(list(prompt_tokens))
        return self.scheduler.add_request(list(prompt_tokens), sp, st, n, best_of, priority, offline, ext_id, ttft_slo_ms,
                                          tpot_slo_ms, int(ttft_weight), int(tpot_weight))

    def _store_prefetch(self, tokens: List[int]) -> int:
        """Complete a new prompt's prefix from the shared store: blocks that neither the device cache nor the host tier
        holds, and that the store has in an unbroken run, are fetched into host blocks which the scheduler publishes under
        their keys; the request then finds them like any other host-tier hit (prefetch_from_storage in the reference,
        hierarchy_block_manager_pool.cpp:209-262).  Runs on the thread that takes the request in; only the short look-up
        and the adoption hold the step lock, the network transfer does not.  Returns the blocks fetched."""
        import contextlib
        from ..service.kv_store import block_key
        bs = self.block_size
        max_blocks = (len(tokens) - 1) // bs
        if max_blocks <= 0:
            return 0
        world = self.comm.tp_size
        dp = max(1, self.opt.dp_size)
        pk = _core.prefix_block_keys(tokens[:max_blocks * bs], bs, self.opt.xxh3_128bits_seed)
        per_rank = [[block_key(k, r, world, self._store_ns) for k in pk] for r in range(world)]
        found = self.kv_store.batch_exist([k for ks in per_rank for k in ks])
        n = len(pk)
        whole = [all(found[r * n + i] for r in range(world)) for i in range(n)]      # every rank's share is there
        upto = next((i for i, f in enumerate(whole) if not f), n)
        if upto == 0:
            return 0
        lock = self.external_step_lock or contextlib.nullcontext()
        with lock:
            # the DP rank that already holds most of the prompt takes the rest (the scheduler will place the request there);
            # with nothing cached anywhere, the emptiest rank
            seen = [self.scheduler.prefix_presence(d, tokens) for d in range(dp)]
            d = max(range(dp), key=lambda r: (max(seen[r]), self.scheduler.block_manager(r).num_available_blocks))
        dev, host = seen[d]
        if upto <= max(dev, host):
            return 0
        upto = min(upto, host + 512)                   # bound the time one request may spend fetching
        if self.world_size == 1:
            data = []
            for i in range(host, upto, 16):             # a few records per message: the socket's time limit is per message
                part = self.kv_store.batch_get(per_rank[0][i:min(i + 16, upto)])
                data += part
                if any(d is None for d in part):
                    break
            n_ok = next((i for i, d in enumerate(data) if d is None or len(d) != self.host_tier.stride), len(data))
            upto = host + n_ok
            if upto <= max(dev, host):
                return 0
            with lock:
                adopted = self.scheduler.host_adopt(d, tokens, host, upto)
                for idx, hid in adopted:
                    self.host_tier.fill(hid, data[idx - host])
        else:
            # several ranks: each fetches its own share inside a control operation between two steps; if one of them
            # comes back short the adopted blocks leave the host cache again
            import json
            with lock:
                adopted = self.scheduler.host_adopt(d, tokens, host, upto)
                if adopted:
                    payload = json.dumps({"keys": [list(pk[i]) for i, _ in adopted], "hids": [h for _, h in adopted]}).encode()
                    oks = self._control(self.OP_STORE_FETCH, d, payload)
                    if not all(oks):
                        self.scheduler.host_manager(d).drop_cached([h for _, h in adopted])
                        adopted = []
        self.store_prefetched_blocks += len(adopted)
        return len(adopted)

    def cancel(self, request_id: int):
        self.scheduler.cancel(request_id)
        self.drop_top_logprobs(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or bool(self._inflight)

    # ------------------------------------------------------------------ stepping (rank 0)
    def _publish(self, batches, patch: bool, want_emb: int = 0):
        """Pack every DP batch into the message, send it, and run the local worker.  Returns the local result."""
        self.bind_thread()
        o = self.opt
        specs, total = [], 0
        need_dummy = self.world_size > 1 and (self.comm.ep_size > 1) and any(not b.empty for b in batches)
        for b in batches:
            if b.empty:
                specs.append(None)
                continue
            decode_only = b.forward_type == 2 and b.num_spec == 0
            T, B, MB, S, P, padded = self.worker.choose_caps(b.num_tokens, b.num_seqs, b.max_blocks, b.num_sample_rows,
                                                            decode_only, graphable=b.num_spec == 0 and not want_emb)
            L = self.worker.layout_for(T, B, MB, S, P)
            specs.append([L, padded, total])
            total += L.total_words
        msg = self._ensure_msg(total)
        ctrl = msg[:CTRL_WORDS].numpy()
        ctrl[:] = 0
        ctrl[0], ctrl[1], ctrl[2], ctrl[3] = CMD_STEP, int(patch), int(want_emb), len(batches)
        for d, (b, sp) in enumerate(zip(batches, specs)):
            base = 4 + d * 7
            if sp is None:
                ctrl[base] = -2 if need_dummy else -1
                continue
            L, padded, off = sp
            while True:
                rc = b.build(L, msg.data_ptr() + (CTRL_WORDS + off) * 4, L.total_words, self.block_size)
                if rc == 0:
                    break
                if rc == -1:
                    raise RuntimeError("batch does not fit its layout")
                P = pow2_bucket(int(-rc - 16), 32)          # penalty section too small: widen and repack
                if off + self.worker.layout_for(L.T_cap, L.B_cap, L.MB_cap, L.S_cap, P).total_words > msg.numel() - CTRL_WORDS \
                        or d + 1 < len(batches):
                    raise RuntimeError("penalty table overflow")
                L = self.worker.layout_for(L.T_cap, L.B_cap, L.MB_cap, L.S_cap, P)
                msg = self._ensure_msg(off + L.total_words)
                ctrl = msg[:CTRL_WORDS].numpy()
                sp[0] = L
                total = off + L.total_words
            ctrl[base:base + 7] = [off, L.T_cap, L.B_cap, L.MB_cap, L.S_cap, L.P_cap, int(padded)]
            ctrl[64 + d] = L.T_cap if padded else b.num_tokens
            if self._pack_hook is not None:
                self._pack_hook(self, msg, L, off)
        for d, sp in enumerate(specs):
            if sp is None:
                ctrl[64 + d] = 1 if need_dummy else 0
        if self.transfer_pairs_provider is not None:
            pairs = self.transfer_pairs_provider(batches)
            if pairs:
                msg = self._ensure_msg(total + 2 * len(pairs))
                ctrl = msg[:CTRL_WORDS].numpy()
                ctrl[72], ctrl[73] = len(pairs), total
                msg[CTRL_WORDS + total:CTRL_WORDS + total + 2 * len(pairs)] = torch.tensor(pairs, dtype=torch.int32).reshape(-1)
                total += 2 * len(pairs)
        if self.host_tier is not None:
            msg, total = self._append_transfers(msg, total)
        if self._chan is not None:
            rc = self._chan.write_ptr(msg.data_ptr(), (CTRL_WORDS + total) * 4, self.opt.rpc_channel_timeout_ms / 1e3)
            if rc != 0:
                raise RuntimeError(f"step channel write failed (code {rc}): a worker rank is not responding")
        self._t_pack = time.perf_counter()
        res = self._run_local(msg, patch, want_emb)
        self._t_issue = time.perf_counter()
        return res

    def _append_transfers(self, msg: torch.Tensor, total: int):
        """Host-tier copy lists of the step, per DP rank: [n_offloads, n_loads, (device, host) ..., (host, device) ...]."""
        words: List[int] = []
        key_words: List[int] = []
        for d, (off_list, load_list) in enumerate(self.scheduler.take_transfers()):
            if self.kv_store is not None:
                # prefix keys of this DP rank's offloaded blocks, in the order of its offload list (four words per key):
                # every rank writes its share of those blocks through to the shared store
                hm = self.scheduler.host_manager(d)
                key_words.append(len(off_list))
                if off_list:
                    key_words += np.array([hm.block_hash(h) for _, h in off_list], dtype=np.uint64).reshape(-1).view(np.int32).tolist()
            words += [len(off_list), len(load_list)]
            for a, b_ in off_list:
                words += [a, b_]
            for a, b_ in load_list:
                words += [a, b_]
        words += key_words
        msg = self._ensure_msg(total + len(words))
        ctrl = msg[:CTRL_WORDS].numpy()
        ctrl[74], ctrl[75] = len(words), total
        msg[CTRL_WORDS + total:CTRL_WORDS + total + len(words)] = torch.tensor(words, dtype=torch.int32)
        return msg, total + len(words)

    def _publish_transfers_only(self, n_batches: int) -> None:
        """A step without any batch still hands the pending host-tier copies to every rank (and lets the scheduler take
        back the device blocks it holds for copies in flight)."""
        msg = self._ensure_msg(0)
        ctrl = msg[:CTRL_WORDS].numpy()
        ctrl[:] = 0
        ctrl[0], ctrl[3] = CMD_STEP, n_batches
        for d in range(n_batches):
            ctrl[4 + d * 7] = -1
        msg, total = self._append_transfers(msg, 0)
        if self._chan is not None:
            rc = self._chan.write_ptr(msg.data_ptr(), (CTRL_WORDS + total) * 4, self.opt.rpc_channel_timeout_ms / 1e3)
            if rc != 0:
                raise RuntimeError(f"step channel write failed (code {rc}): a worker rank is not responding")
        self._host_tier_step(msg)

    def _run_local(self, msg: torch.Tensor, patch: bool, want_emb: int) -> Optional[StepResult]:
        ctrl = msg[:CTRL_WORDS].numpy()
        d = self.comm.dp_rank
        base = 4 + d * 7
        off = int(ctrl[base])
        w = self.worker
        self._host_tier_step(msg)
        if off == -1:
            return None
        impl = getattr(w.model, "moe_impl", None)
        if impl is not None:
            impl.dp_token_counts = [int(v) for v in ctrl[64:64 + max(1, self.opt.dp_size)]]
        if off == -2:
            return self._run_dummy()
        T, B, MB, S, P, padded = (int(v) for v in ctrl[base + 1:base + 7])
        L = w.layout_for(T, B, MB, S, P)
        w._ensure_staging(L.total_words)
        w.set_host(msg[CTRL_WORDS + off:CTRL_WORDS + off + L.total_words])
        by_link = self._kv_pairs_by_link(msg)
        layered = bool(by_link) and hasattr(w.model, "layer_hook") and os.environ.get("XLLM_PD_PUSH_BY_LAYER", "1") != "0"
        if layered:
            # disaggregated prefill: every layer's blocks leave for the decode instance right after the layer wrote them,
            # on a side stream, so the copy over NVLink runs beside the rest of the forward pass.  Such a step runs
            # without a CUDA graph (the pairs change from step to step).
            def hook(layer: int, _by_link=by_link):
                for link, ps in _by_link.items():
                    self._transfer_of(link).push_layer_async(ps, layer)
            w.model.layer_hook = hook
            w.no_graph = True
        try:
            res = w.execute(L, bool(padded), patch_placeholders=patch, want_embeddings=want_emb)
        finally:
            if layered:
                w.model.layer_hook = None
                w.no_graph = False
        if layered:
            for link in by_link:
                self._transfer_of(link).join()      # later steps may reuse the source blocks
        else:
            self._push_kv_pairs(msg)
        return res

    def _host_tier_step(self, msg: torch.Tensor) -> None:
        """Issue this DP rank's host-tier copies of the step (offloads, then loads) ahead of the forward; they are
        run even when the rank has no batch, because the scheduler already counts the blocks as moved."""
        if self.host_tier is None:
            return
        ctrl = msg[:CTRL_WORDS].numpy()
        n = int(ctrl[74])
        if n <= 0:
            self.host_tier.run((), ())
            return
        sec = msg[CTRL_WORDS + int(ctrl[75]):CTRL_WORDS + int(ctrl[75]) + n].numpy()
        pos = 0
        offs, loads = [], []
        for d in range(max(1, self.opt.dp_size)):
            n_off, n_load = int(sec[pos]), int(sec[pos + 1])
            pos += 2
            if d == self.comm.dp_rank:
                offs = sec[pos:pos + 2 * n_off].reshape(-1, 2).tolist()
                loads = sec[pos + 2 * n_off:pos + 2 * (n_off + n_load)].reshape(-1, 2).tolist()
            pos += 2 * (n_off + n_load)
        puts = []
        if self.kv_store is not None:
            for d in range(max(1, self.opt.dp_size)):
                if pos >= n:
                    break
                n_keys = int(sec[pos])
                if d == self.comm.dp_rank and n_keys == len(offs):
                    raw = np.ascontiguousarray(sec[pos + 1:pos + 1 + 4 * n_keys]).view(np.uint64).reshape(-1, 2)
                    puts = [(h, (int(k[0]), int(k[1]))) for (_, h), k in zip(offs, raw) if int(k[0]) or int(k[1])]
                pos += 1 + 4 * n_keys
        self.host_tier.run(offs, loads, puts)

    def _transfer_of(self, link: int):
        return self.kv_transfer if link == 0 else self.kv_transfer_peers[link]

    def _kv_pairs_by_link(self, msg: torch.Tensor) -> Dict[int, List]:
        """(source block, destination block) pairs of the step message, by decode link (the top byte of a destination names
        the link; with one decode instance it is 0)."""
        ctrl = msg[:CTRL_WORDS].numpy()
        n = int(ctrl[72])
        if n <= 0 or (self.kv_transfer is None and not self.kv_transfer_peers):
            return {}
        o = CTRL_WORDS + int(ctrl[73])
        pairs = msg[o:o + 2 * n].view(n, 2).tolist()
        by_link: Dict[int, List] = {}
        for a, d in pairs:
            by_link.setdefault(d >> 24, []).append((a, d & 0xFFFFFF))
        return by_link

    def _push_kv_pairs(self, msg: torch.Tensor) -> None:
        """Disaggregated prefill: copy the KV blocks listed in the step message into the decode instance's cache.
        Runs on the compute stream right after the forward, so a later step cannot overwrite the source blocks first."""
        for link, ps in self._kv_pairs_by_link(msg).items():
            self._transfer_of(link).push(ps)

    @torch.inference_mode()
    def _run_dummy(self) -> None:
        """A DP rank without work still takes part in the step's collectives with one padding token
        (reference: llm_model_base.h:64-67)."""
        from ..framework.step_input import StepInput
        w = self.worker
        L = w.layout_for(1, 1, 1, 1, 32)
        w._ensure_staging(L.total_words)
        host = torch.zeros(L.total_words, dtype=torch.int32)
        w.set_host(host)
        hdr = host[L.header:L.header + 32].numpy()
        hdr[0], hdr[1], hdr[17] = 1, 1, self.block_size
        host[L.q_cu + 1] = 1
        host[L.kv_lens] = 1
        w._dev[:L.total_words].copy_(host)
        inp = StepInput(w._dev, L, hdr.copy(), padded=False)
        w.model.forward(inp, w.kv_caches)
        return None

    def _collect(self, batches, local: Optional[StepResult]):
        """Gather the per-DP results on rank 0: list aligned with `batches`."""
        results: List[Optional[Tuple[np.ndarray, Optional[np.ndarray]]]] = []
        for d, b in enumerate(batches):
            if b.empty:
                results.append(None)
            elif d == 0:
                local.wait()
                n = b.num_sample_rows
                lp = local.logprobs[:n].numpy() if local.logprobs is not None else None
                results.append((local.tokens[:n].numpy(), lp, local))
            else:
                data = self._res_chans[d].read(0, 2 * self.opt.rpc_channel_timeout_ms / 1e3)
                if data is None:
                    raise RuntimeError(f"no result from dp rank {d}")
                arr = np.frombuffer(data, dtype=np.int32)
                n = int(arr[0])
                toks = arr[1:1 + n].copy()
                lp = arr[1 + n:1 + 2 * n].view(np.float32).copy() if arr.size >= 1 + 2 * n else None
                results.append((toks, lp, None))
        return results

    def step(self) -> List["_core.SeqOutput"]:
        """One scheduler iteration on rank 0.  With `enable_schedule_overlap` the tokens of step i are applied
        after step i+1 has been launched (continuous_scheduler.cpp:1085-1115)."""
        self.bind_thread()
        if self._sleep_state.level != 0:
            if sch_busy := self.scheduler.has_unfinished():
                raise RuntimeError("the engine is asleep (device memory released): wake it up before sending requests")
            return []
        t0 = time.perf_counter()
        sch = self.scheduler
        batches = sch.schedule()
        t_sched = self._t_pack = self._t_issue = time.perf_counter()
        for hook in self.pre_execute_hooks:
            hook(self, batches)
        if all(b.empty for b in batches) and self.host_tier is not None and sch.has_pending_transfers:
            self._publish_transfers_only(len(batches))
        if all(b.empty for b in batches) and not self._inflight:
            return sch.take_outputs()
        overlap = self.opt.enable_schedule_overlap
        local = None
        if not all(b.empty for b in batches):
            local = self._publish(batches, patch=overlap)
        if overlap:
            if not all(b.empty for b in batches):
                for b in batches:
                    if not b.empty:
                        sch.process_placeholder_output(b.id)
                # which rows carry top-k alternatives is read now: by the time the tokens are applied the sequences of a
                # finished request may be gone
                self._inflight.append((batches, local, [b.top_logprob_rows() if not b.empty else [] for b in batches]))
            # apply the oldest step's real tokens once a newer one is in flight (or nothing new was scheduled)
            while self._inflight and (len(self._inflight) > 1 or all(b.empty for b in batches)):
                old_batches, old_local, old_rows = self._inflight.pop(0)
                for b, r, rows in zip(old_batches, self._collect(old_batches, old_local), old_rows):
                    if r is not None:
                        self._record_top_logprobs(rows, r[2])
                        sch.update_output(b.id, r[0], r[1])
                if all(b.empty for b in batches):
                    continue
                break
        else:
            for b, r in zip(batches, self._collect(batches, local)):
                if r is not None:
                    self._apply(b, r)
        self.step_count += 1
        if self.eplb is not None and not self._inflight:
            self.eplb.on_step()         # between steps, with nothing in flight: re-plan / prepare / activate a layer
        t_end = time.perf_counter()
        self.last_step_ms = (t_end - t0) * 1e3
        if len(self.host_trace) >= 4096:
            del self.host_trace[:2048]
        self.host_trace.append(((t_sched - t0) * 1e3, (self._t_pack - t_sched) * 1e3, (self._t_issue - self._t_pack) * 1e3,
                                (t_end - self._t_issue) * 1e3))
        return sch.take_outputs()

    def export_chrome_trace(self, path: str, last: int = 0) -> int:
        """Write the host phases of the recorded steps as a Chrome / Perfetto trace (`chrome://tracing`): one track, four
        slices per step (schedule, pack + publish, kernel issue, wait for results).  Returns the number of steps written."""
        import json
        rows = self.host_trace[-last:] if last > 0 else self.host_trace
        names = ("schedule", "pack+publish", "kernel issue", "collect / wait")
        events, t = [], 0.0
        for i, r in enumerate(rows):
            for name, ms in zip(names, r):
                events.append({"name": name, "cat": "step", "ph": "X", "pid": self.rank, "tid": 0, "ts": t * 1e3,
                               "dur": max(ms, 0.0) * 1e3, "args": {"step": i}})
                t += max(ms, 0.0)
        with open(path, "w") as f:
            json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
        return len(rows)

    def host_trace_summary(self, last: int = 0) -> Dict[str, float]:
        """Mean host time per step of each phase over the `last` most recent steps (all recorded ones when 0)."""
        rows = self.host_trace[-last:] if last > 0 else self.host_trace
        if not rows:
            return {}
        n = len(rows)
        names = ("schedule_ms", "pack_publish_ms", "kernel_issue_ms", "collect_wait_ms")
        return {k: sum(r[i] for r in rows) / n for i, k in enumerate(names)}

    def _record_top_logprobs(self, rows, local) -> None:
        """Keep the top-k alternatives of the sampled tokens of the entries that asked for them, keyed by (request,
        sequence index); the master pops them with the token, `drop_top_logprobs` removes what a cancelled or finished
        request left behind."""
        if not rows or local is None or local.top_ids is None:
            return
        ti, tv = local.top_ids.numpy(), local.top_vals.numpy()
        for req, idx, row, n_top in rows:
            if row < ti.shape[0]:
                self.top_logprobs.setdefault((req, idx), []).append((ti[row, :n_top].copy(), tv[row, :n_top].copy()))

    def drop_top_logprobs(self, request_id: int) -> None:
        for key in [k for k in self.top_logprobs if k[0] == request_id]:
            del self.top_logprobs[key]

    def _apply(self, batch, result):
        toks, lps, local = result
        self._record_top_logprobs(batch.top_logprob_rows(), local)
        self.scheduler.process_output(batch.id, toks, lps)

    # ------------------------------------------------------------------ worker ranks
    def worker_loop(self):
        """Ranks != 0: execute published steps until told to stop."""
        assert self.rank != 0
        reader = self.rank - 1
        cap = CTRL_WORDS + self._max_message_words() + self._xfer_words()
        msg = self._ensure_msg(cap - CTRL_WORDS)
        while True:
            rc = self._chan.read_into(reader, msg.data_ptr(), msg.numel() * 4, 3600.0)
            if rc == 3:
                break
            if rc != 0:
                raise RuntimeError(f"step channel read failed (code {rc})")
            ctrl = msg[:CTRL_WORDS].numpy()
            cmd = int(ctrl[0])
            if cmd == CMD_STOP:
                if self.host_tier is not None:
                    self.host_tier.flush_store()
                break
            if cmd == CMD_CALL:
                nbytes = int(ctrl[3])
                payload = bytes(msg[CTRL_WORDS:CTRL_WORDS + (nbytes + 3) // 4].numpy().view(np.uint8)[:nbytes]) if nbytes else b""
                self._do_control(int(ctrl[1]), int(ctrl[2]), payload)
                continue
            if cmd != CMD_STEP:
                continue
            res = self._run_local(msg, bool(ctrl[1]), int(ctrl[2]))       # ctrl[2]: 0 tokens, 1 pooled embeddings, 2 yes / no scores
            d = self.comm.dp_rank
            if res is not None and self.comm.tp_rank == 0 and d > 0:
                res.wait()
                n = res.n_sample * res.width
                out = np.empty(1 + 2 * n, dtype=np.int32)
                out[0] = n
                out[1:1 + n] = res.tokens[:n].numpy()
                if res.logprobs is not None:
                    out[1 + n:] = res.logprobs[:n].numpy().view(np.int32)
                else:
                    out = out[:1 + n]
                self._res_chans[d].write(out.tobytes(), 60.0)

    # ------------------------------------------------------------------ control calls (timing, barriers)
    OP_BARRIER_SYNC, OP_MARK, OP_ELAPSED, OP_GATHER_HANDLES, OP_LINK_KV, OP_SLEEP, OP_WAKEUP, OP_WEIGHT_HANDLES, OP_STORE_FETCH, OP_PULL_KV = 1, 2, 3, 4, 5, 6, 7, 8, 9, 10

    def _control(self, op: int, arg: int = 0, payload: bytes = b""):
        """Rank 0: make every rank run a control operation between steps, then run it locally."""
        if self._chan is not None:
            words = (len(payload) + 3) // 4
            msg = self._ensure_msg(words)
            ctrl = msg[:CTRL_WORDS].numpy()
            ctrl[:] = 0
            ctrl[0], ctrl[1], ctrl[2], ctrl[3] = CMD_CALL, op, arg, len(payload)
            if payload:
                msg[CTRL_WORDS:CTRL_WORDS + words].numpy().view(np.uint8)[:len(payload)] = np.frombuffer(payload, dtype=np.uint8)
            rc = self._chan.write_ptr(msg.data_ptr(), (CTRL_WORDS + words) * 4, self.opt.rpc_channel_timeout_ms / 1e3)
            if rc != 0:
                raise RuntimeError(f"control channel write failed (code {rc})")
        return self._do_control(op, arg, payload)

    def _do_control(self, op: int, arg: int, payload: bytes = b""):
        self.bind_thread()
        if op >= 100:                                   # expert-parallel load balancing commands (runtime/eplb.py)
            return self.eplb.do_control(op, arg, payload) if self.eplb is not None else None
        if op == self.OP_GATHER_HANDLES:
            from ..parallel.kv_transfer import export_cache_handles
            mine = export_cache_handles(self.transfer_caches())
            if self.world_size > 1:
                out = [None] * self.world_size
                torch.distributed.all_gather_object(out, mine)
                return out
            return [mine]
        if op == self.OP_STORE_FETCH:
            import json
            from ..service.kv_store import block_key
            req = json.loads(payload.decode())
            ok = True
            if self.comm.dp_rank == arg:                 # the ranks of the DP group that takes the blocks
                keys = [block_key((int(k[0]), int(k[1])), self.comm.tp_rank, self.comm.tp_size, self._store_ns) for k in req["keys"]]
                data = self.kv_store.batch_get(keys) if self.kv_store is not None else [None] * len(keys)
                ok = all(d is not None and len(d) == self.host_tier.stride for d in data)
                if ok:
                    for hid, d in zip(req["hids"], data):
                        self.host_tier.fill(int(hid), d)
            if self.world_size > 1:
                oks = [None] * self.world_size
                torch.distributed.all_gather_object(oks, ok)
                return oks
            return [ok]
        if op == self.OP_WEIGHT_HANDLES:
            from .sleep import weight_manifest
            from .weight_transfer import _export_handles
            mine = _export_handles(weight_manifest(self.worker.model, self.device)[1])
            if self.world_size > 1:
                out = [None] * self.world_size
                torch.distributed.all_gather_object(out, mine)
                return out
            return [mine]
        if op == self.OP_LINK_KV:
            import json
            from ..parallel.kv_transfer import NvlinkPushTransfer
            handles = json.loads(payload.decode())
            link, pull = arg & 0xFFFF, bool(arg >> 16)
            if len(handles) == self.world_size:
                t = NvlinkPushTransfer(self.transfer_caches(), handles[self.rank], self.device, pull=pull)
            else:
                # the other instance runs another TP degree: possible where every rank holds the same cache (MLA)
                from ..parallel.kv_transfer import MultiTransfer, plan_links, plan_source
                if self.comm.dp_size > 1 or not getattr(self.worker.model, "kv_replicated_over_tp", False):
                    raise ValueError(f"the linked instance has {len(handles)} ranks, this one {self.world_size}: different "
                                     "degrees need a cache that is the same on every rank (MLA) and no attention DP")
                if pull:
                    t = NvlinkPushTransfer(self.transfer_caches(), handles[plan_source(len(handles), self.world_size, self.rank)],
                                           self.device, pull=True)
                else:
                    t = MultiTransfer([NvlinkPushTransfer(self.transfer_caches(), handles[d], self.device)
                                       for d in plan_links(self.world_size, len(handles), self.rank)])
            if pull:
                self.kv_sources[link] = t
            elif link == 0:
                self.kv_transfer = t
            else:
                self.kv_transfer_peers[link] = t
            return None
        if op == self.OP_PULL_KV:
            import json
            src = self.kv_sources.get(arg)
            if src is None:
                return False
            src.push([tuple(p) for p in json.loads(payload.decode())])
            src.wait()                                   # the caller activates the request right after
            return True
        if op == self.OP_SLEEP:
            from .sleep import sleep_rank
            return sleep_rank(self, arg)
        if op == self.OP_WAKEUP:
            from .sleep import wakeup_rank
            source = getattr(self, "_weight_source", None)
            if payload:
                import json
                from .weight_transfer import IpcWeightSource
                source = IpcWeightSource(json.loads(payload.decode())["handles"], self.device)
            try:
                return wakeup_rank(self, source)
            finally:
                if payload:
                    source.close()
        cuda = self.device.type == "cuda"
        if op == self.OP_BARRIER_SYNC:
            if cuda:
                torch.cuda.synchronize(self.device)
            if self.world_size > 1:
                torch.distributed.barrier()
            if cuda:
                torch.cuda.synchronize(self.device)
        elif op == self.OP_MARK:
            if cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(torch.cuda.current_stream(self.device))
                self._marks[arg] = ev
            else:
                self._marks[arg] = time.perf_counter()
        elif op == self.OP_ELAPSED:
            if cuda:
                torch.cuda.synchronize(self.device)
                ms = self._marks[0].elapsed_time(self._marks[1])
            else:
                ms = (self._marks[1] - self._marks[0]) * 1e3
            t = torch.tensor([ms], dtype=torch.float64, device=self.device)
            if self.world_size > 1:
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            return float(t.item())
        return None

    # ------------------------------------------------------------------ sleep / wake-up (master.h:38-55 of the reference)
    @property
    def sleep_level(self) -> int:
        return self._sleep_state.level

    def sleep(self, level: int = 1) -> bool:
        """Give the device memory back on every rank (1: weights to pinned host memory, 2: weights dropped).  Only an idle
        engine can be put to sleep; returns False otherwise."""
        from .sleep import AWAKE
        if self._sleep_state.level != AWAKE or level not in (1, 2) or self.kv_transfer is not None:
            return False
        self._drain_inflight()
        if self.scheduler.has_unfinished():
            return False
        while self.host_tier is not None and self.scheduler.has_pending_transfers:
            self.scheduler.schedule()
            self._publish_transfers_only(max(1, self.opt.dp_size))      # blocks still on their way to the host
        for d in range(max(1, self.opt.dp_size)):
            bm = self.scheduler.block_manager(d)
            bm.evict(bm.num_blocks)                                     # the device copies are about to disappear
        self.bytes_released_by_sleep = self._control(self.OP_SLEEP, level)
        return True

    def wakeup(self, weight_source=None) -> bool:
        """`weight_source` (runtime/weight_transfer.py: WeightPuller): a deep sleeper copies its weights from an awake
        instance of the same model instead of reading the checkpoint.  On CUDA the ranks get the source's IPC handles with
        the control message and copy device to device; otherwise (one process) the bytes come over the source's
        connection.  If the source cannot serve this layout the checkpoint is read as usual."""
        from .sleep import AWAKE, DEEP_SLEEP
        if self._sleep_state.level == AWAKE:
            return False
        payload = b""
        self._weight_source = None
        self.weights_pulled_bytes = 0
        if weight_source is not None and self._sleep_state.level == DEEP_SLEEP:
            import json
            try:
                weight_source.check(self)
                if self.device.type == "cuda" and weight_source.same_host():
                    payload = json.dumps({"handles": weight_source.handles()}).encode()
                elif self.world_size == 1:
                    self._weight_source = weight_source
                else:
                    raise RuntimeError("a multi-process engine pulls weights through CUDA IPC only (source on the same host)")
            except Exception as e:
                log.warning("weight source unusable (%s); waking up from the checkpoint", e)
                payload, self._weight_source = b"", None
        self._control(self.OP_WAKEUP, 0, payload)
        self._weight_source = None
        return True

    def barrier_sync(self):
        """Barrier + device synchronisation on every rank (both sides of a timed region)."""
        self._drain_inflight()
        self._control(self.OP_BARRIER_SYNC)

    def mark_timing(self, which: int):
        """Record a CUDA event on every rank's compute stream (0 = start, 1 = end)."""
        self._control(self.OP_MARK, which)

    def elapsed_ms_max_over_ranks(self) -> float:
        return self._control(self.OP_ELAPSED)

    def _drain_inflight(self):
        """Apply the results of overlapped steps that are still in flight."""
        while self._inflight:
            old_batches, old_local, old_rows = self._inflight.pop(0)
            for b, r, rows in zip(old_batches, self._collect(old_batches, old_local), old_rows):
                if r is not None:
                    self._record_top_logprobs(rows, r[2])
                    self.scheduler.update_output(b.id, r[0], r[1])

    def transfer_caches(self):
        """The cache tensors a disaggregated pair moves for a block id, in one order on both sides: the target model's
        layers (engines with a draft module append its KV)."""
        return list(self.worker.kv_caches)

    def collect_cache_handles(self):
        """CUDA-IPC descriptions of every rank's KV-cache tensors (decode side of a disaggregated pair)."""
        return self._control(self.OP_GATHER_HANDLES)

    def collect_weight_handles(self):
        """CUDA-IPC descriptions of every rank's weight tensors (source side of a remote wake-up)."""
        return self._control(self.OP_WEIGHT_HANDLES)

    def link_kv_peer(self, handles_per_rank, link: int = 0) -> None:
        """Map a decode instance's KV caches on every rank of this (prefill) instance (`link`: which decode instance)."""
        import json
        self._control(self.OP_LINK_KV, link, json.dumps(handles_per_rank).encode())

    def link_kv_source(self, handles_per_rank, source: int = 0) -> None:
        """PULL mode, decode side: map a prefill instance's KV caches on every rank (`source`: which prefill instance)."""
        import json
        self._control(self.OP_LINK_KV, source | (1 << 16), json.dumps(handles_per_rank).encode())

    def pull_kv(self, source: int, pairs) -> bool:
        """PULL mode, decode side: every rank copies the listed (block of the prefill instance, own block) pairs out of
        the mapped cache of prefill instance `source` and waits for the copy (pull_kv_blocks of the reference,
        llm_engine.cpp:680-718)."""
        import json
        return bool(self._control(self.OP_PULL_KV, source, json.dumps([list(p) for p in pairs]).encode()))

    def kernel_launches(self) -> int:
        """Kernels of this library launched so far on this rank (graph replays count their captured kernels)."""
        if self.device.type != "cuda":
            return 0
        from ..ops import cuda_ops
        g = self.worker._graphs
        return cuda_ops.launch_count + (g.replayed_kernels if g is not None else 0)

    def shutdown(self):
        if self.host_tier is not None:
            self.host_tier.flush_store()                 # blocks still on their way to the shared store
        if self.rank == 0 and self._chan is not None:
            msg = self._ensure_msg(0)
            msg[:CTRL_WORDS].zero_()
            msg[0] = CMD_STOP
            self._chan.write_ptr(msg.data_ptr(), CTRL_WORDS * 4, 5.0)
        self._chan = None
        self._res_chans = {}

    # ------------------------------------------------------------------ metrics helpers
    def kv_utilization(self) -> float:
        return float(self.scheduler.kv_utilization) if self.scheduler is not None else 0.0
