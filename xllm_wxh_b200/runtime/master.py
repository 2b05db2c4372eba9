"""LLMMaster: request front door of one serving instance.

Role of the reference's LLMMaster (xllm/core/distributed_runtime/llm_master.cpp:56-121 set-up,
173-248 handle_request, 250-279 run loop, 281-517 generate_request): tokenise / apply the chat
template on a small thread pool, build the scheduler request, run the scheduling loop on one thread,
and turn scheduler outputs into `RequestOutput` deltas (incremental detokenisation, stop strings,
logprobs, usage) delivered to per-request callbacks — the job of the reference's
AsyncResponseProcessor (scheduler/async_response_processor.cpp).
"""
from __future__ import annotations

import logging
import threading
import time
import uuid
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import numpy as np

from ..config import Options
from ..framework.params import (FINISH_REASONS, LogProb, LogProbData, RequestOutput, RequestParams, SequenceOutput, Status,
                                StatusCode, Usage)
from ..utils.metrics import METRICS
from ..utils.tokenizer import IncrementalDecoder, Tokenizer, load_tokenizer
from .engine import LLMEngine

OutputCallback = Callable[[RequestOutput], bool]
log = logging.getLogger("xllm.master")


class _SeqState:
    __slots__ = ("decoder", "token_ids", "text", "logprobs", "finish_reason", "cum_logprob", "held")

    def __init__(self, tokenizer: Tokenizer, skip_special: bool):
        self.decoder = IncrementalDecoder(tokenizer, skip_special)
        self.token_ids: List[int] = []
        self.text = ""
        self.logprobs: List[LogProb] = []
        self.finish_reason: Optional[str] = None
        self.cum_logprob = 0.0
        self.held = ""             # text withheld because it may be the start of a stop string


class _RequestState:
    def __init__(self, ext_id: str, prompt: Optional[str], prompt_ids: List[int], params: RequestParams,
                 callback: OutputCallback):
        self.ext_id, self.prompt, self.prompt_ids, self.params, self.callback = ext_id, prompt, prompt_ids, params, callback
        self.seqs: Dict[int, _SeqState] = {}
        self.arrival = time.monotonic()
        self.first_token_time = 0.0
        self.last_token_time = 0.0
        self.core_id = -1
        self.num_cached = 0
        self.done = False


class LLMMaster:
    def __init__(self, options: Options, engine: Optional[LLMEngine] = None, tokenizer: Optional[Tokenizer] = None):
        self.opt = options
        self.engine = engine or LLMEngine(options)
        self.args = self.engine.args
        self.tokenizer = tokenizer or load_tokenizer(self.engine.model_dir, self.args.vocab_size, self.args.eos_token_id)
        self.chat_template = None
        if getattr(self.tokenizer, "chat_template", None):
            from ..api.chat_template import JinjaChatTemplate
            self.chat_template = JinjaChatTemplate(self.tokenizer.chat_template, self.tokenizer)
        self._states: Dict[int, _RequestState] = {}
        self._lock = threading.Lock()
        # outputs that arrived before their request's state was registered (see _emit_locked); a leaf lock: nothing
        # else is taken while it is held
        self._reg_lock = threading.Lock()
        self._orphans: Dict[int, List] = {}
        self._last_cid = -1
        self._pool = ThreadPoolExecutor(max_workers=max(1, options.num_request_handling_threads))
        self._loop_thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._wake = threading.Event()
        self.model_id = options.model_id or (options.model.rstrip("/").split("/")[-1] if options.model else "model")
        self.extra_step_hooks: List[Callable[["LLMMaster"], None]] = []
        self.idle_wait: Optional[Callable[[], None]] = None
        self._emit_lock = threading.RLock()
        self._step_lock = threading.RLock()          # re-entered by work that runs exclusively and adds requests itself
        self._lock_waiters = 0                       # control operations of other threads waiting for the step lock
        self.engine.external_step_lock = self._step_lock     # request intake that touches the block tables takes it too
        self.time_predictor = None
        self.profiler = None
        # maxima since the last heartbeat to the service layer (xservice_client.cpp:373-383)
        self._recent_max_ttft_ms = 0.0
        self._recent_max_tbt_ms = 0.0
        self.xservice = None
        self.weight_sources: Dict[str, Any] = {}       # address -> open session to an awake instance's weight service
        self.weight_server = None
        if options.enable_profile_step_time and self.engine.scheduler is not None:
            # synthetic prefill / decode steps through the real engine, then the fitted step-time model (and, when asked
            # for, the token budget that keeps a step within the TPOT target) -- profile_manager.h:31-100
            from .profile_manager import ProfileManager
            self.profiler = ProfileManager(self.engine, options.profile_max_prompt_length)
            self.time_predictor = self.profiler.run()
        if getattr(options, "enable_service_routing", False) and options.etcd_addr and self.engine.scheduler is not None:
            from .xservice_client import attach_to_master
            self.xservice = attach_to_master(self, options)

    # ------------------------------------------------------------------ sleep / wake-up (master.h:38-55 of the reference)
    def is_sleeping(self) -> bool:
        return self.engine.sleep_level != 0

    def sleep(self, level: int = 1) -> bool:
        """Release device memory while idle (1: weights kept in pinned host memory, 2: dropped); the serving loop keeps
        running and simply finds nothing to do."""
        return bool(self.run_exclusive(lambda: self.engine.sleep(level)))

    def wakeup(self, remote_addrs: Optional[List[str]] = None) -> bool:
        """`remote_addrs`: weight services of awake instances of this model (WakeupOptions.remote_addrs in the reference);
        a deep sleeper copies its weights from the first one that answers instead of reading the checkpoint."""
        source = None
        for addr in remote_addrs or ():
            try:
                source = self.weight_sources.get(addr) or self.link_d2d([addr])[addr]
                break
            except (OSError, ConnectionError, TimeoutError) as e:
                log.warning("weight source %s unreachable: %s", addr, e)
        return bool(self.run_exclusive(lambda: self.engine.wakeup(source)))

    def link_d2d(self, addrs: List[str]) -> Dict[str, Any]:
        """Open a session to the weight service of each address (link_d2d, worker_impl.cpp:425-436 of the reference)."""
        from .weight_transfer import WeightPuller
        for addr in addrs:
            if addr not in self.weight_sources:
                self.weight_sources[addr] = WeightPuller(addr)
        return {a: self.weight_sources[a] for a in addrs}

    def unlink_d2d(self, addrs: List[str]) -> int:
        n = 0
        for addr in addrs:
            s = self.weight_sources.pop(addr, None)
            if s is not None:
                s.close()
                n += 1
        return n

    def take_latency_metrics(self) -> Dict[str, float]:
        """Largest time to first token and time between tokens (ms) seen since the previous call."""
        with self._lock:
            out = {"recent_max_ttft": self._recent_max_ttft_ms, "recent_max_tbt": self._recent_max_tbt_ms}
            self._recent_max_ttft_ms = self._recent_max_tbt_ms = 0.0
        return out

    # ------------------------------------------------------------------ request intake
    def _eos(self) -> int:
        e = self.args.eos_token_id
        return e if e >= 0 else getattr(self.tokenizer, "eos_token_id", -1)

    def _build(self, prompt: Optional[str], prompt_ids: Optional[Sequence[int]], params: RequestParams,
               callback: OutputCallback) -> Optional[int]:
        t0 = time.perf_counter()
        st = params.verify()
        if not st.ok:
            callback(RequestOutput(request_id=params.request_id, status=st, finished=True))
            return None
        if prompt_ids is None:
            prompt_ids = self.tokenizer.encode(prompt or "", add_special_tokens=params.add_special_tokens)
        prompt_ids = list(prompt_ids)
        METRICS.observe("tokenization_latency_seconds", time.perf_counter() - t0)
        max_ctx = self.args.max_position_embeddings
        if len(prompt_ids) == 0 or len(prompt_ids) >= max_ctx:
            callback(RequestOutput(request_id=params.request_id, finished=True,
                                   status=Status(StatusCode.INVALID_ARGUMENT,
                                                 "prompt is empty" if not prompt_ids else "prompt is too long")))
            return None
        max_tokens = min(params.max_tokens, max_ctx - len(prompt_ids))       # llm_master.cpp: clamp to the context
        p = RequestParams(**{**params.__dict__, "max_tokens": max_tokens})
        stop_seqs: List[List[int]] = []
        ext_id = p.request_id or ("cmpl-" + uuid.uuid4().hex[:24])
        p.request_id = ext_id
        sp, stc = p.to_core(self._eos(), list(self.args.stop_token_ids), stop_seqs)
        state = _RequestState(ext_id, prompt, prompt_ids, p, callback)
        n, best_of = p.n, (p.best_of or p.n)
        if p.beam_width > 1:
            n = best_of = 1
        with self._lock:
            cid = self.engine.add_request(prompt_ids, sp, stc, n, best_of, p.priority, p.offline, ext_id, p.ttft_slo_ms,
                                          p.tpot_slo_ms, p.ttft_priority_weight, p.tpot_priority_weight)
            state.core_id = cid
            with self._reg_lock:
                self._states[cid] = state
                self._last_cid = max(self._last_cid, cid)
                parked = cid in self._orphans
        if parked:                                       # the loop ran ahead of this thread: hand its outputs out now
            LLMMaster._emit(self, [])                    # (the class's own emission: the parked outputs have been through
                                                         # any wrapper a PD coordinator put around `_emit` already)
        METRICS.inc("prompt_tokens_total", len(prompt_ids))
        METRICS.inc("server_request_in_total")
        self._wake.set()
        return cid

    def handle_request(self, prompt: Union[str, Sequence[int], List[Dict[str, Any]]], params: RequestParams,
                       callback: OutputCallback, asynchronous: bool = True):
        """`prompt` is text, token ids, or a list of chat messages (then the chat template is applied)."""
        def job():
            try:
                if isinstance(prompt, str):
                    return self._build(prompt, None, params, callback)
                if prompt and isinstance(prompt[0], dict):
                    if self.chat_template is None:
                        text = "".join(f"{m.get('role')}: {m.get('content')}\n" for m in prompt) + "assistant: "
                    else:
                        text = self.chat_template.apply(prompt, params.tools, params.chat_template_kwargs)
                    return self._build(text, None, params, callback)
                return self._build(None, prompt, params, callback)
            except Exception as e:                                   # surfaces as a failed request, never kills the pool
                callback(RequestOutput(request_id=params.request_id, finished=True,
                                       status=Status(StatusCode.UNKNOWN, f"{type(e).__name__}: {e}")))
                return None
        if asynchronous:
            return self._pool.submit(job)
        return job()

    def cancel(self, core_id: int):
        self.engine.cancel(core_id)
        self._wake.set()

    # ------------------------------------------------------------------ response processing
    def _emit(self, outs) -> None:
        """Scheduler outputs -> RequestOutput deltas."""
        with self._emit_lock:
            self._emit_locked(outs)

    def _emit_locked(self, outs) -> None:
        # A request becomes schedulable inside engine.add_request, one statement before the submitting thread registers
        # its state, and the serving loop can run whole steps in between.  Outputs of a request that is not registered
        # yet are parked and come out, first, as soon as it is (`_register`, or the next call here).
        if self._orphans:
            with self._reg_lock:
                ready = [cid for cid in self._orphans if cid in self._states]
                parked = [o for cid in ready for o in self._orphans.pop(cid)]
            if parked:
                outs = parked + list(outs)
        now = time.monotonic()
        by_req: Dict[int, List] = {}
        for o in outs:
            by_req.setdefault(o.request_id, []).append(o)
        # per-step batches of the metrics: one lock round each instead of one per request
        ttfts: List[float] = []
        tbts: List[float] = []
        generated = 0
        states, tokenizer = self._states, self.tokenizer
        for cid, lst in by_req.items():
            st = states.get(cid)
            if st is None:
                with self._reg_lock:
                    st = states.get(cid)
                    if st is None and cid > self._last_cid:          # ids grow: this one is still being registered
                        # bounded: a request that somebody added to the engine directly never registers here
                        held = self._orphans.get(cid)
                        if held is None and len(self._orphans) < 1024:
                            held = self._orphans[cid] = []
                        if held is not None and len(held) < 64:
                            held.extend(lst)
                        continue
            if st is None or st.done:
                continue
            p = st.params
            streaming = p.streaming
            outputs: List[SequenceOutput] = []
            req_finished = False
            for o in lst:
                ss = st.seqs.get(o.seq_index)
                if ss is None:
                    ss = st.seqs[o.seq_index] = _SeqState(tokenizer, p.skip_special_tokens)
                new_ids = list(o.new_tokens)
                if new_ids:
                    if st.first_token_time == 0.0:
                        st.first_token_time = now
                        ttft = (now - st.arrival) * 1e3
                        ttfts.append(ttft)
                        self._recent_max_ttft_ms = max(self._recent_max_ttft_ms, ttft)
                    elif st.last_token_time:
                        tbt = (now - st.last_token_time) * 1e3 / len(new_ids)
                        tbts.append(tbt)
                        self._recent_max_tbt_ms = max(self._recent_max_tbt_ms, tbt)
                    st.last_token_time = now
                    generated += len(new_ids)
                ss.token_ids.extend(new_ids)
                # text as it grows is needed for streaming and for stop strings only; otherwise the output is decoded
                # once, when the sequence finishes
                incremental = streaming or bool(p.stop)
                delta = ss.decoder.add(new_ids) if incremental else ""
                new_logprobs = o.new_logprobs
                if new_logprobs:
                    tops = self.engine.top_logprobs.pop((cid, o.seq_index), None) if p.top_logprobs > 0 else None
                    for j, (tid, lp) in enumerate(zip(new_ids, new_logprobs)):
                        item = LogProb(token=tokenizer.decode([tid], False), token_id=tid, logprob=float(lp))
                        if tops and j < len(tops):
                            item.top_logprobs = [LogProbData(tokenizer.decode([int(i)], False), int(i), float(v))
                                                 for i, v in zip(tops[j][0][:p.top_logprobs], tops[j][1][:p.top_logprobs])]
                        ss.logprobs.append(item)
                        ss.cum_logprob += float(lp)
                finish = FINISH_REASONS.get(o.finish_reason) if o.finished else None
                # stop strings are matched on text (the scheduler only knows token-level criteria)
                if p.stop:
                    delta, hit = self._apply_stop_strings(ss, delta, p.stop, bool(finish))
                    if hit and not finish:
                        finish = "stop"
                        self.engine.cancel(cid) if len(st.seqs) <= 1 and (p.best_of or p.n) == 1 else None
                if finish:
                    if not incremental:
                        ss.text = tokenizer.decode(ss.token_ids, p.skip_special_tokens)
                    elif not p.stop:
                        delta += ss.decoder.flush()
                    ss.finish_reason = finish
                ss.text += delta
                if o.num_cached_tokens > st.num_cached:
                    st.num_cached = o.num_cached_tokens
                if streaming:
                    so = SequenceOutput(index=o.seq_index, text=delta, token_ids=new_ids, finish_reason=finish)
                    if new_logprobs:
                        so.logprobs = ss.logprobs[-len(new_ids):]
                    outputs.append(so)
                req_finished = req_finished or o.request_finished
            if not req_finished and p.stop:
                want = p.best_of or p.n
                req_finished = len(st.seqs) >= want and all(s.finish_reason for s in st.seqs.values())
            if not req_finished and not (streaming and outputs):
                continue                                  # nothing to hand out this step (the usual case off-line)
            ro = RequestOutput(request_id=st.ext_id, service_request_id=p.service_request_id, status=Status())
            ro.outputs = outputs
            if req_finished:
                st.done = True
                self._finish_request(st, ro)
            keep_going = st.callback(ro)
            if keep_going is False and not st.done:
                self.engine.cancel(cid)
            if st.done:
                states.pop(cid, None)
                self.engine.drop_top_logprobs(cid)
        if generated:
            METRICS.inc("generated_tokens_total", generated)
        METRICS.observe_many("time_to_first_token_latency_milliseconds", ttfts)
        METRICS.observe_many("inter_token_latency_milliseconds", tbts)

    @staticmethod
    def _apply_stop_strings(ss: _SeqState, delta: str, stops: List[str], final: bool):
        buf = ss.held + delta
        cut = -1
        for s in stops:
            i = buf.find(s)
            if i >= 0 and (cut < 0 or i < cut):
                cut = i
        if cut >= 0:
            ss.held = ""
            return buf[:cut], True
        if final:
            ss.held = ""
            return buf, False
        hold = 0
        for s in stops:                     # longest suffix of buf that is a proper prefix of a stop string
            for k in range(min(len(s) - 1, len(buf)), 0, -1):
                if buf.endswith(s[:k]):
                    hold = max(hold, k)
                    break
        ss.held = buf[len(buf) - hold:] if hold else ""
        return buf[:len(buf) - hold] if hold else buf, False

    def _finish_request(self, st: _RequestState, ro: RequestOutput):
        p = st.params
        seqs = sorted(st.seqs.items())
        want_n = p.n
        if (p.best_of or p.n) > p.n:        # keep the n best by cumulative log-probability
            seqs = sorted(seqs, key=lambda kv: -kv[1].cum_logprob)[:want_n]
        gen = sum(len(s.token_ids) for _, s in st.seqs.items())
        ro.usage = Usage(len(st.prompt_ids), gen, len(st.prompt_ids) + gen, st.num_cached)
        ro.finished = True
        ro.prompt = st.prompt
        ro.prompt_token_ids = st.prompt_ids
        reasons = {s.finish_reason for _, s in seqs}
        if "resource_exhausted" in reasons:
            ro.status = Status(StatusCode.RESOURCE_EXHAUSTED, "not enough KV cache blocks for this request")
        elif "cancelled" in reasons and not p.stop:
            ro.status = Status(StatusCode.CANCELLED, "cancelled")
            ro.cancelled = True
        if not p.streaming:
            ro.outputs = []
            for rank, (idx, s) in enumerate(seqs):
                text = (st.prompt or "") + s.text if p.echo else s.text
                fr = s.finish_reason if s.finish_reason != "cancelled" or not p.stop else "stop"
                ro.outputs.append(SequenceOutput(index=rank, text=text, token_ids=list(s.token_ids), finish_reason=fr,
                                                 logprobs=s.logprobs if p.logprobs else None, cumulative_logprob=s.cum_logprob))
        METRICS.observe("end_2_end_latency_milliseconds", (time.monotonic() - st.arrival) * 1e3)
        METRICS.inc("request_status_total", labels={"code": ro.status.code.name})
        METRICS.inc("server_request_total_ok" if ro.status.ok else "server_request_total_fail")
        METRICS.observe("num_prompt_tokens_per_request", len(st.prompt_ids))
        METRICS.observe("num_generated_tokens_per_request", sum(len(s.token_ids) for _, s in seqs))

    def _step_metrics(self, sch, bm) -> None:
        """The rest of the reference's catalogue (core/common/metrics.h:110-210): scheduling and model-execution latency,
        preemptions, running sequences, prefix-cache hit rate, speculative counts, host-tier traffic, memory gauges."""
        eng = self.engine
        if eng.host_trace:
            sched_ms, pack_ms, issue_ms, wait_ms = eng.host_trace[-1]
            if eng.step_count != getattr(self, "_metrics_step", -1):
                self._metrics_step = eng.step_count
                METRICS.observe("scheduling_latency_seconds", sched_ms * 1e-3)
                METRICS.observe("execution_latency_seconds_model", (issue_ms + wait_ms) * 1e-3)
        st = sch.stats()
        METRICS.set("num_preempted_requests", st["num_preemptions"])
        METRICS.set("num_offline_evictions", st["num_offline_evictions"])
        METRICS.set("num_running_sequences", sch.num_running)
        q = bm.match_queries
        METRICS.set("prefix_cache_block_matched_rate", (bm.match_hits / q) if q else 0.0)
        METRICS.set("prefix_cache_matched_blocks_total", bm.match_hits)
        if eng.host_tier is not None:
            METRICS.set("kv_host_tier_offloaded_blocks_total", st["host_offloaded_blocks"])
            METRICS.set("kv_host_tier_loaded_blocks_total", st["host_loaded_blocks"])
        if hasattr(eng, "stat_draft_tokens"):
            METRICS.set("speculative_num_draft_tokens_total", eng.stat_draft_tokens)
            METRICS.set("speculative_num_accepted_tokens_total", eng.stat_accepted_tokens)
        from ..utils.device_monitor import DEVICE_MONITOR
        dev = eng.device.index or 0
        if not getattr(self, "_memory_gauges", False):
            self._memory_gauges = True
            w = eng.worker
            DEVICE_MONITOR.set_weight_memory(dev, w.model.weight_bytes() if hasattr(w.model, "weight_bytes") else 0)
            DEVICE_MONITOR.set_total_kv_cache_memory(dev, sum(t.numel() * t.element_size() for layer in w.kv_caches for t in layer))
            METRICS.set("total_kv_blocks", eng.num_blocks)
            self._monitor_at = 0.0
        now = time.perf_counter()
        if now - self._monitor_at >= 1.0:            # memory and hardware readings once a second
            self._monitor_at = now
            DEVICE_MONITOR.export(METRICS, dev, hardware=eng.device.type == "cuda")

    # ------------------------------------------------------------------ loops
    def step(self) -> int:
        t0 = time.perf_counter()
        outs = self.engine.step()
        METRICS.observe("engine_latency_seconds", time.perf_counter() - t0)
        sch = self.engine.scheduler
        METRICS.set("num_running_requests", sch.num_running)
        METRICS.set("num_waiting_requests", sch.num_waiting)
        METRICS.set("num_pending_requests", sch.num_pending)
        METRICS.set("kv_cache_utilization_perc", sch.kv_utilization)
        bm = sch.block_manager(0)
        METRICS.set("num_free_blocks", bm.num_free_blocks)
        METRICS.set("num_used_blocks", bm.num_used_blocks)
        METRICS.set("num_blocks_in_prefix_cache", bm.num_blocks_in_prefix_cache)
        self._step_metrics(sch, bm)
        for h in self.extra_step_hooks:
            h(self)
        if outs:
            self._emit(outs)
        return len(outs)

    def generate(self, timeout_s: float = 3600.0):
        """Offline: run until every submitted request has finished (continuous_scheduler.cpp:1117-1142).  Requests that
        were handed to a decode instance finish when that instance reports it; `idle_wait` is called while waiting."""
        deadline = time.monotonic() + timeout_s
        while time.monotonic() < deadline:
            if self.engine.has_unfinished():
                self.step()
            elif any(not s.done for s in list(self._states.values())):
                if self.idle_wait is not None:
                    self.idle_wait()
                else:
                    time.sleep(0.001)
            else:
                break

    def _fail_all(self, message: str) -> None:
        """Finish every in-flight request with an error status and drop it from the engine."""
        with self._lock:
            states = [(cid, st) for cid, st in self._states.items() if not st.done]
        for cid, st in states:
            try:
                self.engine.cancel(cid)
            except Exception:
                pass
            st.done = True
            try:
                st.callback(RequestOutput(request_id=st.ext_id, finished=True, status=Status(StatusCode.UNKNOWN, message)))
            except Exception:
                pass
            with self._lock:
                self._states.pop(cid, None)

    def control_lock(self):
        """The step lock for a control operation issued from another thread (a KV fetch, a link).  The serving loop takes
        the lock again right after every step, which can keep a waiting thread out for many steps; a registered waiter
        makes the loop stand back for a moment after its step."""
        master = self

        class _Waiter:
            def __enter__(self):
                master._lock_waiters += 1
                master._step_lock.acquire()
                return self

            def __exit__(self, *exc):
                master._step_lock.release()
                master._lock_waiters -= 1
                return False
        return _Waiter()

    def run_exclusive(self, fn):
        """Run `fn()` while no generation request is in flight and none can enter (the embedding path drives the
        scheduler itself, so it must not interleave with the serving loop)."""
        while True:
            with self._step_lock:
                with self._lock:
                    if not self.engine.has_unfinished():
                        return fn()
            time.sleep(0.002)

    def run(self):
        """Online: scheduling loop thread (llm_master.cpp:250-265)."""
        if self._loop_thread is not None:
            return

        def loop():
            failures = 0
            while not self._stop.is_set():
                if self.engine.has_unfinished():
                    try:
                        with self._step_lock:
                            self.step()
                        failures = 0
                        if self._lock_waiters > 0:              # let a control operation in between two steps
                            time.sleep(0.0005)
                    except Exception as e:                      # keep serving; report through health
                        from ..utils.health import HEALTH
                        HEALTH.set_unhealthy(f"engine step failed: {type(e).__name__}: {e}")
                        failures += 1
                        if failures >= 3:                       # no progress: fail what is in flight instead of hanging it
                            self._fail_all(f"engine step failed: {type(e).__name__}: {e}")
                            failures = 0
                        time.sleep(0.05)
                else:
                    self._wake.wait(0.5)
                    self._wake.clear()
        self._loop_thread = threading.Thread(target=loop, name="xllm-scheduler", daemon=True)
        self._loop_thread.start()

    def stop(self):
        self.unlink_d2d(list(self.weight_sources))
        if self.weight_server is not None:
            self.weight_server.close()
            self.weight_server = None
        if self.xservice is not None:
            self.xservice.stop()
            self.xservice = None
        self._stop.set()
        self._wake.set()
        if self._loop_thread is not None:
            self._loop_thread.join(timeout=5)
            self._loop_thread = None
        self.engine.shutdown()
        self._pool.shutdown(wait=False)


_fork_counter = [0]


def fork_master(master: LLMMaster, model_path: str, model_id: str = "", master_status: int = 0,
                tokenizer: Optional[Tokenizer] = None, **overrides) -> LLMMaster:
    """A second master, for another model, on the devices of `master` (fork_master in the reference, master.cpp:409-446:
    the new master inherits the options of the first one, takes model path / id and its initial state from the request,
    and gets its own server index).  The two models share the device by turns: one sleeps (its weights and KV cache
    are released) while the other serves, which is what `master_status` 1 (light sleep) or 2 (deep sleep) asks for
    right after the load.

    The new engine sizes its KV cache from the device memory that is free at this moment, so fork while the first
    model sleeps, or give the first model a `max_memory_utilization` that leaves room.  Engines that span several rank
    processes are not forked: their ranks belong to one process group that cannot be joined a second time."""
    import dataclasses
    import os
    if master_status not in (0, 1, 2):
        raise ValueError("master_status must be 0 (awake), 1 (light sleep) or 2 (deep sleep)")
    if not model_path.startswith("preset:") and not os.path.exists(model_path):
        raise FileNotFoundError(f"model path {model_path} does not exist")
    if master.engine.world_size > 1:
        raise NotImplementedError("fork_master needs an engine of one process (tensor-parallel rank processes cannot be forked)")
    if not model_id:
        model_id = os.path.basename(os.path.normpath(model_path)) if not model_path.startswith("preset:") else model_path[7:]
    _fork_counter[0] += 1
    # a forked master is reached through the first master's front end: no registration, no PD role, no profiling run of its own
    opts = dataclasses.replace(master.opt, model=model_path, model_id=model_id, enable_service_routing=False,
                               enable_disagg_pd=False, instance_role="DEFAULT", enable_profile_step_time=False,
                               draft_model="", num_speculative_tokens=0, **overrides)
    from .launcher import make_engine
    new = LLMMaster(opts, make_engine(opts), tokenizer)
    new.server_idx = _fork_counter[0]
    new.run()
    if master_status and not new.sleep(master_status):
        new.stop()
        raise RuntimeError(f"forked master for {model_id} could not enter sleep state {master_status}")
    return new
