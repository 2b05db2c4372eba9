"""Start-up profiling of step times and the step-time predictors built from it.

Role of the reference's ProfileManager / TimePredictor (xllm/core/scheduler/profile/profile_manager.h:31-100,
time_predictor.cpp; flags `enable_profile_step_time`, `enable_profile_token_budget`, `profile_max_prompt_length`,
global_flags.cpp:246-268): before serving, synthetic prefill and decode batches are pushed through the real engine,
their step times are measured, and two small least-squares models are fitted:

    prefill_ms(tokens, kv)      = a0 + a1 * tokens + a2 * tokens * (kv + tokens / 2)     (linear layers + causal attention)
    decode_ms(batch, kv_total)  = b0 + b1 * batch + b2 * kv_total                        (weights once, KV streamed)

The scheduler uses them through `token_budget_for_tpot()`: the largest number of prefill tokens that can ride along with
the running decodes without pushing the step over the time-per-output-token target (Sarathi-style budget).
"""
from __future__ import annotations

import dataclasses
import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .. import _core


@dataclasses.dataclass
class TimePredictor:
    prefill_coef: Tuple[float, float, float] = (0.0, 0.0, 0.0)
    decode_coef: Tuple[float, float, float] = (0.0, 0.0, 0.0)

    def prefill_ms(self, tokens: int, kv_before: int = 0) -> float:
        a0, a1, a2 = self.prefill_coef
        return max(0.0, a0 + a1 * tokens + a2 * tokens * (kv_before + tokens / 2.0))

    def decode_ms(self, batch: int, kv_total: int) -> float:
        b0, b1, b2 = self.decode_coef
        return max(0.0, b0 + b1 * batch + b2 * kv_total)

    def mixed_ms(self, prefill_tokens: int, batch: int, kv_total: int, kv_before: int = 0) -> float:
        """A step that decodes `batch` sequences and prefills `prefill_tokens` tokens: the fixed cost is paid once."""
        if prefill_tokens <= 0:
            return self.decode_ms(batch, kv_total)
        if batch <= 0:
            return self.prefill_ms(prefill_tokens, kv_before)
        return self.prefill_ms(prefill_tokens, kv_before) + self.decode_ms(batch, kv_total) - min(self.prefill_coef[0],
                                                                                                 self.decode_coef[0])

    def token_budget_for_tpot(self, tpot_ms: float, batch: int, kv_total: int, max_tokens: int) -> int:
        """Largest prefill-token count (multiple of 16) with mixed_ms(...) <= tpot_ms; at least 16."""
        lo, hi = 0, max(16, max_tokens)
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.mixed_ms(mid, batch, kv_total) <= tpot_ms:
                lo = mid
            else:
                hi = mid - 1
        return max(16, lo // 16 * 16)


def _fit(rows: Sequence[Sequence[float]], y: Sequence[float]) -> Tuple[float, float, float]:
    A = np.asarray(rows, dtype=np.float64)
    b = np.asarray(y, dtype=np.float64)
    coef, *_ = np.linalg.lstsq(A, b, rcond=None)
    coef = np.maximum(coef, 0.0)            # times do not fall with more work: clamp noise-driven negative slopes
    return float(coef[0]), float(coef[1]), float(coef[2])


class ProfileManager:
    def __init__(self, engine, max_prompt_length: int = 2048, seed: int = 0):
        self.engine = engine
        self.max_prompt_length = min(max_prompt_length, engine.opt.max_tokens_per_batch,
                                     engine.args.max_position_embeddings - 8)
        self.rng = np.random.default_rng(seed)
        self.predictor = TimePredictor()
        self.samples: Dict[str, List[Tuple]] = {"prefill": [], "decode": []}

    # ------------------------------------------------------------------ measurement
    def _sync(self):
        if self.engine.device.type == "cuda":
            import torch
            torch.cuda.synchronize(self.engine.device)

    def _timed_step(self) -> float:
        self._sync()
        t0 = time.perf_counter()
        self.engine.step()
        self.engine._drain_inflight()
        self._sync()
        return (time.perf_counter() - t0) * 1e3

    def _drain(self):
        while self.engine.has_unfinished():
            self.engine.step()

    def _add(self, prompt_len: int, max_tokens: int) -> int:
        st = _core.StopCriteria()
        st.max_tokens, st.ignore_eos = int(max_tokens), True
        ids = self.rng.integers(0, self.engine.args.vocab_size, prompt_len).tolist()
        return self.engine.add_request(ids, _core.SamplingParams(), st)

    def profile_prefill(self, lengths: Optional[Sequence[int]] = None, repeats: int = 2) -> List[Tuple[int, float]]:
        if lengths is None:
            lengths, n = [], 32
            while n <= self.max_prompt_length:
                lengths.append(n)
                n *= 2
            if not lengths or lengths[-1] != self.max_prompt_length:
                lengths.append(self.max_prompt_length)
        out = []
        for n in lengths:
            best = float("inf")
            for _ in range(repeats + 1):                     # the first pass pays one-off costs (graph capture, caches)
                self._add(n, 1)
                best = min(best, self._timed_step())
                self._drain()
            out.append((n, best))
            self.samples["prefill"].append((n, 0, best))
        return out

    def profile_decode(self, batches: Optional[Sequence[int]] = None, context: int = 64, steps: int = 3) -> List[Tuple[int, int, float]]:
        cap = self.engine.opt.max_seqs_per_batch
        batches = [b for b in (batches or (1, 4, 16, 64, 256)) if b <= cap] or [1]
        out = []
        for b in batches:
            blocks_needed = b * ((context + steps + 8) // self.engine.block_size + 2)
            if blocks_needed > self.engine.num_blocks - 2:
                continue
            for _ in range(b):
                self._add(context, steps + 2)
            guard = 0
            while self.engine.scheduler.num_waiting > 0 and guard < 10000:      # prefill everything first (untimed)
                self.engine.step()
                guard += 1
            self.engine._drain_inflight()
            ts = [self._timed_step() for _ in range(steps)]
            kv_total = b * (context + 1 + steps // 2)
            out.append((b, kv_total, min(ts)))
            self.samples["decode"].append((b, kv_total, min(ts)))
            for rid in list(self.engine.scheduler.running_ids()):
                self.engine.cancel(rid)
            self._drain()
        return out

    # ------------------------------------------------------------------ fitting
    def fit(self) -> TimePredictor:
        pre, dec = self.samples["prefill"], self.samples["decode"]
        if len(pre) >= 3:
            self.predictor.prefill_coef = _fit([[1.0, n, n * (kv + n / 2.0)] for n, kv, _ in pre], [t for *_, t in pre])
        elif pre:
            n, _, t = pre[-1]
            self.predictor.prefill_coef = (0.0, t / n, 0.0)
        if len(dec) >= 3:
            self.predictor.decode_coef = _fit([[1.0, b, kv] for b, kv, _ in dec], [t for *_, t in dec])
        elif dec:
            b, _, t = dec[-1]
            self.predictor.decode_coef = (t, 0.0, 0.0)
        return self.predictor

    def run(self) -> TimePredictor:
        """Profile and fit; with `enable_profile_token_budget` and a TPOT target also install the token budget."""
        self.profile_prefill()
        self.profile_decode()
        pred = self.fit()
        o = self.engine.opt
        if self.engine.scheduler is not None:
            # the latency-aware policies of the C++ scheduler predict with the same coefficients
            m = _core.StepTimeModel()
            m.a0, m.a1, m.a2 = pred.prefill_coef
            m.b0, m.b1, m.b2 = pred.decode_coef
            self.engine.scheduler.set_step_time_model(m)
        if o.enable_profile_token_budget and o.max_global_tpot_ms > 0 and self.engine.scheduler is not None:
            b = min(o.max_seqs_per_batch, 64)
            budget = pred.token_budget_for_tpot(o.max_global_tpot_ms, b, b * 512, o.max_tokens_per_batch)
            self.engine.scheduler.set_token_budget(budget + b)
        return pred
