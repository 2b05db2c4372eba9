"""Process-wide metrics with a Prometheus text exposition.

Metric names are the reference's bvar names (xllm/core/common/metrics.h:110-210): request status
counts, tokenisation / engine latency, prefix-cache gauges, `num_{pending,running,waiting}_requests`,
`kv_cache_utilization_perc`, `num_{free,used}_blocks`, prompt / generated token counters, TTFT /
inter-token / end-to-end latency histograms, speculative-decoding counters.
"""
from __future__ import annotations

import bisect
import threading
import time
from typing import Dict, Optional, Tuple

_BUCKETS = [0.5, 1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 30000, 60000]


class _Hist:
    __slots__ = ("counts", "total", "n")

    def __init__(self):
        self.counts = [0] * (len(_BUCKETS) + 1)
        self.total = 0.0
        self.n = 0

    def observe(self, v: float):
        self.counts[bisect.bisect_left(_BUCKETS, v)] += 1
        self.total += v
        self.n += 1

    def quantile(self, q: float) -> float:
        if self.n == 0:
            return 0.0
        want, acc = q * self.n, 0
        for i, c in enumerate(self.counts):
            acc += c
            if acc >= want:
                return _BUCKETS[min(i, len(_BUCKETS) - 1)]
        return _BUCKETS[-1]


class Metrics:
    def __init__(self):
        self._lock = threading.Lock()
        self.counters: Dict[Tuple[str, Tuple], float] = {}
        self.gauges: Dict[str, float] = {}
        self.hists: Dict[str, _Hist] = {}

    def inc(self, name: str, v: float = 1.0, labels: Optional[Dict[str, str]] = None):
        key = (name, tuple(sorted((labels or {}).items())))
        with self._lock:
            self.counters[key] = self.counters.get(key, 0.0) + v

    def set(self, name: str, v: float):
        self.gauges[name] = float(v)

    def observe(self, name: str, v: float):
        with self._lock:
            h = self.hists.get(name)
            if h is None:
                h = self.hists[name] = _Hist()
            h.observe(v)

    def observe_many(self, name: str, values) -> None:
        """Several observations of one histogram under one lock (per-step batches of per-request latencies)."""
        if not values:
            return
        with self._lock:
            h = self.hists.get(name)
            if h is None:
                h = self.hists[name] = _Hist()
            for v in values:
                h.observe(v)

    def counter(self, name: str, labels: Optional[Dict[str, str]] = None) -> float:
        return self.counters.get((name, tuple(sorted((labels or {}).items()))), 0.0)

    def prometheus_text(self) -> str:
        out = []
        with self._lock:
            seen = set()
            for (name, labels), v in sorted(self.counters.items()):
                if name not in seen:
                    out.append(f"# TYPE {name} counter")
                    seen.add(name)
                lab = "{" + ",".join(f'{k}="{val}"' for k, val in labels) + "}" if labels else ""
                out.append(f"{name}{lab} {v:g}")
            for name, v in sorted(self.gauges.items()):
                out.append(f"# TYPE {name} gauge")
                out.append(f"{name} {v:g}")
            for name, h in sorted(self.hists.items()):
                out.append(f"# TYPE {name} histogram")
                acc = 0
                for b, c in zip(_BUCKETS, h.counts):
                    acc += c
                    out.append(f'{name}_bucket{{le="{b:g}"}} {acc}')
                out.append(f'{name}_bucket{{le="+Inf"}} {h.n}')
                out.append(f"{name}_sum {h.total:g}")
                out.append(f"{name}_count {h.n}")
        return "\n".join(out) + "\n"

    def reset(self):
        with self._lock:
            self.counters.clear()
            self.gauges.clear()
            self.hists.clear()


METRICS = Metrics()


class AutoCounter:
    """`with AutoCounter("x_latency_seconds"):` — the reference's AUTO_COUNTER RAII timer (metrics.h:25-41)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        METRICS.observe(self.name, time.perf_counter() - self.t0)
        return False
