"""Instance registry of the service layer: leases, revisions, watches, load and prefix-cache state per instance.

In the reference an engine instance registers itself in etcd under a key prefix per role with a TTL lease, keeps the
lease alive, and reports load metrics, latency metrics and prefix-cache events to the xllm-service master with a
heartbeat RPC (xllm/core/runtime/xservice_client.cpp:220-262 register, :322-417 heartbeat; common/etcd_client.cpp).
etcd and the service binary do not exist in this environment, so the same state lives in this in-process registry,
which the service's HTTP front end (service/router.py) exposes to clients.
"""
from __future__ import annotations

import dataclasses
import threading
import time
from typing import Any, Dict, List, Optional, Set, Tuple

ROLES = ("DEFAULT", "PREFILL", "DECODE", "MIX")
KEY_PREFIX = {"DEFAULT": "XLLM:DEFAULT:", "PREFILL": "XLLM:PREFILL:", "DECODE": "XLLM:DECODE:", "MIX": "XLLM:MIX:"}


@dataclasses.dataclass
class InstanceInfo:
    """What an instance publishes about itself (InstanceInfo in common/types.h:208-240 of the reference)."""
    name: str = ""
    rpc_address: str = ""              # host:port of the instance's HTTP API
    type: str = "DEFAULT"              # DEFAULT | PREFILL | DECODE | MIX
    incarnation_id: str = ""
    register_ts_ms: int = 0
    dp_size: int = 1
    block_size: int = 16
    hash_seed: int = 1024
    model: str = ""
    kv_transfer_port: int = 0          # PD pairs: where the decode side listens for KV hand-off
    pd_port: int = 0                   # PD pairs: control service of a decode instance (prefill instances connect here)
    ttft_profiling_data: List[Tuple[int, float]] = dataclasses.field(default_factory=list)       # (prompt tokens, ms)
    tpot_profiling_data: List[Tuple[int, int, float]] = dataclasses.field(default_factory=list)  # (batch, kv tokens, ms)

    def to_json(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    @staticmethod
    def from_json(d: Dict[str, Any]) -> "InstanceInfo":
        known = {f.name for f in dataclasses.fields(InstanceInfo)}
        info = InstanceInfo(**{k: v for k, v in d.items() if k in known})
        info.ttft_profiling_data = [tuple(x) for x in info.ttft_profiling_data]
        info.tpot_profiling_data = [tuple(x) for x in info.tpot_profiling_data]
        return info


@dataclasses.dataclass
class InstanceState:
    info: InstanceInfo
    lease_deadline: float
    ttl_s: float
    # heartbeat payload
    cache_usage: float = 0.0
    waiting_requests: int = 0
    running_requests: int = 0
    recent_max_ttft_ms: float = 0.0
    recent_max_tbt_ms: float = 0.0
    last_heartbeat: float = 0.0
    cached_keys: Set[Tuple[int, int]] = dataclasses.field(default_factory=set)
    inflight: int = 0                  # requests the router has sent and not seen finish


class Registry:
    """Thread-safe.  Every change bumps `revision`; `wait_for_change` is the watch primitive."""

    def __init__(self, clock=time.monotonic):
        self._clock = clock
        self._lock = threading.Condition()
        self._instances: Dict[str, InstanceState] = {}
        self.revision = 0
        self.events: List[Tuple[int, str, str]] = []        # (revision, "PUT" | "DELETE", key)

    # ------------------------------------------------------------------ leases
    def _bump(self, kind: str, key: str):
        self.revision += 1
        self.events.append((self.revision, kind, key))
        if len(self.events) > 4096:
            del self.events[:2048]
        self._lock.notify_all()

    @staticmethod
    def key_of(info: InstanceInfo) -> str:
        return KEY_PREFIX[info.type] + info.name

    def register(self, info: InstanceInfo, ttl_s: float = 3.0) -> Dict[str, Any]:
        if info.type not in ROLES:
            raise ValueError(f"unsupported instance type {info.type!r}")
        if not info.name:
            raise ValueError("instance name is empty")
        with self._lock:
            now = self._clock()
            old = self._instances.get(info.name)
            if old is not None and old.info.incarnation_id != info.incarnation_id:
                # a restarted process under the same name: its cache is empty again
                old = None
            st = InstanceState(info=info, lease_deadline=now + ttl_s, ttl_s=ttl_s)
            if old is not None:
                st.cached_keys, st.inflight = old.cached_keys, old.inflight
            if not info.register_ts_ms:
                info.register_ts_ms = int(time.time() * 1e3)
            self._instances[info.name] = st
            self._bump("PUT", self.key_of(info))
            return {"ok": True, "revision": self.revision, "key": self.key_of(info)}

    def deregister(self, name: str) -> bool:
        with self._lock:
            st = self._instances.pop(name, None)
            if st is None:
                return False
            self._bump("DELETE", self.key_of(st.info))
            return True

    def expire(self) -> List[str]:
        """Drop instances whose lease ran out (etcd would delete the key); returns their names."""
        with self._lock:
            now = self._clock()
            dead = [n for n, st in self._instances.items() if st.lease_deadline < now]
            for n in dead:
                st = self._instances.pop(n)
                self._bump("DELETE", self.key_of(st.info))
            return dead

    # ------------------------------------------------------------------ heartbeat
    def heartbeat(self, name: str, incarnation_id: str, payload: Dict[str, Any]) -> Dict[str, Any]:
        """Keeps the lease alive and folds in the load / latency / cache-event report.  An unknown name or an older
        incarnation gets `registered: false`, which makes the client register again (reconcile loop)."""
        with self._lock:
            st = self._instances.get(name)
            if st is None or st.info.incarnation_id != incarnation_id:
                return {"ok": False, "registered": False}
            now = self._clock()
            st.lease_deadline = now + st.ttl_s
            st.last_heartbeat = now
            lm = payload.get("load_metrics") or {}
            st.cache_usage = float(lm.get("gpu_cache_usage_perc", st.cache_usage))
            st.waiting_requests = int(lm.get("waiting_requests_num", st.waiting_requests))
            st.running_requests = int(lm.get("running_requests_num", st.running_requests))
            lat = payload.get("latency_metrics") or {}
            st.recent_max_ttft_ms = float(lat.get("recent_max_ttft", st.recent_max_ttft_ms))
            st.recent_max_tbt_ms = float(lat.get("recent_max_tbt", st.recent_max_tbt_ms))
            ev = payload.get("cache_event") or {}
            for k in ev.get("stored_cache") or ():
                st.cached_keys.add((int(k[0]), int(k[1])))
            for k in ev.get("removed_cache") or ():
                st.cached_keys.discard((int(k[0]), int(k[1])))
            return {"ok": True, "registered": True}

    # ------------------------------------------------------------------ queries
    def get(self, name: str) -> Optional[InstanceState]:
        with self._lock:
            return self._instances.get(name)

    def instances(self, role: Optional[str] = None) -> List[InstanceState]:
        with self._lock:
            return [st for st in self._instances.values() if role is None or st.info.type == role]

    def names(self, role: Optional[str] = None) -> List[str]:
        return sorted(st.info.name for st in self.instances(role))

    def wait_for_change(self, since_revision: int, timeout_s: float) -> Tuple[int, List[Tuple[int, str, str]]]:
        """Blocks until the registry moved past `since_revision` (or the timeout); returns the new revision and the
        events in between."""
        with self._lock:
            deadline = time.monotonic() + timeout_s
            while self.revision <= since_revision:
                left = deadline - time.monotonic()
                if left <= 0:
                    break
                self._lock.wait(left)
            return self.revision, [e for e in self.events if e[0] > since_revision]

    def track(self, name: str, delta: int) -> None:
        with self._lock:
            st = self._instances.get(name)
            if st is not None:
                st.inflight = max(0, st.inflight + delta)
