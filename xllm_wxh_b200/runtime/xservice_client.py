"""Client of the service layer inside an engine instance: registration with a lease, heartbeats, re-registration.

Role of the reference's XServiceClient (xllm/core/runtime/xservice_client.h:37-110; .cpp:72-147 init, :167-218
registration with retry and the reconcile loop, :220-262 register_instance, :322-417 heartbeat with load metrics,
latency metrics and prefix-cache events, :418-463 static prefill / decode lists).  The reference speaks etcd and brpc; this
client speaks HTTP + JSON to `service/router.py`.

A heartbeat carries
    load_metrics     gpu_cache_usage_perc, waiting_requests_num, running_requests_num
    latency_metrics  recent_max_ttft, recent_max_tbt   (ms, maxima since the previous heartbeat)
    cache_event      stored_cache / removed_cache: prefix keys that entered / left the device prefix cache
and renews the lease.  When the service answers that it does not know this incarnation (it restarted, or the lease ran
out during a stall), the client registers again and re-sends its whole cache content with the next heartbeat.
"""
from __future__ import annotations

import http.client
import json
import logging
import threading
import time
import uuid
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..service.registry import InstanceInfo

log = logging.getLogger("xllm.xservice")


class XServiceClient:
    def __init__(self, service_addr: str, heart_beat_interval: float = 0.5, ttl_s: float = 3.0, timeout_s: float = 2.0):
        host, _, port = service_addr.rpartition(":")
        self.host, self.port = host or "127.0.0.1", int(port)
        self.interval, self.ttl_s, self.timeout_s = heart_beat_interval, ttl_s, timeout_s
        self.incarnation_id = uuid.uuid4().hex
        self.info: Optional[InstanceInfo] = None
        self.register_done = False
        self.num_registrations = 0
        self.num_heartbeats = 0
        self._exited = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()
        # sources of the heartbeat payload (set_scheduler / set_master)
        self._load_fn: Optional[Callable[[], Dict[str, Any]]] = None
        self._latency_fn: Optional[Callable[[], Dict[str, float]]] = None
        self._cache_events_fn: Optional[Callable[[], Tuple[List, List]]] = None
        self._known_keys: set = set()

    # ------------------------------------------------------------------ transport
    def _call(self, method: str, path: str, body: Optional[Dict[str, Any]] = None) -> Optional[Dict[str, Any]]:
        try:
            c = http.client.HTTPConnection(self.host, self.port, timeout=self.timeout_s)
            data = json.dumps(body).encode() if body is not None else None
            c.request(method, path, data, {"Content-Type": "application/json", "Connection": "close"})
            r = c.getresponse()
            raw = r.read()
            c.close()
            return json.loads(raw) if raw else {}
        except (OSError, ValueError) as e:
            log.debug("xservice call %s failed: %s", path, e)
            return None

    # ------------------------------------------------------------------ wiring
    def set_scheduler(self, scheduler, dp_size: int = 1) -> None:
        """Load metrics and cache events come straight from the C++ scheduler and its block managers."""
        for d in range(dp_size):
            scheduler.block_manager(d).record_cache_events(True)

        def load():
            return {"gpu_cache_usage_perc": float(scheduler.kv_utilization),
                    "waiting_requests_num": int(scheduler.num_waiting) + int(scheduler.num_pending),
                    "running_requests_num": int(scheduler.num_running)}

        def events():
            stored, removed = [], []
            for d in range(dp_size):
                s, r = scheduler.block_manager(d).take_cache_events()
                stored += s
                removed += r
            return stored, removed
        self._load_fn, self._cache_events_fn = load, events

    def set_master(self, master) -> None:
        self._latency_fn = master.take_latency_metrics

    # ------------------------------------------------------------------ registration
    def register_instance(self, info: InstanceInfo, retries: int = 5, backoff_s: float = 0.2) -> bool:
        """Registers under the role's key with a lease; retried with back-off (register_instance_with_retry)."""
        info.incarnation_id = self.incarnation_id
        if not info.register_ts_ms:
            info.register_ts_ms = int(time.time() * 1e3)
        with self._lock:
            self.info = info
        for attempt in range(max(1, retries)):
            r = self._call("POST", "/xservice/register", {"info": info.to_json(), "ttl_s": self.ttl_s})
            if r and r.get("ok"):
                self.register_done = True
                self.num_registrations += 1
                return True
            time.sleep(backoff_s * (attempt + 1))
        return False

    def deregister(self) -> None:
        if self.info is not None:
            self._call("POST", "/xservice/deregister", {"name": self.info.name})
        self.register_done = False

    # ------------------------------------------------------------------ heartbeat
    def heartbeat_once(self) -> bool:
        """One heartbeat; returns False when the service did not take it (unreachable, or it asked for re-registration,
        which is then done at once)."""
        if self.info is None:
            return False
        payload: Dict[str, Any] = {"name": self.info.name, "incarnation_id": self.incarnation_id}
        if self._load_fn is not None:
            payload["load_metrics"] = self._load_fn()
        if self._latency_fn is not None:
            payload["latency_metrics"] = self._latency_fn()
        if self._cache_events_fn is not None:
            stored, removed = self._cache_events_fn()
            for k in stored:
                self._known_keys.add(tuple(k))
            for k in removed:
                self._known_keys.discard(tuple(k))
            payload["cache_event"] = {"stored_cache": [list(k) for k in stored], "removed_cache": [list(k) for k in removed]}
        r = self._call("POST", "/xservice/heartbeat", payload)
        if r is None:
            return False
        self.num_heartbeats += 1
        if not r.get("registered", True):
            # the service lost us: register again and replay the cache content it has forgotten
            self.register_done = False
            if self.register_instance(self.info, retries=1):
                replay = {"name": self.info.name, "incarnation_id": self.incarnation_id,
                          "cache_event": {"stored_cache": [list(k) for k in self._known_keys], "removed_cache": []}}
                if self._load_fn is not None:
                    replay["load_metrics"] = self._load_fn()
                self._call("POST", "/xservice/heartbeat", replay)
            return False
        return True

    def start(self) -> None:
        def loop():
            while not self._exited.wait(self.interval):
                if self.info is None:
                    continue
                try:
                    if not self.register_done:
                        self.register_instance(self.info, retries=1)       # reconcile loop
                    else:
                        self.heartbeat_once()
                except Exception as e:                                    # the serving loop must not die with the service
                    log.warning("heartbeat failed: %s", e)
        self._thread = threading.Thread(target=loop, name="xservice-heartbeat", daemon=True)
        self._thread.start()

    def stop(self, deregister: bool = True) -> None:
        self._exited.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        if deregister:
            self.deregister()

    # ------------------------------------------------------------------ queries
    def get_instance_info(self, name: str) -> Optional[InstanceInfo]:
        r = self._call("GET", f"/xservice/instance?name={name}")
        return InstanceInfo.from_json(r["info"]) if r and "info" in r else None

    def _list(self, role: str) -> List[str]:
        r = self._call("GET", f"/xservice/instances?type={role}")
        return sorted(i["name"] for i in r["instances"]) if r else []

    def get_static_prefill_list(self) -> List[str]:
        return self._list("PREFILL")

    def get_static_decode_list(self) -> List[str]:
        return self._list("DECODE")

    def watch(self, revision: int, timeout_s: float = 5.0) -> Tuple[int, List[Dict[str, Any]]]:
        old, self.timeout_s = self.timeout_s, timeout_s + 2.0
        try:
            r = self._call("GET", f"/xservice/watch?revision={revision}&timeout={timeout_s}")
        finally:
            self.timeout_s = old
        return (int(r["revision"]), r["events"]) if r else (revision, [])


def attach_to_master(master, options) -> Optional[XServiceClient]:
    """`--enable_service_routing --etcd_addr host:port`: register this instance with the service and start heartbeats
    (the reference does this in LLMMaster's constructor, llm_master.cpp, through XServiceClient::get_instance())."""
    if not getattr(options, "enable_service_routing", False) or not options.etcd_addr:
        return None
    c = XServiceClient(options.etcd_addr, heart_beat_interval=options.heart_beat_interval, ttl_s=float(options.etcd_ttl))
    eng = master.engine
    c.set_scheduler(eng.scheduler, max(1, options.dp_size))
    c.set_master(master)
    host = options.host if options.host not in ("", "0.0.0.0") else "127.0.0.1"
    info = InstanceInfo(name=options.instance_name or f"{host}:{options.port}", rpc_address=f"{host}:{options.port}",
                        type=options.instance_role if options.instance_role in ("PREFILL", "DECODE", "MIX") else "DEFAULT",
                        dp_size=options.dp_size, block_size=options.block_size, hash_seed=options.xxh3_128bits_seed,
                        model=str(master.model_id), kv_transfer_port=options.transfer_listen_port,
                        pd_port=options.disagg_pd_port if options.instance_role == "DECODE" else 0)
    prof = getattr(master, "profiler", None)
    if prof is not None:
        info.ttft_profiling_data = [(int(n), float(t)) for n, _, t in prof.samples.get("prefill", [])]
        info.tpot_profiling_data = [(int(b), int(kv), float(t)) for b, kv, t in prof.samples.get("decode", [])]
    if not c.register_instance(info):
        log.warning("could not register with the service at %s; will keep trying", options.etcd_addr)
    c.start()
    return c
