"""Instance health state and worker liveness checks.

Reference: xllm/core/common/health_check_manager.h:34-120 (a master thread polls every worker each
`health_check_interval_ms`; one failure marks the instance unhealthy with a reason; `/health` reports
it).  Here a check is any callable returning (ok, reason); the engine registers one per rank process
(process liveness + step-channel acknowledgement age)."""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, Optional, Tuple

Check = Callable[[], Tuple[bool, str]]


class HealthCheckManager:
    def __init__(self):
        self._lock = threading.Lock()
        self._healthy = True
        self._reason = ""
        self._checks: Dict[str, Check] = {}
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.failures = 0

    def register(self, name: str, check: Check):
        with self._lock:
            self._checks[name] = check

    def unregister(self, name: str):
        with self._lock:
            self._checks.pop(name, None)

    def set_unhealthy(self, reason: str):
        with self._lock:
            self._healthy, self._reason = False, reason
            self.failures += 1

    def set_healthy(self):
        with self._lock:
            self._healthy, self._reason = True, ""

    def status(self) -> Tuple[bool, str]:
        with self._lock:
            return self._healthy, self._reason

    def run_checks_once(self) -> Tuple[bool, str]:
        with self._lock:
            checks = list(self._checks.items())
        for name, c in checks:
            try:
                ok, why = c()
            except Exception as e:
                ok, why = False, f"{type(e).__name__}: {e}"
            if not ok:
                self.set_unhealthy(f"{name}: {why}")
                return False, f"{name}: {why}"
        return self.status()

    def start(self, interval_ms: int = 3000):
        if self._thread is not None:
            return
        self._stop.clear()

        def loop():
            while not self._stop.wait(interval_ms / 1000.0):
                self.run_checks_once()
        self._thread = threading.Thread(target=loop, name="xllm-health", daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
            self._thread = None


HEALTH = HealthCheckManager()
