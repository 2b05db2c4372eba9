"""Per-device memory accounting and read-only hardware readings.

Role of the reference's `DeviceMonitor` (xllm/core/common/device_monitor.h:27-50: total / weight / KV-cache / activation
memory per device, fed by the workers and shown by the metrics): here one `DeviceStats` per device of the process, filled
by the engine (weights, KV cache), by the torch allocator's own counters (activations = peak allocated beyond weights and
cache) and, when NVML answers, by its read-only queries (memory in use by all processes, SM / memory utilisation,
temperature, power draw, SM clock).  Nothing here changes a setting of the GPU."""
from __future__ import annotations

import dataclasses
import threading
from typing import Callable, Dict, Optional


@dataclasses.dataclass
class DeviceStats:
    total_memory: int = 0
    weight_memory: int = 0
    total_kv_cache_memory: int = 0
    total_activation_memory: int = 0          # largest amount seen beyond weights and KV cache
    active_activation_memory: int = 0         # at the last update
    temp_buffer_memory: int = 0               # registered work buffers (peer-visible TP / EP buffers, staging)
    # hardware readings (None: no NVML, or the query is not supported)
    used_memory: Optional[int] = None
    sm_utilization: Optional[int] = None
    mem_utilization: Optional[int] = None
    temperature_c: Optional[int] = None
    power_w: Optional[float] = None
    sm_clock_mhz: Optional[int] = None


class DeviceMonitor:
    """`nvml`: an object with the `pynvml` functions used below (a fake in tests); None: import `pynvml` lazily, and do
    without hardware readings when that fails."""

    def __init__(self, nvml=None, allocator: Optional[Callable[[int], Dict[str, int]]] = None):
        self._lock = threading.Lock()
        self._stats: Dict[int, DeviceStats] = {}
        self._nvml = nvml
        self._nvml_ok: Optional[bool] = None if nvml is None else True
        self._handles: Dict[int, object] = {}
        self._allocator = allocator

    # ------------------------------------------------------------------ accounting fed by the engine
    def stats(self, device_id: int) -> DeviceStats:
        with self._lock:
            return self._stats.setdefault(device_id, DeviceStats())

    def set_total_memory(self, device_id: int, nbytes: int):
        self.stats(device_id).total_memory = int(nbytes)

    def set_weight_memory(self, device_id: int, nbytes: int):
        self.stats(device_id).weight_memory = int(nbytes)

    def set_total_kv_cache_memory(self, device_id: int, nbytes: int):
        self.stats(device_id).total_kv_cache_memory = int(nbytes)

    def monitor_buffer(self, device_id: int, nbytes: int):
        self.stats(device_id).temp_buffer_memory += int(nbytes)

    def update_active_activation_memory(self, device_id: int):
        """Allocated bytes beyond weights, cache and registered buffers, now and at its peak."""
        s = self.stats(device_id)
        a = self._allocator_stats(device_id)
        if a is None:
            return
        fixed = s.weight_memory + s.total_kv_cache_memory + s.temp_buffer_memory
        s.active_activation_memory = max(0, a.get("allocated", 0) - fixed)
        s.total_activation_memory = max(s.total_activation_memory, a.get("peak", 0) - fixed, s.active_activation_memory)

    def _allocator_stats(self, device_id: int):
        if self._allocator is not None:
            return self._allocator(device_id)
        try:
            import torch
            if not torch.cuda.is_available():
                return None
            return {"allocated": torch.cuda.memory_allocated(device_id), "peak": torch.cuda.max_memory_allocated(device_id)}
        except Exception:
            return None

    # ------------------------------------------------------------------ read-only hardware readings
    def _nvml_handle(self, device_id: int):
        if self._nvml_ok is False:
            return None
        if self._nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                self._nvml, self._nvml_ok = pynvml, True
            except Exception:
                self._nvml_ok = False
                return None
        h = self._handles.get(device_id)
        if h is None:
            try:
                h = self._nvml.nvmlDeviceGetHandleByIndex(device_id)
            except Exception:
                return None
            self._handles[device_id] = h
        return h

    def poll_hardware(self, device_id: int) -> DeviceStats:
        s = self.stats(device_id)
        h = self._nvml_handle(device_id)
        if h is None:
            return s
        n = self._nvml

        def q(fn, *a):
            try:
                return fn(h, *a)
            except Exception:
                return None
        mem = q(n.nvmlDeviceGetMemoryInfo)
        if mem is not None:
            s.used_memory = int(mem.used)
            if not s.total_memory:
                s.total_memory = int(mem.total)
        util = q(n.nvmlDeviceGetUtilizationRates)
        if util is not None:
            s.sm_utilization, s.mem_utilization = int(util.gpu), int(util.memory)
        t = q(n.nvmlDeviceGetTemperature, getattr(n, "NVML_TEMPERATURE_GPU", 0))
        s.temperature_c = int(t) if t is not None else None
        pw = q(n.nvmlDeviceGetPowerUsage)
        s.power_w = pw / 1000.0 if pw is not None else None
        clk = q(n.nvmlDeviceGetClockInfo, getattr(n, "NVML_CLOCK_SM", 1))
        s.sm_clock_mhz = int(clk) if clk is not None else None
        return s

    def export(self, metrics, device_id: int, hardware: bool = True):
        """Gauges of one device, under the reference's names where it has them (metrics.h: weight / KV-cache / activation
        sizes in kilobytes)."""
        self.update_active_activation_memory(device_id)
        s = self.poll_hardware(device_id) if hardware else self.stats(device_id)
        metrics.set("weight_size_in_kilobytes", s.weight_memory / 1024)
        metrics.set("total_kv_cache_size_in_kilobytes", s.total_kv_cache_memory / 1024)
        metrics.set("total_activation_size_in_kilobytes", s.total_activation_memory / 1024)
        metrics.set("active_activation_size_in_kilobytes", s.active_activation_memory / 1024)
        metrics.set("total_device_memory_in_kilobytes", s.total_memory / 1024)
        for name, v in (("device_used_memory_in_kilobytes", None if s.used_memory is None else s.used_memory / 1024),
                        ("device_sm_utilization_perc", s.sm_utilization), ("device_memory_utilization_perc", s.mem_utilization),
                        ("device_temperature_celsius", s.temperature_c), ("device_power_watts", s.power_w),
                        ("device_sm_clock_mhz", s.sm_clock_mhz)):
            if v is not None:
                metrics.set(name, v)
        return s


DEVICE_MONITOR = DeviceMonitor()
