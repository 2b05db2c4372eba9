"""Device monitor: memory accounting fed by the engine, hardware readings through a fake NVML (no GPU, no setting is
changed), export as metrics gauges."""
import types

from xllm_wxh_b200.utils.device_monitor import DeviceMonitor
from xllm_wxh_b200.utils.metrics import Metrics


class FakeNvml:
    NVML_TEMPERATURE_GPU, NVML_CLOCK_SM = 0, 1

    def __init__(self):
        self.calls = []

    def nvmlDeviceGetHandleByIndex(self, i):
        self.calls.append(("handle", i))
        return ("h", i)

    def nvmlDeviceGetMemoryInfo(self, h):
        return types.SimpleNamespace(total=180 << 30, used=100 << 30, free=80 << 30)

    def nvmlDeviceGetUtilizationRates(self, h):
        return types.SimpleNamespace(gpu=97, memory=61)

    def nvmlDeviceGetTemperature(self, h, which):
        return 64

    def nvmlDeviceGetPowerUsage(self, h):
        return 912345                    # milliwatts

    def nvmlDeviceGetClockInfo(self, h, which):
        raise RuntimeError("not supported")          # an unsupported query leaves its reading out


def test_memory_accounting_and_hardware_readings():
    alloc = {"allocated": 70 << 30, "peak": 75 << 30}
    nv = FakeNvml()
    mon = DeviceMonitor(nvml=nv, allocator=lambda dev: alloc)
    mon.set_weight_memory(0, 16 << 30)
    mon.set_total_kv_cache_memory(0, 50 << 30)
    mon.monitor_buffer(0, 1 << 30)
    m = Metrics()
    s = mon.export(m, 0)
    assert s.total_memory == 180 << 30 and s.used_memory == 100 << 30
    assert s.active_activation_memory == 3 << 30 and s.total_activation_memory == 8 << 30
    alloc["allocated"] = 68 << 30                       # activations shrink, the peak stays
    s = mon.export(m, 0)
    assert s.active_activation_memory == 1 << 30 and s.total_activation_memory == 8 << 30
    assert (s.sm_utilization, s.mem_utilization, s.temperature_c, s.sm_clock_mhz) == (97, 61, 64, None)
    assert abs(s.power_w - 912.345) < 1e-6
    g = m.gauges
    assert g["weight_size_in_kilobytes"] == (16 << 30) / 1024 and g["total_kv_cache_size_in_kilobytes"] == (50 << 30) / 1024
    assert g["device_sm_utilization_perc"] == 97 and "device_sm_clock_mhz" not in g
    assert nv.calls == [("handle", 0)]                 # one handle per device, reused
    # only read-only queries exist on the fake: any attempt to set something would have raised AttributeError


def test_without_nvml_only_the_accounting_is_reported():
    class Broken:
        def nvmlDeviceGetHandleByIndex(self, i):
            raise RuntimeError("no driver")
    mon = DeviceMonitor(nvml=Broken(), allocator=lambda dev: None)
    mon.set_weight_memory(1, 1024)
    m = Metrics()
    s = mon.export(m, 1)
    assert s.used_memory is None and m.gauges["weight_size_in_kilobytes"] == 1.0 and "device_power_watts" not in m.gauges
