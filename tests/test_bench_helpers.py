"""bench.py's clock sampler against a fake NVML: it must collect samples within a few
milliseconds, decode the throttle-reason bits, and never touch a setting."""
import importlib
import os
import sys
import time
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def fake_nvml(reason_bits):
    m = types.ModuleType("pynvml")
    m.calls = []
    m.NVML_CLOCK_SM = 1
    m.nvmlInit = lambda: m.calls.append("init")
    m.nvmlDeviceGetHandleByIndex = lambda i: m.calls.append(("handle", i)) or ("gpu", i)
    m.nvmlDeviceGetClockInfo = lambda h, kind: 1965
    m.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965
    m.nvmlDeviceGetCurrentClocksEventReasons = lambda h: reason_bits
    return m


def load_bench(monkeypatch, module):
    monkeypatch.setitem(sys.modules, "pynvml", module)
    monkeypatch.syspath_prepend(ROOT)
    sys.modules.pop("bench", None)
    return importlib.import_module("bench")


def test_sampler_collects_within_milliseconds_and_decodes_reasons(monkeypatch):
    nvml = fake_nvml(0x4 | 0x40)  # sw_power_cap + hw_thermal_slowdown
    bench = load_bench(monkeypatch, nvml)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,5,6,7")
    s = bench.ClockSampler(2)
    assert ("handle", 6) in nvml.calls  # local rank 2 of the visible list is physical GPU 6
    s.start()
    time.sleep(0.02)
    out = s.stop()
    assert out["samples"] >= 3 and out["sm_mhz"] == 1965.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]
    # Read-only: nothing but queries was ever called on the module.
    assert not any(name.startswith("nvmlDeviceSet") or "Reset" in name for name in dir(nvml))


def test_sampler_reports_idle_reasons_as_empty(monkeypatch):
    bench = load_bench(monkeypatch, fake_nvml(0x1))  # gpu_idle only: not one of the reported reasons
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.005)
    assert s.stop()["reasons"] == []


def test_percentile():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.percentile([1, 2, 3, 4], 0.5) in (2, 3)
    assert bench.percentile([], 0.5) is None
