"""Host-side pieces of bench.py that need no GPU: the clock record."""
import sys
import time
import types

import bench


def _fake_nvml(clock=1500, max_clock=1965, reasons=0x4, milliwatts=987000, fail_handle=False):
    m = types.ModuleType("pynvml")
    m.NVML_CLOCK_SM = 1
    m.nvmlClocksThrottleReasonHwSlowdown = 0x8
    m.nvmlClocksThrottleReasonHwThermalSlowdown = 0x40
    m.nvmlClocksThrottleReasonSwThermalSlowdown = 0x20
    m.nvmlClocksThrottleReasonSwPowerCap = 0x4
    m.calls = []
    m.nvmlInit = lambda: None

    def by_bus(bus):
        if fail_handle:
            raise RuntimeError("no such device")
        m.calls.append(("bus", bus))
        return "handle"
    m.nvmlDeviceGetHandleByPciBusId = by_bus
    m.nvmlDeviceGetHandleByIndex = lambda i: m.calls.append(("index", i)) or "handle"
    m.nvmlDeviceGetMaxClockInfo = lambda h, which: max_clock
    m.nvmlDeviceGetClockInfo = lambda h, which: clock
    m.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: reasons
    m.nvmlDeviceGetPowerUsage = lambda h: milliwatts
    return m


def test_clock_record_from_nvml_reads(monkeypatch):
    fake = _fake_nvml()
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.delenv("HB_BENCH_CLOCK_SOURCE", raising=False)
    s = bench.ClockSampler(3, "0000:1b:00.0")
    s.start()
    time.sleep(0.05)
    rec = s.stop()
    assert fake.calls[0] == ("bus", b"0000:1b:00.0")           # the GPU is found by its bus id, not by an index
    assert rec["source"] == "nvml" and rec["samples"] >= 5
    assert rec["sm_mhz"] == 1500.0 and rec["sm_max_mhz"] == 1965.0
    assert rec["reasons"] == ["sw_power_cap"] and abs(rec["power_w_max"] - 987.0) < 1e-9


def test_clock_record_names_every_slowdown_reason(monkeypatch):
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml(reasons=0x8 | 0x20 | 0x40))
    monkeypatch.delenv("HB_BENCH_CLOCK_SOURCE", raising=False)
    s = bench.ClockSampler(0, None)
    s.start()
    time.sleep(0.02)
    assert s.stop()["reasons"] == ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"]


def test_clock_record_falls_back_when_nvml_does_not_answer(monkeypatch):
    # a handle that cannot be had, and no nvidia-smi on the path: the record says so and nothing raises
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml(fail_handle=True))
    monkeypatch.setenv("PATH", "/nonexistent")
    s = bench.ClockSampler(0, "0000:1b:00.0")
    s.start()
    rec = s.stop()
    assert rec["sm_mhz"] is None and rec["reasons"] == ["nvidia-smi unavailable"]
    # the switch skips NVML without trying it
    fake = _fake_nvml()
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setenv("HB_BENCH_CLOCK_SOURCE", "nvidia-smi")
    s = bench.ClockSampler(0, "0000:1b:00.0")
    s.start()
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"] and fake.calls == []
