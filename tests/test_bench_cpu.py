"""bench.py's clock sampler against a fake NVML (read-only queries; no GPU): samples inside the timed
window win, throttle bits decode to the reason names, a window shorter than the sampling period falls
back to the samples just before it."""
import sys
import time
import types

import bench


def _fake_nvml(clock=1900, reasons=0x4):
    m = types.ModuleType("pynvml")
    m.NVML_CLOCK_SM = 1
    m.calls = {"set": 0}
    m.nvmlInit = lambda: None
    m.nvmlDeviceGetHandleByUUID = lambda u: (_ for _ in ()).throw(RuntimeError("no such uuid"))
    m.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    m.nvmlDeviceGetMaxClockInfo = lambda h, which: 1965
    m.nvmlDeviceGetClockInfo = lambda h, which: clock
    m.nvmlDeviceGetCurrentClocksEventReasons = lambda h: reasons
    return m


def _first_sample(cs, limit=60.0):
    """The sampler thread imports its modules first; wait until it has produced a row."""
    t = time.perf_counter()
    while not cs.rows and time.perf_counter() - t < limit:
        time.sleep(0.01)
    assert cs.rows, "the sampler produced no sample"


def test_sampler_reads_clocks_and_reasons(monkeypatch):
    monkeypatch.setitem(sys.modules, "pynvml", _fake_nvml(clock=1342, reasons=0x4 | 0x20))
    with bench.ClockSampler(0) as cs:
        _first_sample(cs)
        t0 = time.perf_counter()
        n0 = len(cs.rows)
        while len(cs.rows) < n0 + 3 and time.perf_counter() - t0 < 30:       # until samples fall into the window, however busy the machine
            time.sleep(0.01)
        t1 = time.perf_counter()
        time.sleep(0.03)
    cs.mark(t0, t1)
    s = cs.summary()
    assert s["sm_mhz"] == 1342 and s["sm_max_mhz"] == 1965
    assert s["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]
    assert s["sampled_during"] == "timed region" and s["samples"] >= 1           # about 60 at one sample per 2 ms; no bound: the machine may be busy
    # a window shorter than the sampling period: the samples right before it are used, and the summary says so
    first = cs.rows[0][-1]
    cs.mark(first - 1.0, first - 0.9)          # a window that cannot hold a sample
    s2 = cs.summary()
    assert s2["samples"] >= 1 and "warm-up" in s2["sampled_during"]


def test_sampler_never_writes_a_setting(monkeypatch):
    """Only query functions exist on the fake: any attempt to set clocks, power or modes would raise AttributeError."""
    fake = _fake_nvml(reasons=0)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    with bench.ClockSampler(0) as cs:
        _first_sample(cs)
    s = cs.summary()
    assert s["reasons"] == [] and s["samples"] >= 1
