"""Timing helpers shared by bench.py, the quantization sweep and the GEMM sweep.

All device times come from CUDA events recorded on the stream the work is launched on (torch's current stream);
clocks and throttle reasons are READ through NVML while a timed region runs - nothing here changes a GPU setting.
"""
from __future__ import annotations

import threading
import time

import torch


class ClockSampler(threading.Thread):
    """Samples SM clock, power and clock-event reasons through NVML every `period_s` (read-only)."""

    _NAMES = (
        ("nvmlClocksEventReasonSwPowerCap", 0x4, "sw_power_cap"),
        ("nvmlClocksEventReasonHwSlowdown", 0x8, "hw_slowdown"),
        ("nvmlClocksEventReasonSwThermalSlowdown", 0x20, "sw_thermal_slowdown"),
        ("nvmlClocksEventReasonHwThermalSlowdown", 0x40, "hw_thermal_slowdown"),
        ("nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80, "hw_power_brake_slowdown"),
    )

    def __init__(self, index: int, period_s: float = 0.001):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples: list[tuple[float, int, int, float]] = []   # (time, MHz, reason mask, watts)
        self.max_mhz = None
        self._stop_evt = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.names = {getattr(pynvml, attr, bit): name for attr, bit, name in self._NAMES}
        except Exception:  # noqa: BLE001 - no NVML: the sampler reports nothing
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        while not self._stop_evt.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:  # noqa: BLE001
                    watts = 0.0
                self.samples.append((time.perf_counter(), mhz, mask, watts))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()

    def window(self, t0: float, t1: float) -> dict:
        """Median SM MHz, active reasons and peak power over the samples taken in [t0, t1]."""
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        mhz = sorted(s[1] for s in inside)
        reasons = set()
        for s in inside:
            for bit, name in self.names.items():
                if s[2] & bit:
                    reasons.add(name)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(reasons), "samples": len(inside),
                "power_w_max": max((s[3] for s in inside), default=None)}


def time_launches(fn, reps: int, warmup: int = 3) -> float:
    """Mean milliseconds of fn(i) over `reps` back-to-back calls (CUDA events on the current stream)."""
    for i in range(warmup):
        fn(i)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for i in range(reps):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


def time_sustained(fn, min_seconds: float, sampler: ClockSampler | None, est_ms: float | None = None) -> dict:
    """Back-to-back calls of fn(i) for at least `min_seconds` of device time; returns mean us per call, the clock
    record of that window and us x median MHz (what the same work would cost at a given clock)."""
    if est_ms is None:
        est_ms = time_launches(fn, 5)
    reps = max(10, int(min_seconds * 1e3 / max(est_ms, 1e-4)) + 1)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    s.record()
    for i in range(reps):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    us = s.elapsed_time(e) / reps * 1e3
    out = {"us": us, "launches": reps, "seconds": s.elapsed_time(e) * 1e-3}
    if sampler is not None:
        w = sampler.window(t0, t1)
        out.update(sm_mhz_median=w["sm_mhz"], reasons=w["reasons"], clock_samples=w["samples"],
                   power_w_max=w["power_w_max"],
                   us_x_mhz=(us * w["sm_mhz"]) if w["sm_mhz"] else None)
    return out


def time_graph(record, launches_per_replay: int, replays: int = 10) -> float:
    """Microseconds per launch of a sequence recorded by `record()` into a CUDA graph and replayed."""
    dev = torch.cuda.current_device()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        record()                         # warm-up outside capture
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        record()
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / (replays * launches_per_replay) * 1e3


def fp4_peak(sampler: ClockSampler | None = None) -> dict:
    """Measured rate of the GEMM's tensor-core instruction (tcgen05.mma kind::mxf4nvf4, CTA pairs) on operands
    resident in shared memory: a short burst (a few ms, boost clock) and a run long enough to sit under the power
    cap (~0.4 s).  TFLOP/s, with the clocks sampled during the long run."""
    import ctypes

    from . import _lib

    L = _lib.lib()
    stream = _lib.current_stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    sms = ctypes.c_int(0)

    def run(stages):
        _lib.check(L.nvfp4_gemm_peak_probe(stages, 1, ctypes.byref(sms), stream), "nvfp4_gemm_peak_probe")

    def timed(stages, reps):
        run(stages)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        s.record()
        for _ in range(reps):
            run(stages)
        e.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ms = s.elapsed_time(e) / reps
        flop = sms.value * stages * 4 * 2.0 * 128 * 256 * 64
        return flop / (ms * 1e-3) / 1e12, t0, t1

    burst, _, _ = timed(8192, 2)
    sustained, t0, t1 = timed(1 << 19, 2)
    out = {"burst_tflops": burst, "sustained_tflops": sustained, "sms": sms.value,
           "instruction": "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 256x256x64"}
    if sampler is not None:
        w = sampler.window(t0, t1)
        out.update(sustained_sm_mhz=w["sm_mhz"], sustained_reasons=w["reasons"], sustained_power_w_max=w["power_w_max"])
    return out
