"""Named timers / counters (native registry with mean, P50, P99 and an ASCII report) plus CUDA-event
timing and NVTX ranges.

``Timer`` / ``PerfCounter`` / ``Reporter`` mirror the reference's ``timer_module``
(src/base/pybind_timer.cc:9-22) and its Python wrappers ``Timer``, ``GPUTimer``, ``PerfCounter``,
``xmh_nvtx_range`` (src/python/pytorch/recstore/utils.py:107-180).  ``DeviceTimer`` measures a region
with CUDA events on the launching stream (what the benchmarks report), never by host clock.
"""
from __future__ import annotations

import contextlib
import ctypes as C

import torch

from .. import _lib
from .._lib import cstr, f64, i32, u64, vp

_lib.register_signatures({
    "rs_now_ns": (u64, []),
    "rs_timer_get": (vp, [cstr]),
    "rs_counter_get": (vp, [cstr]),
    "rs_series_record": (None, [vp, f64]),
    "rs_timer_record_ns": (None, [cstr, f64]),
    "rs_counter_record": (None, [cstr, f64]),
    "rs_series_stats": (i32, [cstr, C.POINTER(f64)]),
    "rs_report": (i32, [C.c_char_p, i32]),
    "rs_report_thread_start": (i32, [i32]),
    "rs_report_thread_stop": (i32, []),
    "rs_timers_clear": (None, []),
    "rs_hist_new": (vp, []),
    "rs_hist_delete": (None, [vp]),
    "rs_hist_clear": (None, [vp]),
    "rs_hist_add": (None, [vp, f64]),
    "rs_hist_add_many": (None, [vp, C.POINTER(f64), C.c_longlong]),
    "rs_hist_merge": (None, [vp, vp]),
    "rs_hist_percentile": (f64, [vp, f64]),
    "rs_hist_summary": (None, [vp, C.POINTER(f64)]),
    "rs_hist_to_string": (i32, [vp, C.c_char_p, i32]),
})


class Timer:
    """``t = Timer("Forward"); t.Start(); ...; t.End()``; every ``sampling``-th interval is recorded."""

    def __init__(self, name: str, sampling: int = 1):
        self._l = _lib.lib()
        self.name = name
        self._h = self._l.rs_timer_get(name.encode())
        self._sampling = max(1, int(sampling))
        self._n = 0
        self._t0 = 0

    def Start(self):
        self._t0 = self._l.rs_now_ns()

    def End(self):
        self._n += 1
        if self._n % self._sampling == 0:
            self._l.rs_series_record(self._h, float(self._l.rs_now_ns() - self._t0))

    start, stop = Start, End

    # Cumulative form: several separate intervals add up to ONE sample (e.g. the pieces of a phase that is interleaved
    # with others inside a step): CumStart / CumEnd around every piece, CumReport once per step
    # (src/base/timer.h:426-450).
    def CumStart(self):
        self._t0 = self._l.rs_now_ns()

    def CumEnd(self):
        self._cum = getattr(self, "_cum", 0) + (self._l.rs_now_ns() - self._t0)

    def CumReport(self):
        self._l.rs_series_record(self._h, float(getattr(self, "_cum", 0)))
        self._cum = 0

    def __enter__(self):
        self.Start()
        return self

    def __exit__(self, *a):
        self.End()

    @staticmethod
    def ManualRecordNs(name: str, ns: float):
        _lib.lib().rs_timer_record_ns(name.encode(), float(ns))


class GPUTimer(Timer):
    """Host timer around a device region: synchronises before reading the clock, opens an NVTX range."""

    def Start(self):
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
            torch.cuda.synchronize()
        super().Start()

    def End(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
        super().End()

    start, stop = Start, End


class DeviceTimer:
    """Device-side time of a region (CUDA events on the current stream), recorded under ``name`` in ns."""

    def __init__(self, name: str):
        self.name = name
        self._e0 = torch.cuda.Event(enable_timing=True)
        self._e1 = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self._e0.record()
        return self

    def __exit__(self, *a):
        self._e1.record()

    def elapsed_ms(self) -> float:
        self._e1.synchronize()
        ms = self._e0.elapsed_time(self._e1)
        Timer.ManualRecordNs(self.name, ms * 1e6)
        return ms


class PerfCounter:
    @staticmethod
    def Record(name: str, value: float):
        _lib.lib().rs_counter_record(name.encode(), float(value))


class Reporter:
    @staticmethod
    def StartReportThread(period_ms: int = 5000):
        _lib.call("rs_report_thread_start", int(period_ms))

    @staticmethod
    def StopReportThread():
        _lib.call("rs_report_thread_stop")

    @staticmethod
    def Report() -> str:
        l = _lib.lib()
        n = l.rs_report(None, 0)
        buf = C.create_string_buffer(n + 1)
        l.rs_report(buf, n + 1)
        return buf.value.decode()

    @staticmethod
    def Clear():
        _lib.lib().rs_timers_clear()


class Histogram:
    """Distribution of a measurement over its whole life: count, min / max, mean, standard deviation and percentiles
    from log-linear buckets (8 per power of two, so a percentile is within 1/16 of the true value), mergeable across
    threads or ranks, printable with bars (role of the reference's ``Histogram``, src/base/timer.h:102-204)."""

    def __init__(self):
        self._l = _lib.lib()
        self._h = self._l.rs_hist_new()
        if not self._h:
            raise MemoryError("Histogram")

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._l.rs_hist_delete(self._h)
            self._h = None

    __del__ = close

    def Clear(self) -> None:
        self._l.rs_hist_clear(self._h)

    def Add(self, value) -> None:
        """One value, or a sequence / tensor of values."""
        if isinstance(value, (int, float)):
            self._l.rs_hist_add(self._h, float(value))
            return
        v = torch.as_tensor(value, dtype=torch.float64).reshape(-1).contiguous().cpu()
        self._l.rs_hist_add_many(self._h, C.cast(v.data_ptr(), C.POINTER(f64)), v.numel())

    def Merge(self, other: "Histogram") -> None:
        self._l.rs_hist_merge(self._h, other._h)

    def Percentile(self, p: float) -> float:
        return float(self._l.rs_hist_percentile(self._h, float(p)))

    def Median(self) -> float:
        return self.Percentile(50.0)

    def summary(self) -> dict:
        out = (f64 * 5)()
        self._l.rs_hist_summary(self._h, out)
        return {"count": int(out[0]), "min": out[1], "max": out[2], "mean": out[3], "stddev": out[4]}

    def ToString(self) -> str:
        n = self._l.rs_hist_to_string(self._h, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._l.rs_hist_to_string(self._h, buf, n + 1)
        return buf.value.decode()

    __str__ = ToString


def stats(name: str) -> dict:
    """{'mean','p50','p99','last','count'} of a timer (ns) or counter."""
    out = (f64 * 5)()
    _lib.call("rs_series_stats", name.encode(), out)
    return {"mean": out[0], "p50": out[1], "p99": out[2], "last": out[3], "count": int(out[4])}


@contextlib.contextmanager
def nvtx_range(msg: str, enabled: bool = True):
    if enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(msg)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield
