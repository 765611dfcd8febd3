"""Device-side timing helpers.

The reference only has host wall-clock ``--time-stats`` and a CUDA-event
microbench timer (``microbench/bench_utils.py:18-97``).  Everything here times
on the launching stream with CUDA events, reports the maximum over ranks, and
can sample SM clocks / throttle reasons while the timed region runs.
"""

from __future__ import annotations

import statistics
import subprocess
import threading

import torch


def l2_flush_buffer(device=None, nbytes: int = 256 << 20) -> torch.Tensor:
    """A buffer larger than the 126 MB L2; ``buf.zero_()`` between timed iterations evicts it."""
    return torch.empty(nbytes, dtype=torch.uint8, device=device or "cuda")


def cuda_time_ms(fn, warmup: int = 3, iters: int = 10, flush: torch.Tensor | None = None) -> list[float]:
    """Time ``fn()`` with CUDA events; returns the per-iteration milliseconds."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        out.append(start.elapsed_time(end))
    return out


def max_over_ranks(value: float, device=None) -> float:
    """All-reduce(MAX) of a python float when a process group is up; identity otherwise."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    dev = device if device is not None else ("cuda" if dist.get_backend() == "nccl" else "cpu")
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class nvtx_range:
    """``with nvtx_range("optimizer"):`` - an NVTX range around a phase of the step, visible on the timeline of any
    NVTX-aware profiler.  Does nothing without CUDA."""

    def __init__(self, name: str):
        self.name = name
        self._on = torch.cuda.is_available()

    def __enter__(self):
        if self._on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self._on:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """Per-phase device time of a training step (host-to-device copies, forward+backward, gradient reduction,
    optimizer, re-gather + reset), from CUDA events on the launching stream; every phase is also an NVTX range.

    ``with timer.phase("optimizer"): ...`` brackets a phase; ``timer.summary()`` synchronises once and returns the
    milliseconds per phase accumulated since the last ``reset()`` (each the maximum over ranks when a process group
    is up).  Disabled timers cost nothing: no events, no synchronisation.
    """

    def __init__(self, enabled: bool = False, device=None):
        self.enabled = bool(enabled) and torch.cuda.is_available()
        self.device = device
        self._events: dict[str, list] = {}

    class _Phase:
        def __init__(self, timer, name):
            self.timer, self.name = timer, name
            self.range = nvtx_range(name)

        def __enter__(self):
            self.range.__enter__()
            if self.timer.enabled:
                self.start = torch.cuda.Event(enable_timing=True)
                self.start.record()
            return self

        def __exit__(self, *exc):
            if self.timer.enabled:
                end = torch.cuda.Event(enable_timing=True)
                end.record()
                self.timer._events.setdefault(self.name, []).append((self.start, end))
            self.range.__exit__(*exc)

    def phase(self, name: str):
        return PhaseTimer._Phase(self, name)

    def reset(self):
        self._events = {}

    def summary(self, reduce_over_ranks: bool = True, reduce: str = "max") -> dict:
        """``reduce="max"`` gives each phase's longest time over the ranks; ``reduce="min"`` the shortest.  For a phase
        that waits on the other ranks (a collective after the backward pass) the shortest time is the collective
        itself, as seen by the rank that arrived last; the longest adds the time the first rank waited for the last."""
        if not self.enabled or not self._events:
            return {}
        torch.cuda.synchronize(self.device)
        out = {}
        for name, pairs in self._events.items():
            ms = sum(a.elapsed_time(b) for a, b in pairs)
            if not reduce_over_ranks:
                out[name] = ms
            elif reduce == "min":
                out[name] = -max_over_ranks(-ms)
            else:
                out[name] = max_over_ranks(ms)
        return out


class ClockSampler:
    """Samples ``nvidia-smi`` SM clocks and throttle reasons on a background thread.

    Read-only: it never changes a GPU setting.  ``summary()`` returns the median SM
    clock under load, the maximum SM clock and the list of active throttle reasons.
    """

    _QUERY = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )
    _REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int = 0, period_s: float = 0.2):
        self.index = index
        self.period_s = period_s
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self._QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5,
                ).stdout.strip()
                if out:
                    self.samples.append([c.strip() for c in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(self.period_s)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                sm_max.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(self._REASONS, s[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(sm_max) if sm_max else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }
