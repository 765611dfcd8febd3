"""Timing, quality metrics and result I/O shared by the experiments.

Same roles as the reference's ``microbench/bench_utils.py:18-180``: CUDA-event timing with median / quartiles,
paired speed-ups, singular-value and cosine quality of an orthogonalised matrix, JSON results under
``microbench/data/`` (git-ignored).  Every timing flushes the L2 cache between iterations.
"""

from __future__ import annotations

import json
import os
import statistics
import time

import torch

DATA_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")
_FLUSH = None


def _flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def measure(fn, warmup: int = 5, iters: int = 20, flush_l2: bool = True) -> dict:
    """Median / p25 / p75 / mean milliseconds of ``fn()`` (CUDA events on GPU, perf_counter on CPU)."""
    cuda = torch.cuda.is_available()
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if cuda:
            if flush_l2:
                _flush_l2()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    times.sort()
    q = statistics.quantiles(times, n=4) if len(times) >= 4 else [times[0], times[len(times) // 2], times[-1]]
    return {"median_ms": statistics.median(times), "p25_ms": q[0], "p75_ms": q[2], "mean_ms": statistics.fmean(times),
            "iters": iters}


def measure_paired_speedup(baseline_fn, candidate_fn, warmup: int = 5, iters: int = 20) -> dict:
    """Interleaved timing of two callables; speed-up = baseline / candidate per pair, then the median."""
    for _ in range(warmup):
        baseline_fn()
        candidate_fn()
    ratios, base, cand = [], [], []
    for _ in range(iters):
        b = measure(baseline_fn, warmup=0, iters=1)["median_ms"]
        c = measure(candidate_fn, warmup=0, iters=1)["median_ms"]
        base.append(b)
        cand.append(c)
        ratios.append(b / c)
    return {"speedup_median": statistics.median(ratios), "baseline_ms": statistics.median(base),
            "candidate_ms": statistics.median(cand)}


def polar_factor(x: torch.Tensor) -> torch.Tensor:
    """Exact orthogonal polar factor ``U V^T`` in fp64."""
    U, _, Vh = torch.linalg.svd(x.double(), full_matrices=False)
    return U @ Vh


def orth_quality(y: torch.Tensor, x: torch.Tensor) -> dict:
    """How close ``y`` is to the polar factor of ``x``: cosine, relative Frobenius error, singular-value range."""
    p = polar_factor(x)
    yd = y.double()
    cos = (yd * p).sum() / (yd.norm() * p.norm() + 1e-30)
    sv = torch.linalg.svdvals(yd)
    return {"cosine": float(cos), "rel_fro_err": float((yd - p).norm() / p.norm()), "sv_min": float(sv.min()),
            "sv_max": float(sv.max())}


def device_name() -> str:
    return torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"


def save_results(name: str, data: dict) -> str:
    os.makedirs(DATA_DIR, exist_ok=True)
    path = os.path.join(DATA_DIR, f"{name}.json")
    payload = {"experiment": name, "device": device_name(), "torch": torch.__version__, "time": time.strftime("%Y-%m-%d %H:%M:%S"),
               "data": data}
    with open(path, "w") as f:
        json.dump(payload, f, indent=1)
    return path


def load_results(name: str) -> dict:
    with open(os.path.join(DATA_DIR, f"{name}.json")) as f:
        return json.load(f)
