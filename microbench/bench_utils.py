"""Timing, memory, quality metrics, statistics, result I/O and the command-line scaffold shared by the experiments.

Same roles as the reference's ``microbench/bench_utils.py:18-188`` (CUDA-event timing with median / quartiles, peak
memory of a call, paired speed-ups, singular-value and cosine quality, JSON results under ``microbench/data/``), with
two differences that follow from how numbers are taken on a B200: every timed iteration starts with a cold L2 (a
256 MB buffer is rewritten in between, the L2 holds 126 MB), and the timing functions also run on a machine without a
GPU (``perf_counter``), so the numerics experiments can be exercised anywhere.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import time

import torch

DATA_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")
PLOTS_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plots")
_FLUSH = None


def have_cuda() -> bool:
    return torch.cuda.is_available()


def default_device() -> torch.device:
    return torch.device("cuda" if have_cuda() else "cpu")


def _flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


# ----------------------------------------------------------------------------------------------- statistics
def stats(values) -> tuple[float, float, float]:
    """``(median, p25, p75)`` with linear interpolation between order statistics; zeros for an empty list."""
    s = sorted(float(v) for v in values)
    n = len(s)
    if n == 0:
        return 0.0, 0.0, 0.0

    def at(q):
        pos = q * (n - 1)
        lo = int(math.floor(pos))
        hi = min(lo + 1, n - 1)
        return s[lo] + (pos - lo) * (s[hi] - s[lo])

    return at(0.5), at(0.25), at(0.75)


def mean_std(values) -> tuple[float, float]:
    v = [float(x) for x in values]
    if not v:
        return 0.0, 0.0
    return statistics.fmean(v), (statistics.stdev(v) if len(v) > 1 else 0.0)


# ----------------------------------------------------------------------------------------------- timing
def measure(fn, warmup: int = 5, iters: int = 20, flush_l2: bool = True, keep_raw: bool = False) -> dict:
    """Median / p25 / p75 / mean / min milliseconds of ``fn()`` (CUDA events on the current stream on a GPU,
    ``perf_counter`` otherwise).  ``keep_raw`` adds the list of samples."""
    cuda = have_cuda()
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
    med, p25, p75 = stats(times)
    out = {"median_ms": med, "p25_ms": p25, "p75_ms": p75, "mean_ms": statistics.fmean(times), "min_ms": min(times),
           "iters": iters}
    if keep_raw:
        out["raw_ms"] = times
    return out


def measure_memory(fn, repeats: int = 3) -> int:
    """Peak device bytes ``fn()`` allocates above what is live when it is called (minimum over ``repeats`` calls, which
    drops one-time allocations such as workspaces created on first use).  0 without a GPU."""
    if not have_cuda():
        fn()
        return 0
    samples = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        fn()
        torch.cuda.synchronize()
        samples.append(torch.cuda.max_memory_allocated() - base)
    return int(min(samples))


def measure_paired_speedup(baseline_fn, candidate_fn, warmup: int = 5, iters: int = 20) -> dict:
    """Interleaved timing of two callables: per pair ``baseline / candidate``, then median and quartiles of the ratios
    (clock drift under the power cap hits both members of a pair alike)."""
    for _ in range(warmup):
        baseline_fn()
        candidate_fn()
    ratios, base, cand = [], [], []
    for _ in range(iters):
        b = measure(baseline_fn, warmup=0, iters=1)["median_ms"]
        c = measure(candidate_fn, warmup=0, iters=1)["median_ms"]
        base.append(b)
        cand.append(c)
        if c > 0:
            ratios.append(b / c)
    med, p25, p75 = stats(ratios)
    return {"speedup_median": med, "speedup_p25": p25, "speedup_p75": p75, "baseline_ms": statistics.median(base),
            "candidate_ms": statistics.median(cand)}


# ----------------------------------------------------------------------------------------------- quality
def cosine_sim(a: torch.Tensor, b: torch.Tensor) -> float:
    """Cosine between two tensors of the same shape, flattened, in fp64."""
    x, y = a.double().flatten(), b.double().flatten()
    return float((x @ y) / (x.norm() * y.norm() + 1e-30))


def polar_factor(x: torch.Tensor) -> torch.Tensor:
    """Exact orthogonal polar factor ``U V^T`` in fp64 (batched over leading dimensions)."""
    U, _, Vh = torch.linalg.svd(x.double(), full_matrices=False)
    return U @ Vh


def sv_stats(y: torch.Tensor) -> dict:
    """Mean / std / min / max of the singular values of ``y`` (an orthogonalised matrix has them all near 1)."""
    sv = torch.linalg.svdvals(y.double())
    return {"sv_mean": float(sv.mean()), "sv_std": float(sv.std()) if sv.numel() > 1 else 0.0, "sv_min": float(sv.min()),
            "sv_max": float(sv.max())}


def orth_quality(y: torch.Tensor, x: torch.Tensor) -> dict:
    """How close ``y`` is to the polar factor of ``x``: cosine, relative Frobenius error, singular-value statistics."""
    p = polar_factor(x)
    yd = y.double()
    out = {"cosine": cosine_sim(yd, p), "rel_fro_err": float((yd - p).norm() / (p.norm() + 1e-30))}
    out.update(sv_stats(yd))
    return out


def batched_polar_cosine(y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Per-matrix cosine between each ``y[i]`` and the polar factor of ``x[i]`` for ``(B, m, n)`` batches (fp64)."""
    p = polar_factor(x)
    yd = y.double()
    num = (yd * p).sum(dim=(-2, -1))
    return num / (yd.norm(dim=(-2, -1)) * p.norm(dim=(-2, -1)) + 1e-30)


# ----------------------------------------------------------------------------------------------- results
def device_name() -> str:
    return torch.cuda.get_device_name(0) if have_cuda() else "cpu"


def measured_peaks() -> dict:
    """The measured copy bandwidth / GEMM throughput of this machine when a ``MEASURED_PEAKS.json`` sits at the
    repository root (keys ``hbm_gbs``, ``bf16_tflops``, ``bf16_tflops_sustained``); empty otherwise."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def _jsonable(obj):
    if isinstance(obj, torch.Tensor):
        return obj.tolist()
    if hasattr(obj, "item") and callable(obj.item):
        return obj.item()
    if hasattr(obj, "tolist"):
        return obj.tolist()
    if isinstance(obj, (set, tuple)):
        return list(obj)
    raise TypeError(f"{type(obj).__name__} is not JSON serialisable")


def save_results(name: str, data: dict, data_dir: str | None = None) -> str:
    d = data_dir or DATA_DIR
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"{name}.json")
    payload = {"experiment": name, "device": device_name(), "torch": torch.__version__,
               "time": time.strftime("%Y-%m-%d %H:%M:%S"), "data": data}
    with open(path, "w") as f:
        json.dump(payload, f, indent=1, default=_jsonable)
    return path


def load_results(name: str, data_dir: str | None = None) -> dict:
    with open(os.path.join(data_dir or DATA_DIR, f"{name}.json")) as f:
        return json.load(f)


# ----------------------------------------------------------------------------------------------- command line
def experiment_main(name: str, run, plot, add_args=None, argv=None, description: str | None = None):
    """The stand-alone entry point every experiment shares (``python -m microbench.experiments.exp_<name>``):
    experiment-specific flags from ``add_args(parser)``, ``--plot-only`` (re-plot the stored JSON without running),
    ``--no-plot``, ``--data-dir`` / ``--out-dir``.  ``run(**flags)`` returns the data dict that is stored and plotted."""
    p = argparse.ArgumentParser(description=description)
    if add_args is not None:
        add_args(p)
    p.add_argument("--plot-only", action="store_true", help="re-plot the stored results, measure nothing")
    p.add_argument("--no-plot", action="store_true", help="measure and store, do not plot")
    p.add_argument("--data-dir", default=DATA_DIR)
    p.add_argument("--out-dir", default=PLOTS_DIR, help="where figures / text tables go")
    args = p.parse_args(argv)
    kwargs = {k: v for k, v in vars(args).items() if k not in ("plot_only", "no_plot", "data_dir", "out_dir")}
    if args.plot_only:
        data = load_results(name, args.data_dir)["data"]
    else:
        data = run(**kwargs)
        print("saved", save_results(name, data, args.data_dir), flush=True)
    if not args.no_plot:
        plot(data, args.out_dir)
    return data
