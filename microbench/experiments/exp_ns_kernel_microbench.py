"""Newton-Schulz kernel comparison at tile 128: which implementation of five quintic iterations is fastest on a batch
of (B, T, T) bf16 tiles.

Arms (the reference's figure has eager / torch.compile / three Triton kernels / fused ``ns5_smem``,
``microbench/experiments/exp_ns_kernel_microbench.py:58-183``):

* ``eager``    - plain PyTorch ``bmm`` loop (library GEMMs, one launch per product);
* ``compile``  - the same loop under ``torch.compile`` (optional, ``--with-compile``; a baseline only);
* ``3-kernel`` - the three public product kernels per iteration, ``XXT`` -> ``ba_plus_cAA`` -> ``fused_bmm_add``
  (tcgen05 GEMM launches with fused epilogues, the symmetric products computing one triangle), 15 launches + a
  normalisation;
* ``fused``    - ``ns5_smem``: one launch, the whole tile resident in shared memory, accumulators in tensor memory.

Per batch size: median / quartile milliseconds (cold L2), achieved TFLOP/s and fraction of the measured GEMM peak of
the machine, peak extra memory, and the cosine of every arm against an fp32 PyTorch iteration on the same input.
Meant for a GPU (without one every arm falls back to PyTorch ops and only the plumbing is exercised).

    python -m microbench.experiments.exp_ns_kernel_microbench [--batches 32 128 512 2048] [--T 128] [--with-compile]
    python -m microbench.experiments.exp_ns_kernel_microbench --plot-only
"""

from __future__ import annotations

import torch

from himuon_b200 import kernels
from himuon_b200.ops import reference as ref

from ..bench_utils import cosine_sim, default_device, experiment_main, measure, measure_memory, measured_peaks
from ..plot_style import bar_chart, text_table, write_text

NAME = "ns_kernel_microbench"
A, B_, C = ref.NS_COEFFS
EPS = 1e-7


def _iterate(X, steps):
    for _ in range(steps):
        G = X @ X.transpose(-2, -1)
        P = B_ * G + C * (G @ G)
        X = A * X + P @ X
    return X


def ns_eager(x: torch.Tensor, steps: int = 5) -> torch.Tensor:
    return _iterate(x / (x.norm(dim=(-2, -1), keepdim=True) + EPS), steps)


def ns_reference_fp32(x: torch.Tensor, steps: int = 5) -> torch.Tensor:
    return ns_eager(x.float(), steps)


def make_three_kernel(Bn: int, T: int, device):
    """The public product kernels with preallocated outputs (what a caller of the reference's kernel package writes)."""
    gram = torch.empty(Bn, T, T, device=device, dtype=torch.bfloat16)
    poly = torch.empty_like(gram)

    def run(x: torch.Tensor, steps: int = 5) -> torch.Tensor:
        X = x / (x.norm(dim=(-2, -1), keepdim=True) + EPS)
        for _ in range(steps):
            kernels.XXT(X, gram)
            kernels.ba_plus_cAA(gram, C, B_, poly)          # C * (G G^T) + B_ * G
            X = kernels.fused_bmm_add(poly, X, A)
        return X

    return run


def ns_flops(Bn: int, m: int, n: int, steps: int = 5) -> float:
    lo, hi = min(m, n), max(m, n)
    return float(Bn) * steps * (2.0 * lo * lo * hi * 2 + 2.0 * lo ** 3)


def run(batches=(32, 128, 512, 2048), T: int = 128, steps: int = 5, warmup: int = 10, repeats: int = 50,
        with_compile: bool = False, seed: int = 42) -> dict:
    dev = default_device()
    if dev.type != "cuda":
        print("no CUDA device: every arm runs its PyTorch path, the times say nothing about the kernels", flush=True)
    peak = measured_peaks().get("bf16_tflops")
    compiled = torch.compile(ns_eager) if with_compile else None
    rows = []
    for Bn in batches:
        x = torch.randn(Bn, T, T, device=dev, dtype=torch.bfloat16, generator=torch.Generator(dev.type).manual_seed(seed))
        want = ns_reference_fp32(x, steps)
        arms = {"eager": lambda: ns_eager(x, steps), "3-kernel": None, "fused": lambda: kernels.ns5_smem(x)}
        three = make_three_kernel(Bn, T, dev)
        arms["3-kernel"] = lambda: three(x, steps)
        if compiled is not None:
            arms["compile"] = lambda: compiled(x, steps)
        row = {"B": Bn, "T": T, "flops": ns_flops(Bn, T, T, steps), "arms": {}}
        for name, fn in arms.items():
            t = measure(fn, warmup=warmup, iters=repeats)
            t["peak_bytes"] = measure_memory(fn)
            t["cosine_vs_fp32"] = cosine_sim(fn(), want)
            t["tflops"] = row["flops"] / t["median_ms"] / 1e9
            t["fraction_of_measured_peak"] = t["tflops"] / peak if peak else None
            row["arms"][name] = t
        for name in row["arms"]:
            row["arms"][name]["speedup_vs_eager"] = row["arms"]["eager"]["median_ms"] / row["arms"][name]["median_ms"]
        rows.append(row)
        print(f"B={Bn}: " + "  ".join(f"{n} {a['median_ms']:.3f} ms" for n, a in row["arms"].items()), flush=True)
    return {"T": T, "steps": steps, "batches": list(batches), "peak_tflops": peak, "rows": rows}


def plot(data: dict, out_dir: str):
    arms = list(data["rows"][0]["arms"])
    labels = [f"B={r['B']}" for r in data["rows"]]
    bar_chart(labels, {a: [r["arms"][a]["median_ms"] for r in data["rows"]] for a in arms}, "ms (median, cold L2)",
              f"NS5 at T={data['T']}, bf16", out_dir, NAME, log=True,
              errors={a: ([r["arms"][a]["p25_ms"] for r in data["rows"]], [r["arms"][a]["p75_ms"] for r in data["rows"]])
                      for a in arms})
    bar_chart(labels, {a: [r["arms"][a]["speedup_vs_eager"] for r in data["rows"]] for a in arms if a != "eager"},
              "speed-up over eager", f"NS5 at T={data['T']}", out_dir, NAME + "_speedup", value_fmt="{:.1f}x", baseline=1.0)
    rows = []
    for r in data["rows"]:
        for a in arms:
            v = r["arms"][a]
            rows.append((r["B"], a, v["median_ms"], v["p25_ms"], v["p75_ms"], v["tflops"], v["fraction_of_measured_peak"],
                         v["peak_bytes"] / 2 ** 20, v["cosine_vs_fp32"], v["speedup_vs_eager"]))
    txt = text_table(("B", "arm", "median ms", "p25", "p75", "TFLOP/s", "of measured peak", "extra MiB", "cos vs fp32",
                      "x eager"), rows)
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)


def add_args(p):
    p.add_argument("--batches", type=int, nargs="+", default=[32, 128, 512, 2048])
    p.add_argument("--T", type=int, default=128, help="tile side (the fused kernel's domain is rows <= 128)")
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--repeats", type=int, default=50)
    p.add_argument("--with-compile", action="store_true", help="add a torch.compile arm (baseline only)")


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
