"""Rectangular tiles: the tile-resident fused Newton-Schulz kernel against the three-GEMM iteration over a grid of
(M, N) tile shapes, at a constant amount of data per call.

Shapes are all (M, N) with M <= N drawn from ``DIMS`` whose working set ``M N + 2 M^2`` bf16 elements (the tile and the
two M x M intermediates) fits a shared-memory budget - the enumeration of the reference's sweep
(``microbench/experiments/exp_ns5_rect_bench.py:93-107``; its budget of 49152 elements is the 128 x 128 case; the
default here is the 227 KB an sm_100a CTA can hold).  The batch is ``total_elements / (M N)``, so every call moves the
same number of bytes and times compare as throughput.

Per shape the experiment times

* ``fused``  - ``ns5_smem`` (one launch; shapes outside the kernel's domain take the three-GEMM path inside the same
  entry point, and the row says so),
* ``gemm3``  - the batched three-GEMM iteration forced (pre-normalised input, 15 tcgen05 GEMM launches),
* ``eager``  - optional (``--with-eager``) PyTorch ``bmm`` loop,

and checks each result against an fp32 PyTorch iteration of the same input (cosine).  The reference's second axis, the
launch strategy (one CTA per tile or a persistent grid), does not exist here: the sm_100a kernel is always persistent.

    python -m microbench.experiments.exp_ns5_rect_bench [--total-elements 2097152] [--dims 16 32 64 128 256]
    python -m microbench.experiments.exp_ns5_rect_bench --plot-only
"""

from __future__ import annotations

import torch

from himuon_b200 import kernels
from himuon_b200.ops import ns as ns_ops

from ..bench_utils import cosine_sim, default_device, experiment_main, measure
from ..plot_style import heatmap, text_table, write_text
from .exp_ns_kernel_microbench import ns_eager, ns_flops, ns_reference_fp32

NAME = "ns5_rect_bench"
DIMS = (16, 32, 64, 128, 256, 512, 1024, 2048)
SMEM_BUDGET_ELEMS = 227 * 1024 // 2


def enumerate_shapes(dims=DIMS, budget: int = SMEM_BUDGET_ELEMS):
    return [(m, n) for m in dims for n in dims if m <= n and m * n + 2 * m * m <= budget]


def _gemm3(x: torch.Tensor, ws) -> torch.Tensor:
    if not x.is_cuda:
        return kernels.ns5_smem(x)
    return ns_ops.ns_inplace_cuda(ns_ops._pre_normalized(x), 5, workspace=ws, normalize=False)


def run(total_elements: int = 1 << 21, dims=DIMS, budget: int = SMEM_BUDGET_ELEMS, warmup: int = 10, repeats: int = 50,
        with_eager: bool = False, seed: int = 42) -> dict:
    dev = default_device()
    rows = []
    ws = ns_ops.NSWorkspace() if dev.type == "cuda" else None
    for m, n in enumerate_shapes(dims, budget):
        Bn = max(1, total_elements // (m * n))
        x = torch.randn(Bn, m, n, device=dev, dtype=torch.bfloat16, generator=torch.Generator(dev.type).manual_seed(seed))
        want = ns_reference_fp32(x)
        row = {"M": m, "N": n, "B": Bn, "fused_kernel": bool(dev.type == "cuda" and ns_ops.fused_supported(m, n)),
               "flops": ns_flops(Bn, m, n)}
        fused = measure(lambda: kernels.ns5_smem(x), warmup=warmup, iters=repeats)
        row["fused_ms"], row["fused_p25"], row["fused_p75"] = fused["median_ms"], fused["p25_ms"], fused["p75_ms"]
        row["fused_cos"] = cosine_sim(kernels.ns5_smem(x), want)
        if m % 8 == 0 and n % 8 == 0:
            g3 = measure(lambda: _gemm3(x, ws), warmup=warmup, iters=repeats)
            row["gemm3_ms"] = g3["median_ms"]
            row["gemm3_cos"] = cosine_sim(_gemm3(x, ws), want)
            row["speedup_vs_gemm3"] = row["gemm3_ms"] / row["fused_ms"]
        else:
            row["gemm3_ms"] = row["gemm3_cos"] = row["speedup_vs_gemm3"] = None
        if with_eager:
            row["eager_ms"] = measure(lambda: ns_eager(x), warmup=max(1, warmup // 2), iters=max(3, repeats // 2))["median_ms"]
            row["speedup_vs_eager"] = row["eager_ms"] / row["fused_ms"]
        row["gelem_per_s"] = Bn * m * n / row["fused_ms"] / 1e6
        row["tflops"] = row["flops"] / row["fused_ms"] / 1e9
        rows.append(row)
        print(f"({m:4d},{n:4d}) B={Bn:6d} fused {row['fused_ms']:.3f} ms"
              + (f"  gemm3 {row['gemm3_ms']:.3f} ms  x{row['speedup_vs_gemm3']:.2f}" if row["gemm3_ms"] else "")
              + ("" if row["fused_kernel"] else "  [three-GEMM path]"), flush=True)
    return {"total_elements": total_elements, "budget_elems": budget, "device": str(dev), "rows": rows}


def _matrix(rows, key):
    ms = sorted({r["M"] for r in rows})
    ns_ = sorted({r["N"] for r in rows})
    cell = {(r["M"], r["N"]): r.get(key) for r in rows}
    return ms, ns_, [[cell.get((m, n)) for n in ns_] for m in ms]


def plot(data: dict, out_dir: str):
    rows = data["rows"]
    ms, ns_, sp = _matrix(rows, "speedup_vs_gemm3")
    heatmap([f"M={m}" for m in ms], [f"N={n}" for n in ns_], sp, "ns5_smem speed-up over the three-GEMM iteration",
            out_dir, NAME, fmt="{:.2f}", center=1.0, cbar_label="x")
    _, _, thr = _matrix(rows, "gelem_per_s")
    heatmap([f"M={m}" for m in ms], [f"N={n}" for n in ns_], thr, "ns5_smem throughput (G elements / s)", out_dir,
            NAME + "_throughput", fmt="{:.1f}", cbar_label="Gelem/s")
    txt = text_table(("M", "N", "B", "fused kernel", "fused ms", "p25", "p75", "gemm3 ms", "speed-up", "TFLOP/s", "cos fused",
                      "cos gemm3"),
                     [(r["M"], r["N"], r["B"], "yes" if r["fused_kernel"] else "no", r["fused_ms"], r["fused_p25"], r["fused_p75"],
                       r["gemm3_ms"], r["speedup_vs_gemm3"], r["tflops"], r["fused_cos"], r["gemm3_cos"]) for r in rows])
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)


def add_args(p):
    p.add_argument("--total-elements", type=int, default=1 << 21, help="elements per call (batch = total / (M N))")
    p.add_argument("--dims", type=int, nargs="+", default=list(DIMS))
    p.add_argument("--budget", type=int, default=SMEM_BUDGET_ELEMS, help="admit shapes with M N + 2 M^2 <= budget elements")
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--repeats", type=int, default=50)
    p.add_argument("--with-eager", action="store_true")


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
