"""Rectangular tiles: fused tile-resident kernel vs the three-GEMM path at a constant 2^21 elements per call
(reference: ``exp_ns5_rect_bench.py:83-236``).  Shapes outside the fused kernel's domain report ``None``."""

from __future__ import annotations

import torch

from himuon_b200.ops import ns as ns_ops

from ..bench_utils import measure
from ..plot_style import text_table

SHAPES = [(16, 64), (16, 128), (16, 256), (32, 64), (32, 128), (32, 256), (64, 64), (64, 128), (64, 256), (128, 128), (128, 256)]


def run(total_elems: int = 1 << 21) -> dict:
    rows = []
    for m, n in SHAPES:
        B = max(1, total_elems // (m * n))
        x = torch.randn(B, m, n, device="cuda", dtype=torch.bfloat16)
        ws = ns_ops.NSWorkspace()
        xn = ns_ops._pre_normalized(x)
        gemm = measure(lambda: ns_ops.ns_inplace_cuda(xn.clone(), 5, workspace=ws, normalize=False))["median_ms"] if m % 8 == 0 else None
        fused = measure(lambda: ns_ops.ns_inplace_cuda(x.clone(), 5))["median_ms"] if ns_ops.fused_supported(m, n) else None
        rows.append({"m": m, "n": n, "B": B, "gemm3_ms": gemm, "fused_ms": fused,
                     "speedup": (gemm / fused) if gemm and fused else None})
    return {"total_elems": total_elems, "rows": rows}


def plot(data: dict, out_dir: str):
    print(text_table(("M", "N", "B", "3-GEMM ms", "fused ms", "speed-up"),
                     [(r["m"], r["n"], r["B"], r["gemm3_ms"] and f"{r['gemm3_ms']:.3f}", r["fused_ms"] and f"{r['fused_ms']:.3f}",
                       r["speedup"] and f"{r['speedup']:.2f}x") for r in data["rows"]]))
