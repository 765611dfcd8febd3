"""Newton-Schulz kernel timing at tile 128: eager PyTorch vs the batched three-GEMM path vs the tile-resident fused
kernel, over the batch sizes of the reference's figure (``exp_ns_kernel_microbench.py:108-183``: B = 32..2048)."""

from __future__ import annotations

import torch

from himuon_b200.ops import ns as ns_ops
from himuon_b200.ops import reference as ref

from ..bench_utils import measure
from ..plot_style import bar_chart, text_table


def _eager(x, steps=5):
    a, b, c = ref.NS_COEFFS
    X = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.transpose(-2, -1)
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return X


def run(T: int = 128, batches=(32, 128, 512, 2048), steps: int = 5) -> dict:
    out = {"T": T, "batches": list(batches), "eager_ms": [], "gemm3_ms": [], "fused_ms": []}
    for B in batches:
        x = torch.randn(B, T, T, device="cuda", dtype=torch.bfloat16)
        ws = ns_ops.NSWorkspace()
        out["eager_ms"].append(measure(lambda: _eager(x, steps))["median_ms"])
        # force the GEMM path by skipping the fused dispatch: pre-normalise and call with normalize=False
        xn = ns_ops._pre_normalized(x)
        out["gemm3_ms"].append(measure(lambda: ns_ops.ns_inplace_cuda(xn.clone(), steps, workspace=ws, normalize=False))["median_ms"])
        out["fused_ms"].append(measure(lambda: ns_ops.ns_inplace_cuda(x.clone(), steps))["median_ms"])
    out["speedup_fused_vs_eager"] = [e / f for e, f in zip(out["eager_ms"], out["fused_ms"])]
    out["speedup_gemm3_vs_eager"] = [e / g for e, g in zip(out["eager_ms"], out["gemm3_ms"])]
    return out


def plot(data: dict, out_dir: str):
    rows = [(b, f"{e:.3f}", f"{g:.3f}", f"{f:.3f}", f"{s:.1f}x") for b, e, g, f, s in
            zip(data["batches"], data["eager_ms"], data["gemm3_ms"], data["fused_ms"], data["speedup_fused_vs_eager"])]
    print(text_table(("B", "eager ms", "3-GEMM ms", "fused ms", "fused speed-up"), rows))
    bar_chart([str(b) for b in data["batches"]], {"eager": data["eager_ms"], "gemm": data["gemm3_ms"], "fused": data["fused_ms"]},
              "ms", f"NS5 at T={data['T']}", f"{out_dir}/ns_kernel_microbench.png", log=True)
