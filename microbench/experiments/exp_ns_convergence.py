"""Newton-Schulz convergence: worst-tile cosine to the fp64 polar factor and relative Frobenius error against the
iteration count, for tiles 128 / 256 / 512 of a D x D Gaussian matrix (reference: ``exp_ns_convergence.py:148-250``)."""

from __future__ import annotations

import torch

from himuon_b200.optimizers import HiMuon

from ..bench_utils import orth_quality
from ..plot_style import line_chart, text_table


def run(D: int = 1024, tiles=(128, 256, 512), ks=(1, 2, 3, 4, 5, 6, 7, 9), seed: int = 0) -> dict:
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.randn(D, D, generator=torch.Generator().manual_seed(seed)).to(dev)
    out = {"D": D, "ks": list(ks), "tiles": {}}
    for T in tiles:
        tiled, _ = HiMuon._tile(g, (T, T))
        blocks = tiled.reshape(-1, T, T)
        worst_cos, rel = [], []
        for k in ks:
            y = HiMuon.newton_schulz(blocks.to(torch.bfloat16), k).float()
            q = [orth_quality(y[i].cpu(), blocks[i].cpu()) for i in range(min(len(blocks), 16))]
            worst_cos.append(min(v["cosine"] for v in q))
            rel.append(max(v["rel_fro_err"] for v in q))
        out["tiles"][str(T)] = {"worst_cosine": worst_cos, "rel_fro_err": rel}
    return out


def plot(data: dict, out_dir: str):
    rows = [(T, *[f"{c:.3f}" for c in v["worst_cosine"]]) for T, v in data["tiles"].items()]
    print(text_table(("tile \\ K", *data["ks"]), rows))
    line_chart(data["ks"], {f"T={T}": v["worst_cosine"] for T, v in data["tiles"].items()}, "NS iterations",
               "worst-tile cosine", f"D={data['D']}", f"{out_dir}/ns_convergence.png")
