"""One-step recovered items and operator error ``delta_F`` at fp64 / fp32 / bf16 / simulated fp8 for Muon and HiMuon
tiles, mean +- std over seeds (reference table: ``microbench/plots/precision_recovery_table.tex``, d=1024, N=4096,
alpha=1.5, B/d=10, K=5, 5 seeds)."""

from __future__ import annotations

import statistics

from .. import assoc_mem as am
from ..plot_style import text_table


def run(d: int = 256, n: int = 1024, alpha: float = 1.5, batch_over_d: int = 10, steps: int = 5, tiles=(None, 128, 64, 32),
        seeds=(0, 1, 2, 3, 4)) -> dict:
    rows = {}
    for t in tiles:
        name = "muon" if t is None else f"himuon-{t}"
        rec = {p: [] for p in am.PRECISIONS}
        err = {p: [] for p in ("bf16", "fp8e4m3_sim")}
        for s in seeds:
            keys, vals, _, grad = am.zipf_problem(d, n, alpha, batch=batch_over_d * d, seed=s)
            for p in am.PRECISIONS:
                rec[p].append(am.recovered_items(am.himuon_operator(grad, t, steps, p), keys, vals))
            for p in err:
                err[p].append(am.relative_operator_error(grad, t, steps, p))
        rows[name] = {"recovered": {p: [statistics.fmean(v), statistics.pstdev(v)] for p, v in rec.items()},
                      "delta_F": {p: statistics.fmean(v) for p, v in err.items()}}
    return {"d": d, "n": n, "rows": rows}


def plot(data: dict, out_dir: str):
    print(text_table(("method", *am.PRECISIONS, "dF bf16", "dF fp8"),
                     [(m, *[f"{v['recovered'][p][0]:.1f}+-{v['recovered'][p][1]:.1f}" for p in am.PRECISIONS],
                       f"{v['delta_F']['bf16']:.3f}", f"{v['delta_F']['fp8e4m3_sim']:.3f}") for m, v in data["rows"].items()]))
