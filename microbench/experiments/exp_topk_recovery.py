"""Top-k recovery rate after one step for SGD / Muon / HiMuon tiles (reference: ``exp_topk_recovery.py``)."""

from __future__ import annotations

from .. import assoc_mem as am
from ..plot_style import text_table


def run(d: int = 256, n: int = 1024, alpha: float = 1.5, tiles=(None, 128, 64, 32), ks=(1, 5, 10), seed: int = 0) -> dict:
    keys, vals, _, grad = am.zipf_problem(d, n, alpha, seed=seed)
    rows = {"sgd": am.topk_recovery(grad, keys, vals, ks)}
    for t in tiles:
        rows["muon" if t is None else f"himuon-{t}"] = am.topk_recovery(am.himuon_operator(grad, t), keys, vals, ks)
    return {"d": d, "n": n, "ks": list(ks), "rows": {k: {str(kk): vv for kk, vv in v.items()} for k, v in rows.items()}}


def plot(data: dict, out_dir: str):
    print(text_table(("method", *[f"top-{k}" for k in data["ks"]]),
                     [(m, *[f"{v[str(k)]:.3f}" for k in data["ks"]]) for m, v in data["rows"].items()]))
