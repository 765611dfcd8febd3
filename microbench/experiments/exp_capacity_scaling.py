"""Capacity scaling: items recovered after one step by SGD, Muon and HiMuon at several tile sizes as the number of
stored associations grows (reference: ``exp_capacity_scaling.py``)."""

from __future__ import annotations

import torch

from .. import assoc_mem as am
from ..plot_style import line_chart, text_table


def run(d: int = 256, n_list=(256, 512, 1024, 2048), alpha: float = 1.5, tiles=(None, 128, 64, 32), seed: int = 0) -> dict:
    out = {"d": d, "n": list(n_list), "series": {}}
    for n in n_list:
        keys, vals, _, grad = am.zipf_problem(d, n, alpha, seed=seed)
        out["series"].setdefault("sgd", []).append(am.recovered_items(grad, keys, vals))
        for t in tiles:
            name = "muon" if t is None else f"himuon-{t}"
            out["series"].setdefault(name, []).append(am.recovered_items(am.himuon_operator(grad, t), keys, vals))
    return out


def plot(data: dict, out_dir: str):
    print(text_table(("method", *data["n"]), [(k, *v) for k, v in data["series"].items()]))
    line_chart(data["n"], data["series"], "stored items", "recovered", f"d={data['d']}", f"{out_dir}/capacity_scaling.png", logx=True)
