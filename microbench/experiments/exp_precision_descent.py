"""Multi-step descent on the associative-memory loss with the update operator evaluated at several precisions
(reference: ``exp_precision_descent.py``): recovered items per step for Muon and HiMuon at fp32 / bf16 / simulated fp8."""

from __future__ import annotations

import torch

from .. import assoc_mem as am
from ..plot_style import text_table


def run(d: int = 128, n: int = 512, alpha: float = 1.5, steps: int = 8, lr: float = 0.5, tiles=(None, 64),
        precisions=("fp32", "bf16", "fp8e4m3_sim"), seed: int = 0) -> dict:
    keys, vals, freqs, _ = am.zipf_problem(d, n, alpha, seed=seed)
    out = {"steps": steps, "curves": {}}
    for t in tiles:
        for p in precisions:
            W = torch.zeros(d, d)
            curve = []
            for _ in range(steps):
                resid = vals - keys @ W.t()                         # gradient of 0.5 * sum_i f_i ||v_i - W k_i||^2
                grad = (resid * freqs[:, None]).t() @ keys
                W = W + lr * am.himuon_operator(grad, t, 5, p)
                curve.append(am.recovered_items(W, keys, vals))
            out["curves"][f"{'muon' if t is None else f'himuon-{t}'}/{p}"] = curve
    return out


def plot(data: dict, out_dir: str):
    print(text_table(("method/precision", *range(1, data["steps"] + 1)), [(k, *v) for k, v in data["curves"].items()]))
