"""One-step associative-memory capacity against the embedding dimension, the frequency exponent and the tile size.

Question: as ``d``, the Zipf exponent ``alpha`` and the tile size vary, does tile-local orthogonalisation (HiMuon)
store as many associations in one step as full-matrix orthogonalisation (Muon), or does it fall back towards plain
gradient descent?  A tile-local map cannot amplify a singular direction that spans several tiles coherently.

Setup (the reference's, ``microbench/experiments/exp_capacity_scaling.py:57-127``): one update from ``W = 0`` on a
linear associative memory with ``N`` key/value pairs of power-law frequency, the gradient of a minibatch of
``batch_scale * d`` draws (exact softmax form at ``W = 0``), for ``d`` in {256, 512, 1024}, ``alpha`` in
{1.25, 1.5, 1.75}, several seeds.  The metric is the number of items whose own key scores highest after the step;
it does not depend on the (positive) step size, so ``eta = 1``.  Stateless, operator only; runs on CPU or GPU.

    python -m microbench.experiments.exp_capacity_scaling [--ds 256 512 1024] [--alphas 1.25 1.5 1.75] [--num-items 100000]
    python -m microbench.experiments.exp_capacity_scaling --plot-only
"""

from __future__ import annotations

import os
from collections import defaultdict

from .. import assoc_mem as am
from ..bench_utils import DATA_DIR, default_device, experiment_main, have_cuda, mean_std
from ..plot_style import bar_chart, text_table, write_text

NAME = "capacity_scaling"


def methods(tiles):
    return [("Muon", "muon", None)] + [(f"HiMuon-{t}", "himuon", t) for t in sorted(tiles, reverse=True)] + [("SGD", "sgd", None)]


def run(ds=(256, 512, 1024), alphas=(1.25, 1.5, 1.75), batch_scale: float = 10.0, num_items: int = 100000, seeds=(0, 1, 2),
        tiles=(128, 256, 512), ns_steps: int = 5, ns_precision: str = "fp32", jsonl: bool = True) -> dict:
    dev = default_device()
    meths = methods(tiles)
    records, log = [], []
    for d in ds:
        for alpha in alphas:
            for seed in seeds:
                am.assert_memory_budget(160.0 if dev.type == "cuda" else 32.0, d=d, num_items=num_items)
                problem = am.sample_problem(d, num_items, "power_law", alpha, seed, device=str(dev))
                bs = max(1, int(round(batch_scale * d)))
                grad, meta = am.build_gradient(problem, "true_minibatch", batch_size=bs, seed=seed + bs)
                line = []
                for label, opt, tile in meths:
                    update = am.apply_one_step(grad, opt, 1.0, ns_steps, tile if tile is not None else 256, ns_precision)
                    ok, _ = am.evaluate_recovery(problem, update)
                    rec = {"d": d, "alpha": alpha, "seed": seed, "label": label, "tile_size": tile,
                           "recovered_count": int(ok.sum()), "effective_support": meta["effective_support"]}
                    records.append(rec)
                    log.append(am.make_result_record(problem, opt, 1.0, {"recovered_count": rec["recovered_count"],
                                                                         "recovered_fraction": rec["recovered_count"] / num_items,
                                                                         "recovered_probability_mass": float(problem.p.cpu()[ok].sum())},
                                                     tile_size=tile, batch_size=bs, ns_precision=ns_precision))
                    line.append(f"{label}={rec['recovered_count']}")
                print(f"d={d:5d} alpha={alpha:.2f} seed={seed} support={meta['effective_support']} | " + " ".join(line), flush=True)
    if jsonl:
        am.write_jsonl(os.path.join(DATA_DIR, NAME + ".jsonl"), log, append=False)
    return {"config": {"ds": list(ds), "alphas": list(alphas), "batch_scale": batch_scale, "num_items": num_items,
                       "seeds": list(seeds), "tiles": list(tiles), "ns_steps": ns_steps, "ns_precision": ns_precision,
                       "gradient_mode": "true_minibatch", "device": str(dev)},
            "records": records, "summary": am.summarize_records(log)}


def aggregate(records):
    agg = defaultdict(list)
    for r in records:
        agg[(r["alpha"], r["d"], r["label"])].append(r["recovered_count"])
    return {k: mean_std(v) for k, v in agg.items()}


def plot(data: dict, out_dir: str):
    cfg = data["config"]
    agg = aggregate(data["records"])
    labels = [m[0] for m in methods(cfg["tiles"])]
    rows = []
    for alpha in cfg["alphas"]:
        series = {lab: [agg[(alpha, d, lab)][0] for d in cfg["ds"]] for lab in labels}
        errs = {lab: ([agg[(alpha, d, lab)][0] - agg[(alpha, d, lab)][1] for d in cfg["ds"]],
                      [agg[(alpha, d, lab)][0] + agg[(alpha, d, lab)][1] for d in cfg["ds"]]) for lab in labels}
        bar_chart([f"d={d}" for d in cfg["ds"]], series, "one-step recovered items",
                  f"alpha = {alpha:g}, N = {cfg['num_items']}, B/d = {cfg['batch_scale']:g}", out_dir,
                  f"{NAME}_alpha{alpha:g}", log=True, errors=errs)
        for d in cfg["ds"]:
            muon = agg[(alpha, d, "Muon")][0]
            for lab in labels:
                m, s = agg[(alpha, d, lab)]
                rows.append((alpha, d, lab, m, s, m / muon if muon else None))
    txt = text_table(("alpha", "d", "method", "recovered (mean)", "std", "fraction of Muon"), rows)
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)


def add_args(p):
    gpu = have_cuda()
    p.add_argument("--ds", type=int, nargs="+", default=[256, 512, 1024] if gpu else [128, 256])
    p.add_argument("--alphas", type=float, nargs="+", default=[1.25, 1.5, 1.75])
    p.add_argument("--batch-scale", type=float, default=10.0, help="minibatch size / d")
    p.add_argument("--num-items", type=int, default=100000 if gpu else 8192)
    p.add_argument("--seeds", type=int, nargs="+", default=[0, 1, 2])
    p.add_argument("--tiles", type=int, nargs="+", default=[128, 256, 512] if gpu else [32, 64, 128])
    p.add_argument("--ns-steps", type=int, default=5)
    p.add_argument("--ns-precision", default="fp32", choices=list(am.NS_PRECISIONS))
    p.add_argument("--no-jsonl", dest="jsonl", action="store_false", help="do not write the per-run jsonl log")


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
