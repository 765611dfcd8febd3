"""Which items does one step recover: only the frequent head, or the tail too?

Recovery is scored on the unique sampled support ``S`` of the minibatch (items that were drawn at least once), sorted
by falling population frequency, as the recovery rate of the ``k`` most frequent sampled items for every ``k``.
Restricting to ``S`` separates the quality of the update map from finite-sample coverage: an item that was never drawn
has zero gradient and cannot be recovered in one step by any method.  The curve runs up to the common cut-off
``k_max = min |S|`` over the seeds, and the second figure is the gap between Muon's curve and each HiMuon tile's.
(Reference: ``microbench/experiments/exp_topk_recovery.py:58-141``: d = 1024, alpha = 1.5, B/d = 10, N = 1e5, 3 seeds,
tiles 128 / 256 / 512.)  Stateless, operator only; the recovery does not depend on the step size.

    python -m microbench.experiments.exp_topk_recovery [--d 1024] [--alpha 1.5] [--num-items 100000] [--tiles 128 256 512]
    python -m microbench.experiments.exp_topk_recovery --plot-only
"""

from __future__ import annotations

import torch

from .. import assoc_mem as am
from ..bench_utils import default_device, experiment_main, have_cuda
from ..plot_style import line_chart, text_table, write_text

NAME = "topk_recovery"


def methods(tiles):
    return [("SGD", "sgd", None), ("Muon", "muon", None)] + [(f"HiMuon-{t}", "himuon", t) for t in sorted(tiles, reverse=True)]


def run(d: int = 1024, alpha: float = 1.5, seeds=(0, 1, 2), batch_scale: float = 10.0, num_items: int = 100000,
        tiles=(128, 256, 512), ns_steps: int = 5, ns_precision: str = "fp32") -> dict:
    dev = default_device()
    meths = methods(tiles)
    curves = {lab: [] for lab, _, _ in meths}
    support_sizes = {}
    for seed in seeds:
        problem = am.sample_problem(d, num_items, "power_law", alpha, seed, device=str(dev))
        bs = max(1, int(round(batch_scale * d)))
        gseed = seed + bs
        grad, _ = am.build_gradient(problem, "true_minibatch", batch_size=bs, seed=gseed)
        freqs = am.sample_empirical_frequencies(problem.p, bs, gseed)          # the draw build_gradient used
        support = torch.nonzero(freqs > 0).squeeze(1).cpu()
        p_cpu = problem.p.float().cpu()
        support = support[torch.argsort(p_cpu[support], descending=True)]
        support_sizes[str(seed)] = int(support.numel())
        for label, opt, tile in meths:
            update = am.apply_one_step(grad, opt, 1.0, ns_steps, tile if tile is not None else 256, ns_precision)
            ok, _ = am.evaluate_recovery(problem, update)
            hits = ok.float()[support]
            curves[label].append(torch.cumsum(hits, 0) / torch.arange(1, hits.numel() + 1))
        print(f"seed={seed} |S|={support_sizes[str(seed)]} " +
              " ".join(f"{lab}={float(c[-1][-1]):.3f}" for lab, c in curves.items()), flush=True)
    k_max = min(support_sizes.values())
    series = {}
    for label, _, tile in meths:
        stacked = torch.stack([c[:k_max] for c in curves[label]])
        series[label] = {"tile_size": tile, "mean_recovery_rate": stacked.mean(0).tolist(),
                         "std_recovery_rate": stacked.std(0, unbiased=False).tolist()}
    return {"config": {"d": d, "alpha": alpha, "seeds": list(seeds), "batch_scale": batch_scale, "num_items": num_items,
                       "tiles": list(tiles), "ns_steps": ns_steps, "ns_precision": ns_precision, "k_max": k_max,
                       "support_sizes": support_sizes, "mean_support_size": sum(support_sizes.values()) / len(support_sizes),
                       "device": str(dev)},
            "series": series}


def _sample_ks(k_max: int, n: int = 24):
    ks = sorted({max(1, int(round(k_max ** (i / (n - 1))))) for i in range(n)})
    return [k for k in ks if k <= k_max]


def plot(data: dict, out_dir: str, gap_min_k: int = 50):
    cfg, series = data["config"], data["series"]
    ks = _sample_ks(cfg["k_max"])
    pick = lambda xs: [xs[k - 1] for k in ks]
    title = f"d={cfg['d']}, alpha={cfg['alpha']:g}, N={cfg['num_items']}, |S|~{cfg['mean_support_size']:.0f}"
    line_chart(ks, {lab: pick(s["mean_recovery_rate"]) for lab, s in series.items()}, "k (most frequent sampled items)",
               "recovery rate of the top k", title, out_dir, NAME, logx=True,
               bands={lab: ([m - e for m, e in zip(pick(s["mean_recovery_rate"]), pick(s["std_recovery_rate"]))],
                            [m + e for m, e in zip(pick(s["mean_recovery_rate"]), pick(s["std_recovery_rate"]))])
                      for lab, s in series.items()})
    gap_ks = [k for k in ks if k >= min(gap_min_k, cfg["k_max"])]
    muon = series["Muon"]["mean_recovery_rate"]
    gaps = {lab: [muon[k - 1] - s["mean_recovery_rate"][k - 1] for k in gap_ks] for lab, s in series.items()
            if lab.startswith("HiMuon")}
    if gap_ks and gaps:
        line_chart(gap_ks, gaps, "k", "Muon recovery rate - HiMuon recovery rate", "gap to Muon", out_dir, NAME + "_gap",
                   logx=True, hline=0.0)
    marks = [k for k in (10, 50, 100, 500, 1000, 5000) if k <= cfg["k_max"]] + [cfg["k_max"]]
    txt = text_table(("method", *[f"top-{k}" for k in marks]),
                     [(lab, *[s["mean_recovery_rate"][k - 1] for k in marks]) for lab, s in series.items()])
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)


def add_args(p):
    gpu = have_cuda()
    p.add_argument("--d", type=int, default=1024 if gpu else 256)
    p.add_argument("--alpha", type=float, default=1.5)
    p.add_argument("--seeds", type=int, nargs="+", default=[0, 1, 2])
    p.add_argument("--batch-scale", type=float, default=10.0)
    p.add_argument("--num-items", type=int, default=100000 if gpu else 8192)
    p.add_argument("--tiles", type=int, nargs="+", default=[128, 256, 512] if gpu else [32, 64, 128])
    p.add_argument("--ns-steps", type=int, default=5)
    p.add_argument("--ns-precision", default="fp32", choices=list(am.NS_PRECISIONS))


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
