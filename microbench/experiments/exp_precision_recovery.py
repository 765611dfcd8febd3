"""Does low-precision Newton-Schulz cost recovered associations?

For Muon, HiMuon at several tiles and SGD, the one-step update of the associative-memory problem is computed with the
iteration in fp64 (the reference), fp32, bf16, simulated fp8-e4m3 (operands rounded through ``float8_e4m3fn`` under a
per-tensor scale) and - on a GPU with fp8 tensor cores - native fp8-e4m3 products (``torch._scaled_mm``).  Per method
and precision the experiment reports the number of recovered items (mean +- std over the seeds) and the operator gap
``delta_F = ||U_p - U_fp64||_F / ||U_fp64||_F`` of the low-precision update to the fp64 one.  It writes a figure, a
text table and the LaTeX table of the reference (``microbench/plots/precision_recovery_table.tex``; setup of
``microbench/experiments/exp_precision_recovery.py:84-160``: d = 1024, N = 4096, alpha = 1.5, B/d = 10, K = 5, 5 seeds).

    python -m microbench.experiments.exp_precision_recovery [--d 1024] [--num-items 4096] [--precisions fp64_ref fp32 bf16 ...]
    python -m microbench.experiments.exp_precision_recovery --plot-only
"""

from __future__ import annotations

from collections import defaultdict

import torch

from .. import assoc_mem as am
from ..bench_utils import default_device, experiment_main, have_cuda, mean_std
from ..plot_style import bar_chart, latex_table, text_table, write_text

NAME = "precision_recovery"
PREC_LABEL = {"fp64_ref": "fp64", "fp32": "fp32", "bf16": "bf16", "fp8e4m3_sim": "fp8 (sim.)", "fp8e4m3_native": "fp8e4m3"}


def methods(tiles):
    return [("Muon", "muon", None)] + [(f"HiMuon-{t}", "himuon", t) for t in sorted(tiles, reverse=True)] + [("SGD", "sgd", None)]


def native_fp8_available() -> bool:
    """True when a small fp8-e4m3 product actually runs on this machine (GPU with fp8 tensor cores and a PyTorch that
    exposes the scaled matmul)."""
    if not have_cuda() or not hasattr(torch, "_scaled_mm") or torch.cuda.get_device_capability() < (8, 9):
        return False
    try:
        x = torch.randn(32, 32, device="cuda")
        return bool(torch.isfinite(am.fp8_matmul(x, x)).all())
    except Exception:
        return False


def default_precisions():
    return list(am.PRECISIONS) + (["fp8e4m3_native"] if native_fp8_available() else [])


def run(d: int = 1024, alpha: float = 1.5, seeds=(0, 1, 2, 3, 4), batch_scale: float = 10.0, num_items: int = 4096,
        precisions=None, tiles=(128, 256, 512), ns_steps: int = 5, problem_dtype: str = "float32") -> dict:
    dev = default_device()
    precisions = list(precisions or default_precisions())
    if "fp8e4m3_native" in precisions and not native_fp8_available():
        print("fp8e4m3_native needs a GPU with fp8 tensor cores: dropped", flush=True)
        precisions.remove("fp8e4m3_native")
    dtype = {"float32": torch.float32, "float64": torch.float64}[problem_dtype]
    records = []
    for seed in seeds:
        problem = am.sample_problem(d, num_items, "power_law", alpha, seed, device=str(dev), dtype=dtype)
        bs = max(1, int(round(batch_scale * d)))
        grad, _ = am.build_gradient(problem, "true_minibatch", batch_size=bs, seed=seed + bs)
        for label, opt, tile in methods(tiles):
            t = tile if tile is not None else 256
            ref_update = am.apply_one_step(grad, opt, 1.0, ns_steps, t, "fp64_ref")
            for prec in precisions:
                update = ref_update if prec == "fp64_ref" else am.apply_one_step(grad, opt, 1.0, ns_steps, t, prec)
                ok, _ = am.evaluate_recovery(problem, update)
                gap = am.operator_gap_metrics(ref_update, update)
                records.append({"seed": seed, "label": label, "tile_size": tile, "ns_precision": prec,
                                "recovered_count": int(ok.sum()), "rel_fro_gap_to_fp64": gap["operator_relative_fro_gap"],
                                "cosine_to_fp64": gap["operator_cosine_similarity"]})
        print(f"seed={seed}: " + " ".join(f"{r['label']}/{PREC_LABEL[r['ns_precision']]}={r['recovered_count']}"
                                          for r in records[-len(precisions) * (len(tiles) + 2):] if r["label"] != "SGD"), flush=True)
    return {"config": {"d": d, "alpha": alpha, "seeds": list(seeds), "batch_scale": batch_scale, "num_items": num_items,
                       "precisions": precisions, "tiles": list(tiles), "ns_steps": ns_steps, "problem_dtype": problem_dtype,
                       "device": str(dev)},
            "records": records}


def aggregate(records):
    rec, gap = defaultdict(list), defaultdict(list)
    for r in records:
        rec[(r["label"], r["ns_precision"])].append(r["recovered_count"])
        gap[(r["label"], r["ns_precision"])].append(r["rel_fro_gap_to_fp64"])
    return {k: mean_std(v) for k, v in rec.items()}, {k: mean_std(v)[0] for k, v in gap.items()}


def plot(data: dict, out_dir: str):
    cfg = data["config"]
    rec, gap = aggregate(data["records"])
    precs = cfg["precisions"]
    labels = [m[0] for m in methods(cfg["tiles"]) if m[0] != "SGD"]
    bar_chart(labels, {PREC_LABEL[p]: [rec[(lab, p)][0] for lab in labels] for p in precs}, "one-step recovered items",
              f"d={cfg['d']}, N={cfg['num_items']}, alpha={cfg['alpha']:g}, K={cfg['ns_steps']}", out_dir, NAME,
              errors={PREC_LABEL[p]: ([rec[(lab, p)][0] - rec[(lab, p)][1] for lab in labels],
                                      [rec[(lab, p)][0] + rec[(lab, p)][1] for lab in labels]) for p in precs})
    low = [p for p in precs if p not in ("fp64_ref", "fp32")]
    header = ("method", *[PREC_LABEL[p] for p in precs], *[f"dF {PREC_LABEL[p]}" for p in low])
    rows = [(lab, *[f"{rec[(lab, p)][0]:.1f}+-{rec[(lab, p)][1]:.1f}" for p in precs], *[gap[(lab, p)] for p in low])
            for lab in labels + ["SGD"]]
    txt = text_table(header, rows)
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)
    tex_rows = [(lab.replace("HiMuon-", "HiMuon-$") + ("$" if lab.startswith("HiMuon-") else ""),
                 *[rf"${rec[(lab, p)][0]:.1f}\!\pm\!{rec[(lab, p)][1]:.1f}$" for p in precs],
                 *[f"{gap[(lab, p)]:.3f}" for p in low]) for lab in labels]
    tex = latex_table(("Method", *[PREC_LABEL[p] for p in precs], *[rf"$\delta_F$ {PREC_LABEL[p]}" for p in low]), tex_rows,
                      caption=(f"One-step recovered items and operator gap to fp64 (d={cfg['d']}, N={cfg['num_items']}, "
                               f"$\\alpha$={cfg['alpha']:g}, B/d={cfg['batch_scale']:g}, K={cfg['ns_steps']}, "
                               f"{len(cfg['seeds'])} seeds; {cfg['device']})."), label="tab:precision_recovery")
    print("LaTeX table:", write_text(out_dir, NAME + "_table", tex, ext="tex"))


def add_args(p):
    gpu = have_cuda()
    p.add_argument("--d", type=int, default=1024 if gpu else 256)
    p.add_argument("--alpha", type=float, default=1.5)
    p.add_argument("--seeds", type=int, nargs="+", default=[0, 1, 2, 3, 4])
    p.add_argument("--batch-scale", type=float, default=10.0)
    p.add_argument("--num-items", type=int, default=4096 if gpu else 1024)
    p.add_argument("--precisions", nargs="+", default=None, choices=list(am.NS_PRECISIONS),
                   help="default: fp64_ref fp32 bf16 fp8e4m3_sim, plus fp8e4m3_native where the GPU has fp8 tensor cores")
    p.add_argument("--tiles", type=int, nargs="+", default=[128, 256, 512] if gpu else [32, 64, 128])
    p.add_argument("--ns-steps", type=int, default=5)
    p.add_argument("--problem-dtype", default="float32", choices=["float32", "float64"])


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
