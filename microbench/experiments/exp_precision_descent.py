"""Does low-precision or tile-local Newton-Schulz degrade the update as a descent direction?

Two closed-form quantities, tracked along a training trajectory:

    alignment          gamma = <G, D> / <G~, D>            (does the update computed from a minibatch gradient G~
                                                             point along the full-batch gradient G as well?)
    descent potential  phi   = <G~, D>^2 / <D, H D>        (the decrease a line search along D could realise)

with ``D`` the update and ``H`` the Hessian, on a teacher-student matrix least-squares problem
``f(W) = 1/2 E_x ||(W - W*) x||^2`` with ``x ~ N(0, Sigma)`` and a power-law spectrum of ``Sigma``, for which
``G = (W - W*) Sigma``, ``G~ = (W - W*) Sigma_hat_b`` (``Sigma_hat_b`` the covariance of a minibatch) and
``H D = D Sigma`` - no network needed.  One fp32 full-matrix trajectory generates the iterates ``W_k``; at every step
each (tile, precision) operator is applied to the same ``(G, G~)``.  (Setup of the reference,
``microbench/experiments/exp_precision_descent.py:110-190``: dim 1024, alpha 1, 40 steps, lr 0.03, batch 256, tiles
128 / 256 / 512 and full, precisions fp32 / bf16 / fp8-e4m3.)

The figure pair plots gamma and phi against the step, one line per tile at fp32; the table gives, per tile and
precision, the mean of both over the trajectory and their ratio to the fp32 full-matrix values.  Runs on CPU or GPU
(native fp8 products need a GPU with fp8 tensor cores; elsewhere the simulated fp8 rounding is used).

    python -m microbench.experiments.exp_precision_descent [--dim 1024] [--alpha 1.0] [--steps 40] [--tiles 128 256 512]
    python -m microbench.experiments.exp_precision_descent --plot-only
"""

from __future__ import annotations

import torch

from .. import assoc_mem as am
from ..bench_utils import default_device, experiment_main, have_cuda
from ..plot_style import line_chart, text_table, write_text
from .exp_precision_recovery import native_fp8_available

NAME = "precision_descent"


def make_problem(dim: int, alpha: float, device, seed: int):
    """Anisotropic input covariance with eigenvalues ``i^-alpha`` (unit mean) in a random basis; unit-norm teacher and
    starting point."""
    g = torch.Generator(device=device.type).manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(dim, dim, generator=g, device=device))
    lam = torch.arange(1, dim + 1, device=device, dtype=torch.float32).pow(-alpha)
    lam = lam / lam.mean()
    sigma = (q * lam) @ q.t()
    sigma_half = (q * lam.sqrt()) @ q.t()
    w_star = torch.randn(dim, dim, generator=g, device=device)
    w0 = torch.randn(dim, dim, generator=g, device=device)
    return sigma, sigma_half, w_star / w_star.norm(), w0 / w0.norm()


def inner(x: torch.Tensor, y: torch.Tensor) -> float:
    return float((x.double() * y.double()).sum())


def run(dim: int = 1024, alpha: float = 1.0, steps: int = 40, lr: float = 0.03, batch: int = 256, tiles=(128, 256, 512),
        precisions=None, ns_steps: int = 5, seed: int = 0) -> dict:
    dev = default_device()
    if precisions is None:
        precisions = ["fp32", "bf16", "fp8e4m3_native" if native_fp8_available() else "fp8e4m3_sim"]
    tiles = [t for t in tiles if t < dim]
    cats = [(f"t{t}", t) for t in tiles] + [("full", None)]
    sigma, sigma_half, w_star, w = make_problem(dim, alpha, dev, seed)
    curves = {f"{c}/{p}": {"gamma": [], "phi": []} for c, _ in cats for p in precisions}
    losses = []
    gen = torch.Generator(device=dev.type).manual_seed(seed + 1)
    for _ in range(steps):
        err = w - w_star
        g_full = err @ sigma
        z = torch.randn(batch, dim, generator=gen, device=dev) @ sigma_half
        g_mb = err @ (z.t() @ z / batch)
        losses.append(0.5 * inner(err @ sigma_half, err @ sigma_half))
        for cat, tile in cats:
            for p in precisions:
                upd = am.himuon_operator(g_mb, tile, ns_steps, p).float()
                gd = inner(g_mb, upd)
                hd = inner(upd, upd @ sigma)
                curves[f"{cat}/{p}"]["gamma"].append(inner(g_full, upd) / (gd + 1e-20))
                curves[f"{cat}/{p}"]["phi"].append(gd * gd / (hd + 1e-20))
        step_dir = am.himuon_operator(g_mb, None, ns_steps, "fp32").float()
        w = w - lr * step_dir / (step_dir.norm() + 1e-7)
    print(f"loss {losses[0]:.5f} -> {losses[-1]:.5f} over {steps} steps", flush=True)
    return {"config": {"problem": "teacher-student-quadratic", "dim": dim, "alpha": alpha, "steps": steps, "lr": lr,
                       "batch": batch, "tiles": tiles, "precisions": list(precisions), "ns_steps": ns_steps, "device": str(dev)},
            "curves": curves, "loss": losses}


def plot(data: dict, out_dir: str):
    cfg, curves = data["config"], data["curves"]
    cats = [f"t{t}" for t in cfg["tiles"]] + ["full"]
    name_of = lambda c: "full matrix" if c == "full" else f"tile {c[1:]}"
    xs = list(range(cfg["steps"]))
    base = cfg["precisions"][0]
    for metric, ylabel in (("gamma", "alignment gamma"), ("phi", "descent potential phi")):
        line_chart(xs, {name_of(c): curves[f"{c}/{base}"][metric] for c in cats}, "training step", ylabel,
                   f"{ylabel} ({base}), dim={cfg['dim']}, alpha={cfg['alpha']:g}", out_dir, f"{NAME}_{metric}",
                   logy=metric == "phi")
    mean = lambda v: sum(v) / max(1, len(v))
    ref_g, ref_p = mean(curves[f"full/{base}"]["gamma"]), mean(curves[f"full/{base}"]["phi"])
    rows = []
    for c in cats:
        for p in cfg["precisions"]:
            g, ph = mean(curves[f"{c}/{p}"]["gamma"]), mean(curves[f"{c}/{p}"]["phi"])
            rows.append((name_of(c), p, g, g / ref_g if ref_g else None, ph, ph / ref_p if ref_p else None))
    txt = text_table(("operator", "precision", "mean gamma", f"/ full {base}", "mean phi", f"/ full {base}"), rows)
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)
    line_chart(xs, {"loss": data["loss"]}, "training step", "population loss", "fp32 full-matrix trajectory", out_dir,
               NAME + "_loss", logy=True)


def add_args(p):
    gpu = have_cuda()
    p.add_argument("--dim", type=int, default=1024 if gpu else 256)
    p.add_argument("--alpha", type=float, default=1.0, help="exponent of the input covariance spectrum")
    p.add_argument("--steps", type=int, default=40)
    p.add_argument("--lr", type=float, default=0.03)
    p.add_argument("--batch", type=int, default=256)
    p.add_argument("--tiles", type=int, nargs="+", default=[128, 256, 512] if gpu else [32, 64, 128])
    p.add_argument("--precisions", nargs="+", default=None, choices=[x for x in am.NS_PRECISIONS if x != "fp64_ref"])
    p.add_argument("--ns-steps", type=int, default=5)
    p.add_argument("--seed", type=int, default=0)


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
