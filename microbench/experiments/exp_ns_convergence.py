"""How many Newton-Schulz iterations are enough: convergence to the polar factor against the iteration count K.

For K = 1 .. ``max_k`` and every tile size the experiment orthogonalises a D x D Gaussian matrix

* whole (full-matrix NS, what Muon does) and compares with the fp64 polar factor of the whole matrix, and
* tile by tile (what HiMuon does) and compares every tile with the fp64 polar factor of that tile,

reporting for each (K, tile) the mean and the worst per-tile cosine, the relative Frobenius error and the spread of the
singular values, averaged over seeds.  The quintic iteration with the (3.4445, -4.7750, 2.0315) coefficients does not
converge to singular values of exactly 1 (it oscillates in a band around it), so the cosine saturates near 0.98 after
five iterations; that plateau is what justifies the default ``ns_steps = 5``.  (Reference:
``microbench/experiments/exp_ns_convergence.py:148-250``: D = 4096, tiles 128/256/512, 3 seeds.)

Runs on CPU or GPU (on a GPU the bf16 iteration is the library's kernel path).

    python -m microbench.experiments.exp_ns_convergence [--D 4096] [--max-k 10] [--tiles 128 256 512] [--seeds 3]
    python -m microbench.experiments.exp_ns_convergence --plot-only
"""

from __future__ import annotations

import torch

from himuon_b200.optimizers import HiMuon

from ..bench_utils import default_device, experiment_main, mean_std, polar_factor
from ..plot_style import line_chart, text_table, write_text

NAME = "ns_convergence"
MAX_TILES_SCORED = 64          # per (K, tile): the fp64 SVD of every tile is the expensive part


def _tiles_of(g: torch.Tensor, T: int) -> torch.Tensor:
    tiled, _ = HiMuon._tile(g, (T, T))
    return tiled.reshape(-1, T, T)


def _pick(n: int, limit: int, seed: int) -> torch.Tensor:
    if n <= limit:
        return torch.arange(n)
    return torch.randperm(n, generator=torch.Generator().manual_seed(seed))[:limit]


def run(D: int = 1024, max_k: int = 8, tiles=(128, 256, 512), seeds: int = 2, dtype: str = "bf16") -> dict:
    dev = default_device()
    work = {"bf16": torch.bfloat16, "fp32": torch.float32}[dtype]
    ks = list(range(1, max_k + 1))
    tiles = [t for t in tiles if t <= D]
    acc = {"full": {k: {"cos": [], "rel": []} for k in ks}}
    for T in tiles:
        acc[str(T)] = {k: {"cos": [], "worst": [], "rel": [], "sv_lo": [], "sv_hi": []} for k in ks}
    for seed in range(seeds):
        g = torch.randn(D, D, generator=torch.Generator().manual_seed(seed)).to(dev)
        p_full = polar_factor(g)
        per_tile = {}
        for T in tiles:
            blocks = _tiles_of(g, T)
            sel = _pick(blocks.shape[0], MAX_TILES_SCORED, seed).to(dev)
            per_tile[T] = (blocks, sel, polar_factor(blocks[sel]))
        for k in ks:
            y = HiMuon.newton_schulz(g.to(work), k).double()
            acc["full"][k]["cos"].append(float((y * p_full).sum() / (y.norm() * p_full.norm())))
            acc["full"][k]["rel"].append(float((y - p_full).norm() / p_full.norm()))
            for T in tiles:
                blocks, sel, p_tiles = per_tile[T]
                yt = HiMuon.newton_schulz(blocks.to(work), k)[sel].double()
                cos = (yt * p_tiles).sum(dim=(-2, -1)) / (yt.norm(dim=(-2, -1)) * p_tiles.norm(dim=(-2, -1)))
                sv = torch.linalg.svdvals(yt)
                a = acc[str(T)][k]
                a["cos"].append(float(cos.mean()))
                a["worst"].append(float(cos.min()))
                a["rel"].append(float(((yt - p_tiles).norm(dim=(-2, -1)) / p_tiles.norm(dim=(-2, -1))).mean()))
                a["sv_lo"].append(float(sv.min()))
                a["sv_hi"].append(float(sv.max()))
    out = {"D": D, "ks": ks, "tiles": tiles, "seeds": seeds, "dtype": dtype, "device": str(dev), "series": {}}
    for name, per_k in acc.items():
        s = {}
        for key in next(iter(per_k.values())):
            ms = [mean_std(per_k[k][key]) for k in ks]
            s[key] = [m for m, _ in ms]
            s[key + "_std"] = [sd for _, sd in ms]
        out["series"][name] = s
    return out


def plot(data: dict, out_dir: str):
    ks = data["ks"]
    cos = {("full matrix" if n == "full" else f"tile {n}"): s["cos"] for n, s in data["series"].items()}
    bands = {("full matrix" if n == "full" else f"tile {n}"): ([m - sd for m, sd in zip(s["cos"], s["cos_std"])],
                                                              [m + sd for m, sd in zip(s["cos"], s["cos_std"])])
             for n, s in data["series"].items()}
    line_chart(ks, cos, "NS iterations K", "cosine to the fp64 polar factor",
               f"NS convergence, D={data['D']}, {data['dtype']}, {data['seeds']} seeds", out_dir, NAME, bands=bands)
    rel = {("full matrix" if n == "full" else f"tile {n}"): s["rel"] for n, s in data["series"].items()}
    line_chart(ks, rel, "NS iterations K", "relative Frobenius error", f"NS error, D={data['D']}", out_dir,
               NAME + "_error", logy=True)
    rows = []
    for n, s in data["series"].items():
        if n == "full":
            continue
        for i, k in enumerate(ks):
            rows.append((n, k, s["cos"][i], s["worst"][i], s["rel"][i], s["sv_lo"][i], s["sv_hi"][i]))
    txt = text_table(("tile", "K", "mean cosine", "worst-tile cosine", "rel. Frobenius err", "sv min", "sv max"), rows)
    print(txt)
    write_text(out_dir, NAME + "_tiles", txt)


def add_args(p):
    p.add_argument("--D", type=int, default=1024, help="matrix side (the reference figure uses 4096)")
    p.add_argument("--max-k", type=int, default=8)
    p.add_argument("--tiles", type=int, nargs="+", default=[128, 256, 512])
    p.add_argument("--seeds", type=int, default=2, help="number of random matrices averaged")
    p.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16", help="arithmetic of the iteration")


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
