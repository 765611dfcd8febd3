"""Tile-local against full-matrix Newton-Schulz on the projection shapes of real models.

For every distinct Muon-eligible matrix shape of the chosen models (q, k, v, o, gate, up, down of one decoder block;
the shapes come from the in-tree architecture table, no weights are downloaded) the experiment measures

* the time of full-matrix NS (what Muon runs) and of tile-local NS (what HiMuon runs) with the tile size under test,
  interleaved, with the paired speed-up and its quartiles,
* the extra memory of both,
* the padding overhead of the tiling (zero elements added so that both sides become multiples of the tile),
* the quality of both outputs: spread of the singular values, and for the tile-local result the mean cosine of each
  tile to the fp64 polar factor of that tile, against the cosine of the full result to the polar factor of the matrix,

and then, per model, the whole-step cost: all layers of a role stacked into one bank (the layout of the sharded
engine) and orthogonalised in one batched call, swept over the tile sizes 128 / 256 / 512 / 1024 / full, with the
achieved TFLOP/s and its fraction of the measured GEMM peak.  (Reference: per-layer speed-ups and qualities,
``microbench/experiments/exp_real_shapes_bench.py:93-238``.)

    python -m microbench.experiments.exp_real_shapes_bench [--models Qwen3-0.6B Qwen3-1.7B Qwen3-4B] [--tile 512]
    python -m microbench.experiments.exp_real_shapes_bench --plot-only
"""

from __future__ import annotations

import torch

from himuon_b200.models import get_config
from himuon_b200.ops import ns as ns_ops
from himuon_b200.ops import reference as ref
from himuon_b200.optimizers import HiMuon

from ..bench_utils import (batched_polar_cosine, cosine_sim, default_device, experiment_main, measure, measure_memory,
                           measure_paired_speedup, measured_peaks, polar_factor, sv_stats)
from ..plot_style import bar_chart, line_chart, text_table, write_text
from .exp_ns_kernel_microbench import ns_flops

NAME = "real_shapes_bench"
ROLES = ("q", "k", "v", "o", "gate", "up", "down")
FULL = 10 ** 9


def role_shapes(name: str):
    c = get_config(name)
    H, D = c.hidden_size, c.head_dim
    shapes = {"q": (c.num_attention_heads * D, H), "k": (c.num_key_value_heads * D, H),
              "v": (c.num_key_value_heads * D, H), "o": (H, c.num_attention_heads * D),
              "gate": (c.intermediate_size, H), "up": (c.intermediate_size, H), "down": (H, c.intermediate_size)}
    return shapes, c.num_hidden_layers


def padding_overhead(h: int, w: int, tile: int) -> float:
    th, tw = min(tile, h), min(tile, w)
    ph, pw = -(-h // th) * th, -(-w // tw) * tw
    return ph * pw / (h * w) - 1.0


def _ns(x3d: torch.Tensor, ws) -> torch.Tensor:
    if x3d.is_cuda:
        return ns_ops.ns_inplace_cuda(x3d.clone(), 5, workspace=ws)
    return ref.newton_schulz(x3d, 5)


def tiled_ns(x3d: torch.Tensor, tile: int, ws):
    """NS over every (tile x tile) block of a (B, h, w) batch; returns the orthogonalised tiles ``(B * R * C, th, tw)``."""
    B, h, w = x3d.shape
    if tile >= max(h, w):
        return _ns(x3d, ws)
    th, tw = min(tile, h), min(tile, w)
    tiles = torch.cat([HiMuon._tile(x3d[i], (th, tw))[0].reshape(-1, th, tw) for i in range(B)], 0)
    return _ns(tiles.contiguous(), ws)


def _quality(x2d: torch.Tensor, tile: int, ws, max_tiles: int = 16) -> dict:
    """Singular-value spread and polar cosines of the full and the tile-local result for one matrix."""
    full = _ns(x2d[None], ws)[0].float()
    out = {"full": {**sv_stats(full), "polar_cosine": cosine_sim(full, polar_factor(x2d.float()))}}
    th, tw = min(tile, x2d.shape[0]), min(tile, x2d.shape[1])
    blocks = HiMuon._tile(x2d, (th, tw))[0].reshape(-1, th, tw)
    sel = torch.linspace(0, blocks.shape[0] - 1, min(max_tiles, blocks.shape[0])).long().to(blocks.device)
    y = tiled_ns(x2d[None], tile, ws)[sel].float()
    cos = batched_polar_cosine(y, blocks[sel].float())
    sv = torch.linalg.svdvals(y.double())
    out["tile"] = {"sv_mean": float(sv.mean()), "sv_std": float(sv.std()), "sv_min": float(sv.min()), "sv_max": float(sv.max()),
                   "polar_cosine": float(cos.mean()), "polar_cosine_worst": float(cos.min())}
    return out


def run(models=("Qwen3-0.6B", "Qwen3-1.7B", "Qwen3-4B"), tile: int = 512, ns_steps: int = 5, warmup: int = 3, repeats: int = 30,
        sweep_tiles=(128, 256, 512, 1024, FULL), quality: bool = True, seed: int = 0) -> dict:
    assert ns_steps == 5, "the kernels under test run five iterations"
    dev = default_device()
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    peak = measured_peaks().get("bf16_tflops")
    ws = ns_ops.NSWorkspace() if dev.type == "cuda" else None
    gen = torch.Generator(dev.type).manual_seed(seed)
    out = {"tile": tile, "models": list(models), "device": str(dev), "peak_tflops": peak, "per_layer": {}, "sweep": {}}
    for name in models:
        shapes, L = role_shapes(name)
        res, seen = {}, {}
        for role in ROLES:
            h, w = shapes[role]
            if (h, w) in seen:                                 # k/v and gate/up share a shape: measure it once
                res[role] = dict(res[seen[(h, w)]], same_as=seen[(h, w)])
                continue
            seen[(h, w)] = role
            x = torch.randn(1, h, w, device=dev, dtype=dtype, generator=gen)
            pair = measure_paired_speedup(lambda: _ns(x, ws), lambda: tiled_ns(x, tile, ws), warmup=warmup, iters=repeats)
            r = {"shape": [h, w], "full_ms": pair["baseline_ms"], "tile_ms": pair["candidate_ms"],
                 "speedup": pair["speedup_median"], "speedup_p25": pair["speedup_p25"], "speedup_p75": pair["speedup_p75"],
                 "full_peak_bytes": measure_memory(lambda: _ns(x, ws)),
                 "tile_peak_bytes": measure_memory(lambda: tiled_ns(x, tile, ws)),
                 "padding_overhead": padding_overhead(h, w, tile),
                 "tiles": (-(-h // min(tile, h))) * (-(-w // min(tile, w)))}
            if quality:
                r["quality"] = _quality(x[0], tile, ws)
            res[role] = r
            print(f"{name} {role:5s} {h}x{w}: full {r['full_ms']:.3f} ms  tile {r['tile_ms']:.3f} ms  x{r['speedup']:.2f}", flush=True)
        out["per_layer"][name] = res
        # ---- whole banks, tile sweep
        banks = {"q": (L, *shapes["q"]), "kv": (2 * L, *shapes["k"]), "o": (L, *shapes["o"]),
                 "gate_up": (2 * L, *shapes["gate"]), "down": (L, *shapes["down"])}
        sweep = []
        for t in sweep_tiles:
            total_ms = total_fl = 0.0
            for n, h, w in banks.values():
                xb = torch.randn(n, h, w, device=dev, dtype=dtype, generator=gen)
                total_ms += measure(lambda: tiled_ns(xb, t, ws), warmup=2, iters=max(3, repeats // 6))["median_ms"]
                th, tw = min(t, h), min(t, w)
                total_fl += ns_flops(n * (-(-h // th)) * (-(-w // tw)), th, tw)
                del xb
            tf = total_fl / total_ms / 1e9
            sweep.append({"tile": "full" if t >= FULL else t, "ms": total_ms, "tflops": tf,
                          "fraction_of_measured_peak": tf / peak if peak else None})
            print(f"{name} all banks, tile {sweep[-1]['tile']}: {total_ms:.2f} ms  {tf:.0f} TFLOP/s", flush=True)
        out["sweep"][name] = sweep
    return out


def plot(data: dict, out_dir: str):
    for name, res in data["per_layer"].items():
        tag = name.replace("/", "_")
        bar_chart(list(ROLES), {"speed-up": [res[r]["speedup"] for r in ROLES]}, "full-NS time / tile-NS time",
                  f"{name}, tile {data['tile']}", out_dir, f"{NAME}_{tag}", value_fmt="{:.1f}x", baseline=1.0,
                  errors={"speed-up": ([res[r]["speedup_p25"] for r in ROLES], [res[r]["speedup_p75"] for r in ROLES])})
        rows = []
        for r in ROLES:
            v = res[r]
            q = v.get("quality")
            rows.append((r, "x".join(map(str, v["shape"])), v["tiles"], v["full_ms"], v["tile_ms"], v["speedup"],
                         v["full_peak_bytes"] / 2 ** 20, v["tile_peak_bytes"] / 2 ** 20, 100 * v["padding_overhead"],
                         q and q["full"]["sv_std"], q and q["tile"]["sv_std"], q and q["full"]["polar_cosine"],
                         q and q["tile"]["polar_cosine"]))
        txt = text_table(("role", "shape", "tiles", "full ms", "tile ms", "speed-up", "full MiB", "tile MiB", "pad %",
                          "sv std full", "sv std tile", "cos full", "cos tile"), rows)
        print(f"# {name}\n{txt}")
        write_text(out_dir, f"{NAME}_{tag}_detail", txt)
    if data["sweep"]:
        tiles = [str(s["tile"]) for s in next(iter(data["sweep"].values()))]
        line_chart(tiles, {m: [s["ms"] for s in sw] for m, sw in data["sweep"].items()}, "tile", "ms, all banks of the model",
                   "Newton-Schulz over whole banks", out_dir, NAME + "_sweep", logy=True)
        rows = [(m, s["tile"], s["ms"], s["tflops"], s["fraction_of_measured_peak"]) for m, sw in data["sweep"].items() for s in sw]
        txt = text_table(("model", "tile", "ms (all banks)", "TFLOP/s", "of measured peak"), rows)
        print(txt)
        write_text(out_dir, NAME + "_sweep_detail", txt)


def add_args(p):
    p.add_argument("--models", nargs="+", default=["Qwen3-0.6B", "Qwen3-1.7B", "Qwen3-4B"])
    p.add_argument("--tile", type=int, default=512)
    p.add_argument("--ns-steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--repeats", type=int, default=30)
    p.add_argument("--sweep-tiles", type=int, nargs="*", default=[128, 256, 512, 1024, FULL],
                   help=f"tile sizes of the whole-bank sweep ({FULL} = full matrix); empty to skip")
    p.add_argument("--no-quality", dest="quality", action="store_false", help="skip the fp64 SVD quality columns")


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
