"""Tile-local vs full-matrix Newton-Schulz on the projection shapes of real models, per layer role and as whole
banks (reference: ``exp_real_shapes_bench.py:93-238``), plus the tile sweep 128/256/512/1024/full on the
Qwen3-0.6B bank shapes with the achieved fraction of the measured GEMM peak."""

from __future__ import annotations

import json
import os

import torch

from himuon_b200.models import get_config
from himuon_b200.ops import ns as ns_ops
from himuon_b200.ops import reference as ref

from ..bench_utils import measure
from ..plot_style import text_table


def role_shapes(name):
    c = get_config(name)
    H, D = c.hidden_size, c.head_dim
    return {"q": (c.num_attention_heads * D, H), "k": (c.num_key_value_heads * D, H), "v": (c.num_key_value_heads * D, H),
            "o": (H, c.num_attention_heads * D), "gate": (c.intermediate_size, H), "up": (c.intermediate_size, H),
            "down": (H, c.intermediate_size)}, c.num_hidden_layers


def _tiled_ns(x3d, tile, ws):
    """NS over every (tile x tile) block of a (B, h, w) batch of matrices (zero padded)."""
    B, h, w = x3d.shape
    th, tw = min(tile, h), min(tile, w)
    if tile >= max(h, w):
        return ns_ops.ns_inplace_cuda(x3d.clone(), 5, workspace=ws)
    tiles = torch.cat([ref.tile(x3d[i], (th, tw))[0].reshape(-1, th, tw) for i in range(B)], 0)
    return ns_ops.ns_inplace_cuda(tiles.contiguous(), 5, workspace=ws)


def ns_flops(B, m, n, steps=5):
    lo, hi = min(m, n), max(m, n)
    return B * steps * (2 * lo * lo * hi * 2 + 2 * lo ** 3)


def run(models=("Qwen3-0.6B", "Qwen3-1.7B", "Qwen3-4B"), tile: int = 512, sweep_model: str = "Qwen3-0.6B",
        sweep_tiles=(128, 256, 512, 1024, 10 ** 9)) -> dict:
    peak = None
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak = json.load(f).get("bf16_tflops")
    out = {"tile": tile, "per_layer": {}, "sweep": [], "peak_tflops": peak}
    ws = ns_ops.NSWorkspace()
    for name in models:
        shapes, _ = role_shapes(name)
        res = {}
        for role, (h, w) in shapes.items():
            x = torch.randn(1, h, w, device="cuda", dtype=torch.bfloat16)
            full = measure(lambda: ns_ops.ns_inplace_cuda(x.clone(), 5, workspace=ws))["median_ms"]
            tiled = measure(lambda: _tiled_ns(x, tile, ws))["median_ms"]
            res[role] = {"shape": [h, w], "full_ms": full, "tile_ms": tiled, "speedup": full / tiled}
        out["per_layer"][name] = res
    shapes, L = role_shapes(sweep_model)
    banks = {"q": (L, *shapes["q"]), "kv": (2 * L, *shapes["k"]), "o": (L, *shapes["o"]), "gate_up": (2 * L, *shapes["gate"]),
             "down": (L, *shapes["down"])}
    for t in sweep_tiles:
        total_ms, total_fl = 0.0, 0.0
        for bank, (n, h, w) in banks.items():
            x = torch.randn(n, h, w, device="cuda", dtype=torch.bfloat16)
            ms = measure(lambda: _tiled_ns(x, t, ws), warmup=2, iters=5)["median_ms"]
            th, tw = min(t, h), min(t, w)
            nt = n * (-(-h // th)) * (-(-w // tw))
            total_ms += ms
            total_fl += ns_flops(nt, th, tw)
        tf = total_fl / total_ms / 1e9
        out["sweep"].append({"tile": "full" if t >= 10 ** 8 else t, "ms": total_ms, "tflops": tf,
                             "fraction_of_measured_peak": tf / peak if peak else None})
    return out


def plot(data: dict, out_dir: str):
    for name, res in data["per_layer"].items():
        print(name, " ".join(f"{r}:{v['speedup']:.2f}x" for r, v in res.items()))
    print(text_table(("tile", "ms (all banks)", "TFLOP/s", "of measured peak"),
                     [(s["tile"], f"{s['ms']:.2f}", f"{s['tflops']:.0f}",
                       f"{s['fraction_of_measured_peak']:.2f}" if s["fraction_of_measured_peak"] else "-") for s in data["sweep"]]))
