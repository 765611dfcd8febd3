"""Optimizer-step latency and peak memory: Muon vs HiMuonLegacy vs HiMuon (cross-layer batching + CUDA graph) on
8 x Linear(H, H) in bf16 at tile 512 (reference: ``exp_optimizer_step_microbench.py:58-86,146-164``)."""

from __future__ import annotations

import torch

from himuon_b200.optimizers import HiMuon, HiMuonLegacy, Muon

from ..bench_utils import measure
from ..plot_style import bar_chart, text_table


def _model(H, n=8):
    return torch.nn.ModuleList([torch.nn.Linear(H, H, bias=False, device="cuda", dtype=torch.bfloat16) for _ in range(n)])


def _time(make_opt, H):
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    model = _model(H)
    for p in model.parameters():
        p.grad = torch.randn_like(p)
    opt = make_opt(model.parameters())
    for _ in range(6):                      # eager warm-up, then graph capture where enabled
        opt.step()
    res = measure(opt.step, warmup=3, iters=15)
    res["peak_mb"] = torch.cuda.max_memory_allocated() / 2**20
    return res


def run(hiddens=(1024, 2048, 4096), tile: int = 512) -> dict:
    out = {"H": list(hiddens), "tile": tile, "muon": [], "legacy": [], "himuon": []}
    for H in hiddens:
        out["muon"].append(_time(lambda ps: Muon(ps, lr=0.02), H))
        out["legacy"].append(_time(lambda ps: HiMuonLegacy(ps, lr=0.02, tile_size=tile), H))
        out["himuon"].append(_time(lambda ps: HiMuon(ps, lr=0.02, tile_size=tile, cuda_graph=True, cuda_graph_warmup=3), H))
    return out


def plot(data: dict, out_dir: str):
    rows = []
    for i, H in enumerate(data["H"]):
        m, l, h = data["muon"][i], data["legacy"][i], data["himuon"][i]
        rows.append((H, f"{m['median_ms']:.3f}", f"{l['median_ms']:.3f}", f"{h['median_ms']:.3f}",
                     f"{m['median_ms'] / l['median_ms']:.1f}x", f"{m['median_ms'] / h['median_ms']:.1f}x",
                     f"{m['peak_mb']:.0f}", f"{100 * (h['peak_mb'] / m['peak_mb'] - 1):+.0f}%"))
    print(text_table(("H", "muon ms", "legacy ms", "himuon ms", "legacy x", "himuon x", "muon MB", "himuon mem"), rows))
    bar_chart([str(h) for h in data["H"]], {k: [r["median_ms"] for r in data[k]] for k in ("muon", "legacy", "himuon")},
              "ms / step", "optimizer step, 8 x Linear(H,H)", f"{out_dir}/optimizer_step_microbench.png", log=True)
