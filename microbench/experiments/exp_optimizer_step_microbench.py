"""Optimizer step time and peak memory on a synthetic stack of K x Linear(H, H) in bf16.

Arms (the reference compares Muon, per-parameter HiMuon and cross-layer HiMuon with a CUDA graph,
``microbench/experiments/exp_optimizer_step_microbench.py:58-86,146-234``):

* ``muon``          - full-matrix Newton-Schulz per parameter;
* ``legacy``        - ``HiMuonLegacy``: tile-local NS, one parameter at a time;
* ``himuon``        - ``HiMuon``: all parameters' tiles batched into one NS call, multi-tensor momentum / apply kernels;
* ``himuon+graph``  - the same with the step replayed from a CUDA graph (the shipped default);
* ``adamw``         - the fused multi-tensor AdamW, as the floor of what an optimizer step can cost.

A fresh random gradient is written before every timed step (outside the timed region), the step is timed with CUDA
events, and the peak memory is taken over five further steps after warm-up, so one-time allocations (tile buffers, graph
pools) count the way they do in a training run.  Reported per hidden size: median / quartile milliseconds, speed-up
over Muon, peak bytes and their ratio to Muon's.

    python -m microbench.experiments.exp_optimizer_step_microbench [--sizes 1024 2048 4096] [--K 8] [--tile 512]
    python -m microbench.experiments.exp_optimizer_step_microbench --plot-only
"""

from __future__ import annotations

import gc

import torch
import torch.nn as nn

from himuon_b200.optimizers import AdamW, HiMuon, HiMuonLegacy, Muon

from ..bench_utils import default_device, experiment_main, stats
from ..plot_style import bar_chart, text_table, write_text

NAME = "optimizer_step_microbench"
COMMON = dict(lr=0.02, momentum=0.95, nesterov=True, weight_decay=0.1)


def arms(tile: int, with_graph: bool):
    out = [
        ("muon", lambda ps: Muon(ps, **COMMON)),
        ("legacy", lambda ps: HiMuonLegacy(ps, tile_size=tile, ns_steps=5, **COMMON)),
        ("himuon", lambda ps: HiMuon(ps, tile_size=tile, ns_steps=5, cuda_graph=False, **COMMON)),
    ]
    if with_graph:
        out.append(("himuon+graph", lambda ps: HiMuon(ps, tile_size=tile, ns_steps=5, cuda_graph=True, cuda_graph_warmup=3, **COMMON)))
    out.append(("adamw", lambda ps: AdamW(ps, lr=1e-3, weight_decay=0.1)))
    return out


def make_model(H: int, K: int, device, dtype) -> nn.Module:
    return nn.Sequential(*[nn.Linear(H, H, bias=False, dtype=dtype) for _ in range(K)]).to(device)


def fill_random_grads(model: nn.Module, seed: int):
    dev = next(model.parameters()).device
    gen = torch.Generator(device=dev.type).manual_seed(seed)
    for p in model.parameters():
        if p.grad is None:
            p.grad = torch.empty_like(p)
        p.grad.normal_(generator=gen)


def _sync(dev):
    if dev.type == "cuda":
        torch.cuda.synchronize()


def measure_step(opt, model, warmup: int, repeats: int, seed_base: int = 5000) -> list[float]:
    import time

    dev = next(model.parameters()).device
    for i in range(warmup):
        fill_random_grads(model, seed_base + i)
        opt.step()
    _sync(dev)
    times = []
    for i in range(repeats):
        fill_random_grads(model, seed_base + warmup + i)
        _sync(dev)
        if dev.type == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            opt.step()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            opt.step()
            times.append((time.perf_counter() - t0) * 1e3)
    return times


def measure_peak(opt, model, n_steps: int = 5, seed_base: int = 9000) -> int:
    dev = next(model.parameters()).device
    if dev.type != "cuda":
        return 0
    for i in range(n_steps):
        fill_random_grads(model, seed_base + i)
        opt.step()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    for i in range(n_steps):
        fill_random_grads(model, seed_base + 100 + i)
        opt.step()
    torch.cuda.synchronize()
    return int(torch.cuda.max_memory_allocated())


def bench_one(H: int, K: int, make_opt, warmup: int, repeats: int) -> dict:
    dev = default_device()
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    torch.manual_seed(7)
    model = make_model(H, K, dev, dtype)
    fill_random_grads(model, 1)
    opt = make_opt(list(model.parameters()))
    times = measure_step(opt, model, warmup, repeats)
    peak = measure_peak(opt, model)
    med, p25, p75 = stats(times)
    del opt, model
    gc.collect()
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    return {"median_ms": med, "p25_ms": p25, "p75_ms": p75, "peak_bytes": peak}


def run(sizes=(1024, 2048, 4096), K: int = 8, tile: int = 512, warmup: int = 20, repeats: int = 50) -> dict:
    dev = default_device()
    out = {"config": {"sizes": list(sizes), "K": K, "tile": tile, "device": str(dev)}, "per_H": {}}
    for H in sizes:
        res = {}
        for label, make_opt in arms(tile, with_graph=dev.type == "cuda"):
            res[label] = bench_one(H, K, make_opt, warmup, repeats)
            print(f"H={H} {label:13s} {res[label]['median_ms']:8.3f} ms  peak {res[label]['peak_bytes'] / 2**20:8.1f} MiB", flush=True)
        for label in res:
            res[label]["speedup_vs_muon"] = res["muon"]["median_ms"] / res[label]["median_ms"]
            res[label]["peak_vs_muon"] = (res[label]["peak_bytes"] / res["muon"]["peak_bytes"]) if res["muon"]["peak_bytes"] else None
        out["per_H"][str(H)] = res
    return out


def plot(data: dict, out_dir: str):
    sizes = [str(h) for h in data["config"]["sizes"]]
    labels = list(next(iter(data["per_H"].values())))
    per = data["per_H"]
    bar_chart([f"H={h}" for h in sizes], {m: [per[h][m]["median_ms"] for h in sizes] for m in labels}, "ms / step",
              f"optimizer step, {data['config']['K']} x Linear(H,H), tile {data['config']['tile']}", out_dir, NAME, log=True,
              errors={m: ([per[h][m]["p25_ms"] for h in sizes], [per[h][m]["p75_ms"] for h in sizes]) for m in labels})
    bar_chart([f"H={h}" for h in sizes], {m: [per[h][m]["speedup_vs_muon"] for h in sizes] for m in labels if m != "muon"},
              "speed-up over Muon", "optimizer step", out_dir, NAME + "_speedup", value_fmt="{:.1f}x", baseline=1.0)
    bar_chart([f"H={h}" for h in sizes], {m: [per[h][m]["peak_bytes"] / 2 ** 20 for h in sizes] for m in labels}, "peak MiB",
              "peak memory over five steps", out_dir, NAME + "_memory")
    rows = [(h, m, per[h][m]["median_ms"], per[h][m]["p25_ms"], per[h][m]["p75_ms"], per[h][m]["speedup_vs_muon"],
             per[h][m]["peak_bytes"] / 2 ** 20, per[h][m]["peak_vs_muon"]) for h in sizes for m in labels]
    txt = text_table(("H", "optimizer", "median ms", "p25", "p75", "x Muon", "peak MiB", "peak / Muon"), rows)
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)


def add_args(p):
    p.add_argument("--sizes", type=int, nargs="+", default=[1024, 2048, 4096], help="hidden sizes H")
    p.add_argument("--K", type=int, default=8, help="number of Linear(H, H) layers")
    p.add_argument("--tile", type=int, default=512)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--repeats", type=int, default=50)


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
