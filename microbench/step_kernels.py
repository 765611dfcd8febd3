"""One optimizer step of the headline configuration between cudaProfilerStart / cudaProfilerStop, for a per-kernel
time table:

    python -m microbench.step_kernels                      # plain run (prints the step time from CUDA events)
    ncu --profile-from-start off --metrics gpu__time_duration.sum --clock-control none --csv \\
        --log-file launches.csv python -m microbench.step_kernels
    python -m microbench.step_kernels --summarise launches.csv      # per-kernel totals (no GPU needed)

Qwen3-4B, sequence 1024, micro-batch 2, gradient accumulation 8, HiMuon tile 512, one GPU, bf16, synthetic tokens,
eager launches (no CUDA graphs, so that every kernel is an ordinary launch the profiler can see by name).  One metric
means one pass: nothing is saved or restored around the launches, which is what makes a full-size step capturable.
Under the profiler the launches are serialised and cold, so compare shares, not absolute times.
"""

from __future__ import annotations

import argparse
import csv
import re
import sys
from collections import defaultdict


def summarise(path: str) -> None:
    rows = []
    with open(path, newline="") as f:
        lines = [ln for ln in f if not ln.startswith("==")]
    for rec in csv.DictReader(lines):
        if rec.get("Metric Name") != "gpu__time_duration.sum":
            continue
        val = float(rec["Metric Value"].replace(",", ""))
        unit = rec.get("Metric Unit", "ns")
        scale = {"ns": 1e-6, "us": 1e-3, "usecond": 1e-3, "nsecond": 1e-6, "ms": 1.0, "msecond": 1.0}.get(unit, 1e-6)
        rows.append((rec["Kernel Name"], val * scale))
    tot = defaultdict(lambda: [0.0, 0])
    for name, ms in rows:
        key = re.sub(r"<.*", "", name.split("(")[0]).strip()
        tot[key][0] += ms
        tot[key][1] += 1
    total = sum(v[0] for v in tot.values())
    print(f"{len(rows)} launches, {total:.1f} ms of kernel time")
    print("| kernel | launches | ms | share |\n|---|---|---|---|")
    for k, (ms, n) in sorted(tot.items(), key=lambda kv: -kv[1][0]):
        print(f"| `{k}` | {n} | {ms:.2f} | {100 * ms / total:.1f} % |")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--summarise", type=str, default=None)
    ap.add_argument("--model", type=str, default="Qwen3-4B")
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--grad-acc", type=int, default=8)
    ap.add_argument("--tile", type=int, default=512)
    args = ap.parse_args()
    if args.summarise:
        summarise(args.summarise)
        return

    import torch

    from himuon_b200 import ops
    from himuon_b200.models import CausalLM, get_config
    from himuon_b200.optim import get_optimizer
    from himuon_b200.parallel.fsdp import ShardedEngine
    from himuon_b200.trainer import Trainer

    device = torch.device("cuda:0")
    torch.manual_seed(0)
    cfg = get_config(args.model)
    with torch.device(device):
        model = CausalLM(cfg).to(torch.bfloat16)
    engine = ShardedEngine(model, use_banks=True)
    opt = get_optimizer("himuon", model, argparse.Namespace(lr=1e-2, weight_decay=0.1, tile_size=args.tile, cuda_graph=False))
    engine.attach_optimizer(opt)
    trainer = Trainer(model, opt, None, engine, args.grad_acc, device)
    trainer.zero_set_to_none = False
    g = torch.Generator().manual_seed(0)

    def batches():
        return [{"input_ids": (ids := torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq_len), generator=g).to(device)),
                 "labels": ids} for _ in range(args.grad_acc)]

    for _ in range(2):
        trainer.train_step(batches())
    step = batches()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0 = ops.launch_count()
    torch.cuda.profiler.start()
    e0.record()
    loss = trainer.train_step(step)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ops.check_status()
    print(f"one eager step: {e0.elapsed_time(e1):.1f} ms, {ops.launch_count() - n0} library launches, loss {float(loss):.3f}")
    engine.close()


if __name__ == "__main__":
    sys.exit(main())
