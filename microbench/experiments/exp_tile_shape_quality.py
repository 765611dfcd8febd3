"""Training quality against the tile shape: a small Llama trained for a few hundred steps with HiMuon at several
square and rectangular tiles, reporting the mean loss of the last third of the run and the wall clock (reference:
``exp_tile_shape_quality.py:56-137`` uses llama_220m, 300 steps, batch 8 x 1024, lr 0.02, on FineWeb).  Offline the
data is a fixed synthetic Markov-chain corpus so that the loss can actually fall."""

from __future__ import annotations

import argparse
import time

import torch

from himuon_b200.models import CausalLM, get_config
from himuon_b200.optim import get_optimizer
from himuon_b200.trainer import wsd_schedule

from ..plot_style import text_table


def _markov_batches(vocab, batch, seq, steps, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    nxt = torch.randint(0, vocab, (vocab, 4), generator=g)          # each token has 4 likely successors
    out = []
    for _ in range(steps):
        ids = torch.empty(batch, seq, dtype=torch.long)
        ids[:, 0] = torch.randint(0, vocab, (batch,), generator=g)
        choice = torch.randint(0, 4, (batch, seq), generator=g)
        for t in range(1, seq):
            ids[:, t] = nxt[ids[:, t - 1], choice[:, t]]
        out.append(ids.to(device))
    return out


def run(model_name: str = "llama_220m", tiles=((512, 512), (256, 256), (128, 128), (256, 512), (128, 256)), steps: int = 60,
        batch: int = 8, seq: int = 512, lr: float = 0.02) -> dict:
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    cfg = get_config(model_name)
    data = _markov_batches(min(cfg.vocab_size, 4096), batch, seq, steps, device=dev)
    rows = []
    for tile in tiles:
        torch.manual_seed(0)
        model = CausalLM(cfg).to(dev, dtype)
        opt = get_optimizer("himuon", model, argparse.Namespace(lr=lr, weight_decay=0.1, tile_size=tuple(tile), cuda_graph=dev.type == "cuda"))
        sched = wsd_schedule(opt, max(1, steps // 10), 0, steps, 0.1)
        losses, t0 = [], time.perf_counter()
        for ids in data:
            loss = model(ids, labels=ids).loss
            loss.backward()
            opt.step()
            sched.step()
            opt.zero_grad(set_to_none=False)
            losses.append(float(loss))
        if dev.type == "cuda":
            torch.cuda.synchronize()
        tail = losses[-max(1, steps // 3):]
        plan = opt.xlayer_plan()
        rows.append({"tile": list(tile), "final_loss": sum(tail) / len(tail), "wall_s": time.perf_counter() - t0,
                     "buckets": len(plan), "tiles_total": sum(b["B_total"] for b in plan)})
    return {"model": model_name, "steps": steps, "rows": rows}


def plot(data: dict, out_dir: str):
    print(text_table(("tile", "mean loss (last third)", "wall s", "tiles"),
                     [(tuple(r["tile"]), f"{r['final_loss']:.3f}", f"{r['wall_s']:.1f}", r["tiles_total"]) for r in data["rows"]]))
