"""Training quality against the HiMuon tile shape.

One small Llama is trained for a few hundred steps once per tile shape - squares of decreasing size, rectangles of
equal area on both sides of the fused-kernel boundary, and their tall (M > N) mirror images - with the same seed, the
same replayed list of batches and the same warm-up / stable / decay schedule, and the loss curves are compared.  The
run checks before training that every Muon parameter really goes through the tiled path (no full-matrix fallback for
a tile larger than the matrix), as the reference does (``microbench/experiments/exp_tile_shape_quality.py:56-137``:
llama_220m, 300 steps of 8 x 1024 FineWeb tokens, lr 0.02, 20 warm-up and 60 decay steps).

There is no network here, so the corpus is synthetic: a fixed sparse Markov chain over a few thousand tokens (each
token has a handful of likely successors), which a transformer can actually learn, so the loss falls and tile shapes
can be told apart; the absolute losses do not compare with FineWeb numbers.

Reported per shape: mean loss of the last ``tail`` steps (+- std), its gap to the reference shape (the first one), the
wall clock of the run, the number of NS buckets / tiles per step, and which kernel path the shape takes.

    python -m microbench.experiments.exp_tile_shape_quality [--steps 300] [--shapes 512x512 256x256 128x128 64x256]
    python -m microbench.experiments.exp_tile_shape_quality --plot-only
"""

from __future__ import annotations

import argparse
import time

import torch

from himuon_b200.models import CausalLM, get_config
from himuon_b200.ops import ns as ns_ops
from himuon_b200.optim import get_optimizer
from himuon_b200.trainer import wsd_schedule

from ..bench_utils import default_device, experiment_main, mean_std
from ..plot_style import bar_chart, line_chart, text_table, write_text

NAME = "tile_shape_quality"
# the reference square, two smaller squares, rectangles of area 2^14 (fused-kernel boundary) and 2^15, and tall mirrors
SHAPES = [(512, 512), (256, 256), (128, 128), (16, 1024), (32, 512), (64, 256), (32, 1024), (64, 512), (128, 256),
          (1024, 16), (512, 32), (256, 64), (256, 128), (256, 512), (512, 256)]
SEED = 42


def parse_shape(s) -> tuple[int, int]:
    if isinstance(s, (tuple, list)):
        return int(s[0]), int(s[1])
    a, _, b = str(s).lower().partition("x")
    return int(a), int(b or a)


def shape_label(ts) -> str:
    return f"{ts[0]}x{ts[1]}"


def markov_corpus(vocab: int, batch: int, seq: int, steps: int, fanout: int = 4, seed: int = SEED) -> list[torch.Tensor]:
    """``steps`` batches of token ids from a fixed random chain in which every token has ``fanout`` equally likely
    successors (entropy rate log(fanout) nats: the loss floor a model can reach)."""
    g = torch.Generator().manual_seed(seed)
    nxt = torch.randint(0, vocab, (vocab, fanout), generator=g)
    out = []
    for _ in range(steps):
        ids = torch.empty(batch, seq, dtype=torch.long)
        ids[:, 0] = torch.randint(0, vocab, (batch,), generator=g)
        choice = torch.randint(0, fanout, (batch, seq), generator=g)
        for t in range(1, seq):
            ids[:, t] = nxt[ids[:, t - 1], choice[:, t]]
        out.append(ids)
    return out


def kernel_path(tile) -> str:
    th, tw = tile
    lo, hi = min(th, tw), max(th, tw)
    return "fused tile-resident" if ns_ops.fused_supported(lo, hi) else "three batched GEMMs"


def check_tiled_path(opt, tile) -> dict:
    """Every Muon matrix must be cut into tiles of the requested shape (a tile that covers a whole matrix would be
    the full-matrix iteration and say nothing about the tile shape)."""
    plan = opt.xlayer_plan()                                    # the tiled buckets only
    whole = len(getattr(opt, "_cached_plan", None) or []) - len(plan)
    return {"buckets": len(plan), "tiles_per_step": sum(b["B_total"] for b in plan), "full_matrix_buckets": whole}


def train_one(cfg, tile, batches, lr: float, warmup_steps: int, decay_steps: int, device, dtype) -> dict:
    torch.manual_seed(SEED)
    model = CausalLM(cfg).to(device, dtype)
    ns = argparse.Namespace(lr=lr, weight_decay=0.1, tile_size=tuple(tile), cuda_graph=device.type == "cuda", cuda_graph_warmup=3)
    opt = get_optimizer("himuon", model, ns)
    steps = len(batches)
    sched = wsd_schedule(opt, warmup_steps, max(0, steps - warmup_steps - decay_steps), decay_steps, 0.1)
    losses, plan_info = [], None
    t0 = time.perf_counter()
    for i, ids in enumerate(batches):
        ids = ids.to(device, non_blocking=True)
        loss = model(ids, labels=ids).loss
        loss.backward()
        opt.step()
        if i == 0:
            plan_info = check_tiled_path(opt, tile)
        sched.step()
        opt.zero_grad(set_to_none=False)
        losses.append(float(loss.detach()))
    if device.type == "cuda":
        torch.cuda.synchronize()
    return {"tile": list(tile), "losses": losses, "wall_s": time.perf_counter() - t0, "kernel_path": kernel_path(tile), **plan_info}


def run(model: str = "llama_220m", shapes=None, steps: int = 300, batch: int = 8, seq: int = 1024, lr: float = 0.02,
        warmup_steps: int = 20, decay_steps: int = 60, tail: int = 100, vocab: int = 4096) -> dict:
    dev = default_device()
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    cfg = get_config(model)
    shapes = [parse_shape(s) for s in (shapes or SHAPES)]
    batches = markov_corpus(min(cfg.vocab_size, vocab), batch, seq, steps)
    tail = max(1, min(tail, steps))
    rows = []
    for tile in shapes:
        r = train_one(cfg, tile, batches, lr, min(warmup_steps, steps // 4), min(decay_steps, steps // 3), dev, dtype)
        r["tail_mean"], r["tail_std"] = mean_std(r["losses"][-tail:])
        rows.append(r)
        print(f"tile {shape_label(tile):>9s}: loss(last {tail}) {r['tail_mean']:.4f} +- {r['tail_std']:.4f}  {r['wall_s']:.1f} s  "
              f"{r['tiles_per_step']} tiles/step  [{r['kernel_path']}]"
              + ("  WARNING: some matrices fall back to the full-matrix iteration" if r["full_matrix_buckets"] else ""), flush=True)
    ref_loss = rows[0]["tail_mean"]
    for r in rows:
        r["gap_to_reference"] = r["tail_mean"] - ref_loss
    return {"model": model, "steps": steps, "batch": batch, "seq": seq, "lr": lr, "tail": tail, "device": str(dev),
            "entropy_floor": float(torch.log(torch.tensor(4.0))), "rows": rows}


def _smooth(xs, k=10):
    out, acc = [], 0.0
    for i, x in enumerate(xs):
        acc += x
        if i >= k:
            acc -= xs[i - k]
        out.append(acc / min(i + 1, k))
    return out


def plot(data: dict, out_dir: str):
    rows = data["rows"]
    labels = [shape_label(r["tile"]) for r in rows]
    bar_chart(labels, {"loss": [r["tail_mean"] for r in rows]}, f"mean loss of the last {data['tail']} steps",
              f"{data['model']}, {data['steps']} steps, lr {data['lr']}", out_dir, NAME,
              errors={"loss": ([r["tail_mean"] - r["tail_std"] for r in rows], [r["tail_mean"] + r["tail_std"] for r in rows])},
              baseline=rows[0]["tail_mean"])
    stride = max(1, data["steps"] // 30)
    xs = list(range(0, data["steps"], stride))
    line_chart(xs, {shape_label(r["tile"]): _smooth(r["losses"])[::stride] for r in rows}, "step", "loss (10-step mean)",
               "loss curves by tile shape", out_dir, NAME + "_curves")
    txt = text_table(("tile", "area", "loss (tail mean)", "std", "gap to first", "wall s", "tiles/step", "buckets", "kernel path"),
                     [(shape_label(r["tile"]), r["tile"][0] * r["tile"][1], r["tail_mean"], r["tail_std"], r["gap_to_reference"],
                       r["wall_s"], r["tiles_per_step"], r["buckets"], r["kernel_path"]) for r in rows])
    print(txt)
    write_text(out_dir, NAME + "_detail", txt)


def add_args(p):
    p.add_argument("--model", default="llama_220m")
    p.add_argument("--shapes", nargs="+", default=None, help="tile shapes as HxW (default: the 15 shapes of the sweep)")
    p.add_argument("--steps", type=int, default=300)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--seq", type=int, default=1024)
    p.add_argument("--lr", type=float, default=0.02)
    p.add_argument("--warmup-steps", type=int, default=20)
    p.add_argument("--decay-steps", type=int, default=60)
    p.add_argument("--tail", type=int, default=100, help="number of final steps whose loss is averaged")
    p.add_argument("--vocab", type=int, default=4096, help="tokens of the synthetic chain (capped by the model's vocabulary)")


def main(argv=None):
    return experiment_main(NAME, run, plot, add_args, argv, __doc__)


if __name__ == "__main__":
    main()
