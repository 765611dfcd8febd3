#!/usr/bin/env python
"""Headline benchmark: training tokens/s of Qwen3-4B with bank-sharded parameters and the HiMuon optimizer.

Configuration (fixed, weak scaling): Qwen3-4B (36 layers, hidden 2560, 32 Q / 8 KV heads, head_dim 128,
SwiGLU 9728, vocab 151936), bf16, sequence 1024, micro-batch 2 per GPU, gradient accumulation 8,
HiMuon tile 512 (lr 1e-2, wd 0.1) with the AdamW fallback, uniform-random tokens, random init.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Rank 0 prints one JSON line.  ``value`` is timed on the device (CUDA events around exactly K optimizer
steps, barrier + synchronize on both sides, maximum over ranks) with the step's inputs already on the
device; ``e2e`` repeats the measurement through the public ``Trainer.train_step`` call with the
host->device copy of every micro-batch from pinned memory and the device->host read of the loss inside
the timed region.  Every step streams > 8 GB of weights, far more than the 126 MB L2, so no explicit L2
flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = "Qwen3-4B"
SEQ_LEN = 1024
MICRO_BATCH = 2
GRAD_ACC = 8
TILE = 512
LR, WD = 1e-2, 0.1


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--model", type=str, default=MODEL, help="architecture name (the headline number uses the default)")
    p.add_argument("--seq-len", type=int, default=SEQ_LEN)
    p.add_argument("--micro-batch", type=int, default=MICRO_BATCH)
    p.add_argument("--grad-acc", type=int, default=GRAD_ACC)
    p.add_argument("--tile", type=int, default=TILE)
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--peer-weights", action="store_true",
                   help="no gathered copy of the banks: the GEMMs read weight tiles from the owner rank over NVLink")
    p.add_argument("--fsdp-weights", type=str, default="gathered", choices=["gathered", "ring", "peer"],
                   help="bank working copy: full gathered copy (default), two-slot staging ring, or peer reads")
    p.add_argument("--fsdp-grads", type=str, default="replicated", choices=["replicated", "sharded"],
                   help="bank gradient accumulation: full buffer per rank (default) or per-group reduce-scatter")
    p.add_argument("--grad-prefetch", action="store_true",
                   help="sharded engine: pull the peers' gradient replicas with the copy engines during the last "
                        "micro-batch's backward pass instead of leaving them to momentum_tile's peer loads")
    p.add_argument("--nvls", action="store_true",
                   help="gradient reductions through the NVLink switch (multimem) instead of peer loads")
    p.add_argument("--ddp-overlap", action="store_true",
                   help="data-parallel engine: per-bucket all-reduces on a side stream beside the backward pass instead of "
                        "one full-grid all-reduce after it (the default)")
    p.add_argument("--ddp-serial", action="store_true",
                   help="data-parallel engine: one all-reduce after backward instead of per-bucket all-reduces beside it")
    p.add_argument("--ddp-comm-blocks", type=int, default=16, help="grid cap of the overlapped bucket all-reduces")
    p.add_argument("--no-step-graph", action="store_true",
                   help="run forward/backward eagerly instead of replaying the captured micro-batch CUDA graphs")
    p.add_argument("--engine", type=str, default="fsdp", choices=["fsdp", "ddp"],
                   help="fsdp: bank-sharded engine (headline); ddp: replicated parameters + fused all-reduce")
    p.add_argument("--optimizer", type=str, default="himuon", help="himuon | muon-fsdp | muon | adamw (headline: himuon)")
    p.add_argument("--activation-checkpointing", type=str, default=None, choices=["on", "off"],
                   help="per-layer recomputation in backward, honoured by both arms.  Default: each arm's own stock "
                        "setting (ours off, the reference's train_fsdp.py default on); pass the same value to both "
                        "arms for a like-for-like comparison")
    p.add_argument("--reference-cuda-graph", action="store_true",
                   help="reference arm only: construct its HiMuon with cuda_graph=True (its FSDP default is False)")
    return p.parse_args()


def init_dist(n_gpus):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    return rank, world, local


def barrier_sync():
    import torch
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


def timed_region(step_fn, k):
    """CUDA-event time of exactly k calls of step_fn, barrier + synchronize on both sides; max over ranks (ms)."""
    import torch

    from himuon_b200.utils import max_over_ranks

    barrier_sync()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(k):
        step_fn(i)
    end.record()
    barrier_sync()
    return max_over_ranks(start.elapsed_time(end))


def host_batches(vocab, n_steps, grad_acc, micro_batch, seq_len, rank, seed=0, pinned=True):
    import torch

    out = []
    g = torch.Generator().manual_seed(seed + 1000 * rank)
    for _ in range(n_steps):
        step = []
        for _ in range(grad_acc):
            ids = torch.randint(0, vocab, (micro_batch, seq_len), generator=g, dtype=torch.long)
            if pinned:
                ids = ids.pin_memory()
            step.append({"input_ids": ids, "labels": ids})
        out.append(step)
    return out


def run_ours(args):
    import torch

    from himuon_b200 import ops
    from himuon_b200.models import CausalLM, get_config
    from himuon_b200.optim import get_optimizer
    from himuon_b200.parallel.fsdp import ShardedEngine
    from himuon_b200.trainer import Trainer, wsd_schedule
    from himuon_b200.utils import ClockSampler, seed_everything

    rank, world, local = init_dist(args.gpus)
    device = torch.device(f"cuda:{local}")
    seed_everything(42)
    cfg = get_config(args.model)
    with torch.device(device):
        model = CausalLM(cfg).to(torch.bfloat16)
    checkpointing = args.activation_checkpointing == "on"
    if checkpointing:
        model.gradient_checkpointing_enable()
    if args.engine == "fsdp":
        weights = "peer" if args.peer_weights else args.fsdp_weights
        engine = ShardedEngine(model, use_banks=args.optimizer in ("himuon", "muon-fsdp", "adamw"), weights=weights,
                               grads=args.fsdp_grads, nvls=args.nvls,
                               grad_prefetch=args.grad_prefetch)
    else:
        from himuon_b200.parallel.ddp import DataParallelEngine
        engine = DataParallelEngine(model, nvls=args.nvls, overlap=args.ddp_overlap and not args.ddp_serial, comm_blocks=args.ddp_comm_blocks)
    ns = argparse.Namespace(lr=LR if args.optimizer != "adamw" else 1e-3, weight_decay=WD, tile_size=args.tile, cuda_graph=True,
                            cuda_graph_warmup=1)
    optimizer = get_optimizer(args.optimizer, model, ns)
    if args.engine == "fsdp":
        engine.attach_optimizer(optimizer)
    scheduler = wsd_schedule(optimizer, 100, 0, 400, 0.1)
    trainer = Trainer(model, optimizer, scheduler, engine, args.grad_acc, device,
                      graph_microbatch=not args.no_step_graph, graph_warmup_steps=min(2, max(1, args.warmup - 1)))
    trainer.zero_set_to_none = False
    model.train()

    n_total = args.warmup + args.steps
    hb = host_batches(cfg.vocab_size, n_total + 1 + args.steps, args.grad_acc, args.micro_batch, args.seq_len, rank)
    dev_batches = [[{k: v.to(device) for k, v in mb.items()} for mb in step] for step in hb[:n_total]]
    for i in range(args.warmup):
        trainer.train_step(dev_batches[i])
    torch.cuda.synchronize()
    ops.check_status()

    tokens_per_step = args.micro_batch * args.seq_len * args.grad_acc * world
    launches0 = ops.launch_count()
    with ClockSampler(index=local) as clocks:
        ms = timed_region(lambda i: trainer.train_step(dev_batches[args.warmup + i]), args.steps)
    launches = ops.launch_count() - launches0
    ops.check_status()
    value = tokens_per_step * args.steps / (ms / 1e3)

    # optimizer step alone (device time of one step on the zeroed gradients left by the last step, max over ranks)
    from himuon_b200.utils import max_over_ranks
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    engine.finish_backward()
    barrier_sync()
    ev0.record()
    optimizer.step()
    ev1.record()
    barrier_sync()
    opt_ms = max_over_ranks(ev0.elapsed_time(ev1))
    engine.zero_grad(set_to_none=False)

    e2e = None
    if not args.no_e2e:
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        trainer.read_loss(trainer.train_step(hb[n_total]))      # one untimed pass through the host path
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        losses = []

        def e2e_step(i):
            losses.append(trainer.read_loss(trainer.train_step(hb[n_total + 1 + i])))

        ms_e2e = timed_region(e2e_step, args.steps)
        e2e = {"value": tokens_per_step * args.steps / (ms_e2e / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": trainer.h2d_bytes // args.steps, "d2h_bytes_per_step": trainer.d2h_bytes // args.steps,
               "ms_per_step": ms_e2e / args.steps, "last_loss": losses[-1]}
    # Where a step goes: device time per phase (CUDA events) over two more steps, outside the timed regions, as the
    # maximum and the minimum over ranks.  grad_reduce and regather_reset wait for the other ranks, so their maximum
    # holds the time the fastest rank waited for the slowest (already counted in the slowest rank's forward_backward)
    # and their minimum, seen by the rank that arrived last, is the communication not hidden behind compute.
    from himuon_b200.utils import PhaseTimer
    trainer.phases = PhaseTimer(True, device)
    n_phase = 2
    for i in range(n_phase):
        trainer.train_step(dev_batches[args.warmup + (i % args.steps)])
    phases = {k: round(v / n_phase, 3) for k, v in trainer.phases.summary().items()}
    phases_min = {k: round(v / n_phase, 3) for k, v in trainer.phases.summary(reduce="min").items()}
    trainer.phases = PhaseTimer(False)
    ops.check_status()
    if rank == 0:
        out = {
            "metric": "tokens/s Qwen3-4B FSDP HiMuon @1/2/4/8 B200 (max over ranks); optimizer step ms",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": args.model, "global_batch": args.micro_batch * args.grad_acc * world,
                       "seq_len": args.seq_len, "micro_batch_per_gpu": args.micro_batch, "grad_acc": args.grad_acc,
                       "parallelism": (f"fsdp-banks{world}" + (f" weights={engine.weights_mode} grads={engine.grads_mode}" + (" nvls" if engine.nvls else "") + (" grad-prefetch" if engine.grad_prefetch else "") if world > 1 else "")) if args.engine == "fsdp" else f"dp{world}" + ("" if world == 1 else (" overlapped bucket all-reduce" if engine.overlap else " serial all-reduce")),
                       "optimizer": f"{args.optimizer} tile {args.tile}, lr {ns.lr}, wd {WD}, cuda graph",
                       "forward_backward": "eager" if args.no_step_graph else "micro-batch CUDA graphs (public Trainer option)",
                       "activation_checkpointing": checkpointing,
                       "l2": "no flush: each step streams >8 GB of weights and activations (L2 is 126 MB)"},
            "optimizer_step_ms": opt_ms, "phases_ms_per_step": phases,
            "phases_min_over_ranks_ms_per_step": phases_min,
            "exposed_comm_ms_per_step": round(phases_min.get("grad_reduce", 0.0) + phases_min.get("regather_reset", 0.0), 3),
            "rank_skew_ms_per_step": round(phases.get("grad_reduce", 0.0) - phases_min.get("grad_reduce", 0.0), 3),
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": launches, "impl": "ours",
        }
        print(json.dumps(out), flush=True)
    engine.close()
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


def run_reference(args):
    """The unmodified reference (installed under baseline/_ref) on the same configuration, through its own
    public API: HF model -> wrap_with_banks -> FSDP2 fully_shard -> get_optimizer('himuon') -> train loop as in
    its train_fsdp.py (stock defaults: gradient checkpointing on, cuda_graph off)."""
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
    except Exception as e:
        print(json.dumps({"impl": "reference", "unavailable": f"reference harness cannot be imported: {e}"[:300]}), flush=True)
        return
    try:
        out = reference_arm.run(args, timed_region, host_batches, init_dist, barrier_sync)
    except Exception as e:
        out = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:400]}
        rank = int(os.environ.get("RANK", "0"))
        if rank != 0:
            return
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
