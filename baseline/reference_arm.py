"""Benchmark arm that runs the UNMODIFIED reference package (``baseline/_ref/himuon``).

The reference's ``train_fsdp.py`` cannot run offline (it resolves the architecture through the HF Hub
and streams FineWeb), so this harness performs the same calls in the same order with an offline
``Qwen3Config`` and synthetic batches: HF ``AutoModelForCausalLM.from_config`` -> gradient checkpointing
(the script's default) -> bf16 -> ``wrap_with_banks(Qwen3BankScheme)`` -> one root ``fully_shard`` with the
bf16/bf16 mixed-precision policy -> ``release_pre_shard_refs`` -> ``get_optimizer("himuon")`` with
``cuda_graph=False`` (the script's FSDP default) -> WSD schedule -> the micro-step loop with
``set_requires_gradient_sync``.  None of this repository's models, kernels or engines are imported.
"""

from __future__ import annotations

import argparse
import os

LR, WD = 1e-2, 0.1


def _qwen3_config(name):
    from transformers import AutoConfig

    table = {
        "Qwen3-4B": dict(hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32,
                         num_key_value_heads=8, tie_word_embeddings=True),
        "Qwen3-0.6B": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                           num_key_value_heads=8, tie_word_embeddings=True),
    }
    kw = table[name]
    return AutoConfig.for_model("qwen3", vocab_size=151936, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                                max_position_embeddings=40960, hidden_act="silu", attention_bias=False,
                                use_cache=False, **kw)


def run(args, timed_region, host_batches, init_dist, barrier_sync):
    import torch
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, OffloadPolicy, fully_shard
    from transformers import AutoModelForCausalLM, get_wsd_schedule

    from himuon.fsdp_bank import Qwen3BankScheme, release_pre_shard_refs, wrap_with_banks   # the reference package
    from himuon.optim import get_optimizer
    from himuon.utils import seed_everything

    rank, world, local = init_dist(args.gpus)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device(f"cuda:{local}"))
    device = torch.device(f"cuda:{local}")
    seed_everything(42)
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    config = _qwen3_config(args.model)
    model = AutoModelForCausalLM.from_config(config)
    # the reference's train_fsdp.py enables gradient checkpointing by default (--gradient-checkpointing, on);
    # `--activation-checkpointing off` is its --no-gradient-checkpointing
    checkpointing = getattr(args, "activation_checkpointing", None) != "off"
    if checkpointing:
        model.gradient_checkpointing_enable()
    model.config.use_cache = False
    model.to(device=device, dtype=torch.bfloat16)
    model, banks = wrap_with_banks(model, Qwen3BankScheme(), world_size=world)
    mp_policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    fully_shard(model, mesh=mesh, mp_policy=mp_policy, offload_policy=OffloadPolicy())
    release_pre_shard_refs(banks)
    torch.cuda.empty_cache()
    ref_graph = bool(getattr(args, "reference_cuda_graph", False))
    opt_args = argparse.Namespace(lr=LR, weight_decay=WD, tile_size=args.tile, cuda_graph=ref_graph)
    optimizer = get_optimizer("himuon", model, opt_args)
    scheduler = get_wsd_schedule(optimizer, num_warmup_steps=100, num_stable_steps=0, num_decay_steps=400,
                                 num_training_steps=10000, min_lr_ratio=0.1, decay_type="cosine", warmup_type="linear")
    model.train()
    grad_acc = args.grad_acc
    n_total = args.warmup + args.steps
    hb = host_batches(config.vocab_size, n_total + 1 + args.steps, grad_acc, args.micro_batch, args.seq_len, rank)

    opt_events = []

    def train_step(batches, from_host):
        total = None
        for i, b in enumerate(batches):
            if from_host:
                b = {k: v.to(device, non_blocking=True) for k, v in b.items()}
            model.set_requires_gradient_sync(i == grad_acc - 1)
            out = model(input_ids=b["input_ids"], labels=b["labels"])
            loss = out.loss / grad_acc
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        optimizer.step()
        ev1.record()
        opt_events.append((ev0, ev1))
        scheduler.step()
        optimizer.zero_grad(set_to_none=not ref_graph)
        return total

    dev = [[{k: v.to(device) for k, v in mb.items()} for mb in step] for step in hb[:n_total]]
    for i in range(args.warmup):
        train_step(dev[i], False)
    tokens_per_step = args.micro_batch * args.seq_len * grad_acc * world
    opt_events.clear()
    ms = timed_region(lambda i: train_step(dev[args.warmup + i], False), args.steps)
    value = tokens_per_step * args.steps / (ms / 1e3)
    # device time of its own optimizer.step(), mean over the timed steps, max over ranks
    opt_ms = sum(a.elapsed_time(b) for a, b in opt_events) / max(1, len(opt_events))
    if world > 1:
        t = torch.tensor([opt_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        opt_ms = float(t.item())
    e2e = None
    if not args.no_e2e:
        float(train_step(hb[n_total], True).item())
        nbytes = sum(t.numel() * t.element_size() for mb in hb[n_total] for t in mb.values())
        losses = []
        ms2 = timed_region(lambda i: losses.append(float(train_step(hb[n_total + 1 + i], True).item())), args.steps)
        e2e = {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": nbytes,
               "d2h_bytes_per_step": 4, "ms_per_step": ms2 / args.steps, "last_loss": losses[-1]}
    out = None
    if rank == 0:
        out = {
            "impl": "reference",
            "metric": "tokens/s Qwen3-4B FSDP HiMuon @1/2/4/8 B200 (max over ranks); optimizer step ms",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": args.model, "global_batch": args.micro_batch * grad_acc * world, "seq_len": args.seq_len,
                       "parallelism": f"fsdp2-banks{world}", "optimizer": f"reference himuon tile {args.tile}, cuda_graph {'on' if ref_graph else 'off'}",
                       "activation_checkpointing": checkpointing},
            "optimizer_step_ms": opt_ms,
            "e2e": e2e, "gpu_launches": 0,
        }
    barrier_sync()
    dist.destroy_process_group()
    return out
