"""Worker run as gloo CPU ranks by tests/test_distributed_cpu.py (host-side logic of the engines)."""

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _cfg(layers=3):
    from himuon_b200.models import DecoderConfig

    return DecoderConfig(model_type="qwen3", vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=layers,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=8, tie_word_embeddings=True,
                         max_position_embeddings=64)


def _batches(rank, world, steps, grad_acc):
    g = torch.Generator().manual_seed(100 + rank)
    return [[{"input_ids": (ids := torch.randint(0, 64, (2, 16), generator=g)), "labels": ids} for _ in range(grad_acc)]
            for _ in range(steps)]


def scenario_train(mode, optimizer_name):
    """Sharded / data-parallel training over `world` CPU ranks must follow single-process training on the
    concatenated batch (same seed), which is what rank 0 recomputes here."""
    from himuon_b200.models import CausalLM
    from himuon_b200.optim import get_optimizer
    from himuon_b200.trainer import Trainer

    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    # "fsdp:<weights>:<grads>[:ckpt]" selects the engine's staging modes; 5 layers on 2 ranks give 3 layer groups, the last
    # one half empty, so the ring rotates and a pad layer takes part
    mode, *opts = mode.split(":")
    layers = 5 if opts else 3
    for o in opts:                         # "L7": another depth
        if o[:1] == "L" and o[1:].isdigit():
            layers = int(o[1:])
    model = CausalLM(_cfg(layers))
    if "ckpt" in opts:
        model.gradient_checkpointing_enable()
    if mode == "fsdp":
        from himuon_b200.parallel.fsdp import ShardedEngine
        engine = ShardedEngine(model, use_banks=True, weights=opts[0] if opts else None,
                               grads=opts[1] if len(opts) > 1 else "replicated", debug="debug" in opts)
        if opts and world > 1:
            assert engine.weights_mode == opts[0] and engine.grads_mode == opts[1]
            assert engine.uses_fences == (opts[0] == "ring" or opts[1] == "sharded")
            b = engine.bank_bytes()
            # this rank holds its 1/world share plus the staging slots, not the whole banks
            groups = engine.n_groups
            if opts[0] == "ring":
                assert b["weights"] <= (1.0 / world + 2.0 / groups) * b["banks_padded"] + 1, b
            if opts[1] == "sharded":
                assert b["grads"] <= (1.0 / world + 1.0 / groups) * b["banks_padded"] + 1, b
    else:
        from himuon_b200.parallel.ddp import DataParallelEngine
        engine = DataParallelEngine(model, bucket_layers=2, overlap="overlap" in opts)
        assert engine.overlap == (world > 1 and "overlap" in opts) and engine.n_buckets == -(-layers // 2)
    ns = argparse.Namespace(lr=0.02, weight_decay=0.1, tile_size=16, cuda_graph=False)
    opt = get_optimizer(optimizer_name, model, ns)
    if mode == "fsdp":
        engine.attach_optimizer(opt)
    trainer = Trainer(model, opt, None, engine, grad_acc=2, device=torch.device("cpu"))
    losses = [float(trainer.train_step(b)) for b in _batches(rank, world, 3, 2)]
    all_losses = [None] * world
    dist.all_gather_object(all_losses, losses)
    sd = engine.full_state_dict() if mode == "fsdp" else {k: v.detach().clone() for k, v in model.state_dict().items()}
    if mode == "ddp" and engine.overlap:     # every optimizer step reduced all buckets from inside its last backward pass
        assert engine.overlapped_launches == 3 * engine.n_buckets, engine.overlapped_launches
    if mode == "fsdp" and opts and world > 1:
        groups = engine.n_groups
        if opts[0] == "ring":
            # 3 steps x 2 micro-batches, forward and backward.  With more groups than slots every step's first forward
            # fetches all groups and every backward re-fetches all but the last two; the second micro-batch finds
            # groups 0 and 1 still staged from the first one's backward.
            per_step = (groups + max(0, groups - 2)) + (max(0, groups - 2) + max(0, groups - 2)) if groups > 2 else groups
            assert engine.ring_fetches == 3 * per_step, (engine.ring_fetches, groups)
        if opts[1] == "sharded":
            assert engine.group_reductions == 3 * 2 * groups, engine.group_reductions
    if rank == 0:
        torch.manual_seed(0)
        ref_model = CausalLM(_cfg(layers))
        ref_opt = get_optimizer(optimizer_name if optimizer_name != "muon-fsdp" else "muon", ref_model, ns)
        per_rank = [_batches(r, world, 3, 2) for r in range(world)]
        ref_losses = []
        for s in range(3):
            tot = 0.0
            for mb in range(2):
                for r in range(world):
                    b = per_rank[r][s][mb]
                    loss = ref_model(b["input_ids"], labels=b["labels"]).loss
                    (loss / (2 * world)).backward()
                    tot += float(loss)
            ref_opt.step()
            ref_opt.zero_grad()
            ref_losses.append(tot / (2 * world))
        mean_losses = [sum(l[s] for l in all_losses) / world for s in range(3)]
        for a, b in zip(mean_losses, ref_losses):
            assert abs(a - b) < 2e-3, (mean_losses, ref_losses)
        ref_sd = ref_model.state_dict()
        assert set(sd) == set(ref_sd), sorted(set(sd) ^ set(ref_sd))
        worst = max(float((sd[k].float() - ref_sd[k].float()).abs().max()) for k in ref_sd)
        assert worst < 5e-3, worst
        print(f"PARITY OK {mode} {optimizer_name} worst={worst:.2e}", flush=True)
    engine.close()


def scenario_dtensor():
    """HiMuon on a DTensor bank sharded on the layer axis (what torch FSDP2 produces) against per-matrix HiMuon on one
    process, with injected gradients: divisible and zero-padded tiles (reference: tests/integration/_fsdp_worker.py)."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    from himuon_b200.optimizers import HiMuon

    rank, world = dist.get_rank(), dist.get_world_size()
    mesh = init_device_mesh("cpu", (world,))
    for (H, W) in ((64, 96), (50, 75)):
        torch.manual_seed(0)
        full = torch.randn(8, H, W) * 0.02
        bank = torch.nn.Parameter(distribute_tensor(full.clone(), mesh, [Shard(0)]))
        opt = HiMuon([bank], tile_size=32, cuda_graph=False, lr=0.02)
        mats = [torch.nn.Parameter(full[i].clone()) for i in range(8)]
        ref_opt = HiMuon(mats, tile_size=32, cuda_graph=False, lr=0.02)
        assert opt._has_dtensor_muon()
        for s in range(4):
            g = torch.randn(8, H, W, generator=torch.Generator().manual_seed(s))
            bank.grad = distribute_tensor(g.clone(), mesh, [Shard(0)])
            for i, m in enumerate(mats):
                m.grad = g[i].clone()
            opt.step()
            ref_opt.step()
        got = bank.detach().full_tensor()
        want = torch.stack([m.detach() for m in mats])
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), (got - want).abs().max()
    if rank == 0:
        print("PARITY OK dtensor", flush=True)


def scenario_missing_rank():
    """A rank that never joins: the others' collective ends with an error instead of hanging."""
    rank = dist.get_rank()
    if rank == dist.get_world_size() - 1:
        print("rank leaves between steps", flush=True)
        return
    try:
        t = torch.ones(4)
        dist.all_reduce(t)
        print("UNEXPECTED completion", flush=True)
    except Exception as e:
        print(f"DETECTED {type(e).__name__}", flush=True)


if __name__ == "__main__":
    scenario, mode, optname = sys.argv[1], sys.argv[2], sys.argv[3]
    import datetime
    timeout = datetime.timedelta(seconds=8 if scenario == "missing" else 120)
    dist.init_process_group("gloo", timeout=timeout)
    if scenario == "train":
        scenario_train(mode, optname)
    elif scenario == "dtensor":
        scenario_dtensor()
    else:
        scenario_missing_rank()
    if scenario != "missing":
        dist.barrier()
        dist.destroy_process_group()
