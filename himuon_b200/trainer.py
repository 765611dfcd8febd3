"""Training-loop glue shared by ``train.py``, ``train_ddp.py`` and ``train_fsdp.py``.

The reference inlines the same loop three times (``train.py:14-170``, ``train_ddp.py:19-241``,
``train_fsdp.py:36-302``); here it is one module with three execution modes:

* ``single`` - one process, one device;
* ``ddp``    - replicated parameters, gradients all-reduced by the fused NVLink kernels of
  :mod:`himuon_b200.parallel.ddp` (``no_sync`` semantics on accumulation micro-steps);
* ``fsdp``   - parameter banks sharded on the layer axis by :mod:`himuon_b200.parallel.fsdp`
  when the optimizer is ``himuon`` or ``muon-fsdp``.

Flags, defaults, metric line, reconfigure schedule, stop-flag broadcast, time budget and the
end-of-run Hugging Face checkpoint follow the reference scripts.  ``--dataset synthetic`` selects
uniform-random tokens (no network); ``--dtype`` picks the parameter dtype.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import time
from contextlib import nullcontext
from datetime import datetime

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader

from .dataset import SyntheticTokenDataset, ToyDataset
from .model import count_model_parameters, count_num_training_tokens, get_model_and_tokenizer
from .optim import get_optimizer
from .utils import PhaseTimer, TimeBudget, merge_kv_args, seed_everything


# ------------------------------------------------------------------------------------------- CLI
def build_arg_parser(mode: str) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=f"himuon_b200 training ({mode})")
    p.add_argument("--model", type=str, default="Qwen3-0.6B")
    p.add_argument("-d", "--dataset", type=str, default="sample-10BT",
                   help="FineWeb subset name, or 'synthetic' for uniform-random tokens")
    p.add_argument("--optimizer", "--opt", dest="optimizer", type=str, default="adamw")
    p.add_argument("--learning-rate", "--lr", dest="lr", type=float, default=None)
    p.add_argument("--weight-decay", "--wd", dest="weight_decay", type=float, default=None)
    p.add_argument("--batch-size", "--bs", dest="batch_size", type=int, default=16)
    p.add_argument("--gradient-accumulation-steps", "--grad-acc", dest="gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--max-length", type=int, default=1024)
    p.add_argument("--num-training-steps", "--steps", dest="num_training_steps", type=int, default=None)
    p.add_argument("--num-warmup-steps", type=int, default=100)
    p.add_argument("--reconfigure-schedule", type=str, default=None,
                   help='JSON list such as \'[{"step": 0, "tile_size": 1000000000}, {"step": 200, "tile_size": 512}]\'')
    p.add_argument("--cuda-graph", dest="cuda_graph", action=argparse.BooleanOptionalAction,
                   default=(mode != "fsdp"))
    p.add_argument("--cuda-graph-step", dest="cuda_graph_step", action="store_true",
                   help="replay forward+backward of each micro-batch from captured CUDA graphs (static batch shapes)")
    p.add_argument("--time-budget", type=float, default=None, help="hours")
    p.add_argument("--eval-interval", type=int, default=0)
    p.add_argument("--eval-steps", type=int, default=10)
    p.add_argument("--eval-dataset", type=str, default="CC-MAIN-2024-51")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--wandb", action="store_true")
    p.add_argument("--save-checkpoint", action="store_true")
    p.add_argument("--run-name", type=str, default=None)
    p.add_argument("--kwargs", nargs="*", default=[], help="extra key=value pairs merged into the arguments")
    p.add_argument("--dtype", type=str, default=None, choices=["bf16", "fp32"],
                   help="parameter dtype (default: bf16 on CUDA, fp32 on CPU)")
    p.add_argument("--device", type=str, default=None)
    if mode == "ddp":
        p.add_argument("--ddp-overlap", dest="ddp_overlap", action="store_true",
                       help="start per-bucket all-reduces from inside the last backward pass (side stream) instead of one "
                            "full-grid all-reduce after it")
    if mode in ("ddp", "fsdp"):
        p.add_argument("--nvls", action="store_true",
                       help="bind the gradient heap to an NVLink multicast object and reduce through the switch (multimem)")
        p.add_argument("--time-stats", action="store_true")
        p.add_argument("--gradient-checkpointing", dest="gradient_checkpointing",
                       action=argparse.BooleanOptionalAction, default=True)
    if mode == "fsdp":
        p.add_argument("--num-decay-steps", type=int, default=400)
        p.add_argument("--min-lr-ratio", type=float, default=0.1)
        p.add_argument("--cpu-offload", action="store_true",
                       help="keep the optimizer state in pinned host memory between steps")
        p.add_argument("--fsdp-weights", dest="fsdp_weights", type=str, default="gathered",
                       choices=["gathered", "ring", "peer"],
                       help="working copy of the parameter banks: a full gathered copy refreshed once per step, a "
                            "two-slot staging ring of layer groups fetched from the owners during forward/backward, or "
                            "none (the GEMMs read the owner's shard over NVLink)")
        p.add_argument("--fsdp-grads", dest="fsdp_grads", type=str, default="replicated", choices=["replicated", "sharded"],
                       help="gradient accumulation: full-bank buffer per rank reduced once per step, or per-layer-group "
                            "reduce-scatter onto the owner's shard-sized accumulator")
        p.add_argument("--peer-weights", dest="peer_weights", action="store_true",
                       help="same as --fsdp-weights peer")
        p.add_argument("--grad-prefetch", dest="grad_prefetch", action="store_true",
                       help="pull the peers' gradient replicas with the copy engines during the last micro-batch's "
                            "backward pass (HiMuon otherwise reads them over NVLink inside the optimizer step)")
    return p


# ------------------------------------------------------------------------------------------- schedules
def cosine_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int):
    """Linear warm-up then half-cosine decay to zero (HF ``get_cosine_schedule_with_warmup``)."""
    def lr_lambda(step):
        if step < num_warmup_steps:
            return step / max(1, num_warmup_steps)
        progress = (step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps)
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * progress)))
    return torch.optim.lr_scheduler.LambdaLR(optimizer, lr_lambda)


def wsd_schedule(optimizer, num_warmup_steps: int, num_stable_steps: int, num_decay_steps: int, min_lr_ratio: float):
    """Warm-up / stable / cosine-decay schedule; stays at ``min_lr_ratio`` afterwards (``train_fsdp.py:168-177``)."""
    def lr_lambda(step):
        if step < num_warmup_steps:
            return step / max(1, num_warmup_steps)
        if step < num_warmup_steps + num_stable_steps:
            return 1.0
        if step < num_warmup_steps + num_stable_steps + num_decay_steps:
            progress = (step - num_warmup_steps - num_stable_steps) / max(1, num_decay_steps)
            return min_lr_ratio + (1.0 - min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * progress))
        return min_lr_ratio
    return torch.optim.lr_scheduler.LambdaLR(optimizer, lr_lambda)


def parse_reconfigure_schedule(text: str | None) -> dict[int, dict]:
    if not text:
        return {}
    entries = json.loads(text)
    out: dict[int, dict] = {}
    for e in entries:
        e = dict(e)
        step = int(e.pop("step"))
        out.setdefault(step, {}).update(e)
    return out


def make_apply_reconfigure(optimizer, schedule: dict[int, dict], log):
    """Closure applied at step 0 (before training) and after every optimizer step (``train.py:91-110``)."""
    def apply(step: int):
        if step not in schedule or not hasattr(optimizer, "reconfigure"):
            return
        updates = schedule[step]
        old = {k: optimizer.param_groups[0].get(k) for k in updates}
        optimizer.reconfigure(**updates)
        new = {k: optimizer.param_groups[0].get(k) for k in updates}
        log(f"[reconfigure @ step {step}] {old} -> {new}")
    return apply


# ------------------------------------------------------------------------------------------- data
def build_dataloader(args, tokenizer, vocab_size, rank, world_size, eval_split=False):
    name = args.eval_dataset if eval_split else args.dataset
    if str(name).lower() == "synthetic" or str(args.dataset).lower() == "synthetic":
        ds = SyntheticTokenDataset(vocab_size, args.max_length, seed=args.seed + (7919 if eval_split else 0),
                                   rank=rank, world_size=world_size)
    else:
        try:
            from datasets import load_dataset

            raw = load_dataset("HuggingFaceFW/fineweb", name=name, split="train", streaming=True)
            raw = raw.shuffle(seed=args.seed)
            if world_size > 1:
                raw = raw.shard(num_shards=world_size, index=rank)
        except Exception as e:  # offline machines
            raise RuntimeError(f"cannot stream FineWeb subset {name!r} ({e}); pass --dataset synthetic for "
                               "uniform-random tokens") from e
        ds = ToyDataset(raw, tokenizer, max_length=args.max_length)
    return DataLoader(ds, batch_size=args.batch_size, num_workers=0, pin_memory=torch.cuda.is_available())


# ------------------------------------------------------------------------------------------- trainer
class Trainer:
    """One optimizer step = ``grad_acc`` micro-batches through forward/backward + optimizer.

    ``train_step(host_batches)`` is the public per-step call: it copies each micro-batch from
    (pinned) host memory, runs the step on the configured engine and returns the mean loss as a
    device scalar; ``float(loss)`` is the only device-to-host read.
    """

    def __init__(self, model, optimizer, scheduler=None, engine=None, grad_acc: int = 1, device=None,
                 autocast_dtype=None, graph_microbatch: bool = False, graph_warmup_steps: int = 2,
                 phase_timing: bool = False):
        self.model, self.optimizer, self.scheduler, self.engine = model, optimizer, scheduler, engine
        self.grad_acc = int(grad_acc)
        self.device = device if device is not None else next(model.parameters()).device
        self.autocast_dtype = autocast_dtype
        self.zero_set_to_none = not bool(getattr(optimizer, "_cuda_graph_enabled", False))
        if hasattr(model, "set_loss_scale"):
            model.set_loss_scale(1.0 / self.grad_acc)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # per-phase device time (CUDA events) of every step when enabled; the phases are NVTX ranges either way
        self.phases = PhaseTimer(phase_timing, self.device if self.device.type == "cuda" else None)
        # Optional: forward+backward of one micro-batch replayed from a CUDA graph (removes ~30k kernel launches'
        # worth of host work per step).  Two graphs are captured after `graph_warmup_steps` eager steps: one for
        # the first micro-batch of a step (weight gradients overwrite) and one for the others (they accumulate).
        # Needs static shapes and gradients that are zeroed in place, never dropped.
        self.graph_microbatch = bool(graph_microbatch) and self.device.type == "cuda"
        self.graph_warmup_steps = int(graph_warmup_steps)
        self._steps_done = 0
        self._mb_graphs = {}          # (first, own graph for the sync step) -> (graph, static loss, launches, sinks written, engine state)
        self._mb_static = None
        self._mb_pool = None
        if self.graph_microbatch:
            self.zero_set_to_none = False

    # ------------------------------------------------------------------ micro-batch forward + backward
    def _eager_microbatch(self, batch, sync: bool) -> torch.Tensor:
        ctx = self.engine.no_sync() if (self.engine is not None and not sync) else nullcontext()
        with ctx:
            loss = self.model(batch["input_ids"], labels=batch["labels"]).loss
            (loss / self.grad_acc).backward()
        return loss.detach()

    def _graph_microbatch(self, batch, first: bool, sync: bool) -> torch.Tensor:
        from . import ops

        ids, labels = batch["input_ids"], batch["labels"]
        usable = (self._steps_done >= self.graph_warmup_steps and self.model.training and not self.zero_set_to_none
                  and (self._mb_static is None or (self._mb_static["input_ids"].shape == ids.shape
                                                   and self._mb_static["labels"].shape == labels.shape)))
        if not usable:
            return self._eager_microbatch(batch, sync)
        if self._mb_static is None:
            self._mb_static = {"input_ids": torch.empty_like(ids), "labels": torch.empty_like(labels)}
        self._mb_static["input_ids"].copy_(ids)
        self._mb_static["labels"].copy_(labels)
        # an engine whose synchronising micro-step differs from the accumulating ones (it starts collectives from
        # inside backward) gets a graph of its own for it
        key = (first, bool(sync and getattr(self.engine, "graph_key_sync", False)))
        entry = self._mb_graphs.get(key)
        if entry is None:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            n0 = ops.launch_count()
            ops.GradSink.start_log()
            ctx = self.engine.no_sync() if (self.engine is not None and not sync) else nullcontext()
            try:
                with ctx, torch.cuda.graph(graph, pool=self._mb_pool):
                    loss = self.model(self._mb_static["input_ids"], labels=self._mb_static["labels"]).loss
                    (loss / self.grad_acc).backward()
                    static_loss = loss.detach()
            finally:
                written = ops.GradSink.stop_log()
            self._mb_pool = graph.pool()
            # the capture ran the wrappers once (launches counted); it also tells which gradient sinks a replay writes
            # and what host-side state the engine's hooks left behind
            state = self.engine.graph_capture_state() if hasattr(self.engine, "graph_capture_state") else None
            entry = (graph, static_loss, ops.launch_count() - n0, written, state)
            self._mb_graphs[key] = entry
        else:
            ops.add_launches(entry[2])
        entry[0].replay()
        for ref_sink in entry[3]:
            sink = ref_sink()
            if sink is not None:
                sink.fresh = False
        if entry[4] is not None:
            self.engine.graph_replay_state(entry[4])
        return entry[1].clone()

    def _to_device(self, batch):
        out = {}
        for k, v in batch.items():
            if torch.is_tensor(v):
                self.h2d_bytes += v.numel() * v.element_size()
                out[k] = v.to(self.device, non_blocking=True)
        return out

    def train_step(self, host_batches) -> torch.Tensor:
        assert len(host_batches) == self.grad_acc
        total = None
        ph = self.phases
        for i, hb in enumerate(host_batches):
            with ph.phase("h2d"):
                batch = self._to_device(hb)
            sync = i == self.grad_acc - 1
            with ph.phase("forward_backward"):
                if self.graph_microbatch:
                    loss = self._graph_microbatch(batch, first=(i == 0), sync=sync)
                else:
                    loss = self._eager_microbatch(batch, sync)
            total = loss if total is None else total + loss
        if self.engine is not None:
            with ph.phase("grad_reduce"):
                self.engine.finish_backward()
        with ph.phase("optimizer"):
            self.optimizer.step()
        if self.scheduler is not None:
            self.scheduler.step()
        with ph.phase("regather_reset"):
            if self.engine is not None:
                self.engine.zero_grad(set_to_none=self.zero_set_to_none)
            else:
                self.optimizer.zero_grad(set_to_none=self.zero_set_to_none)
        self._steps_done += 1
        return total / self.grad_acc

    def read_loss(self, loss: torch.Tensor) -> float:
        """Device-to-host read of the step's loss.  The read synchronises with the device anyway, so the kernels'
        status word is checked here too: a bounded wait that ran out (a GEMM / attention / Newton-Schulz barrier, a
        peer-flag handshake of a collective) leaves invalid results behind, and training must stop, not diverge."""
        self.d2h_bytes += loss.numel() * loss.element_size()
        value = float(loss.item())
        self.check_device_status()
        return value

    def device_status(self) -> int:
        """The sticky status word of this rank's kernels (0 = healthy); no synchronisation beyond the read itself."""
        if self.device.type != "cuda":
            return 0
        from . import _ext
        return int(_ext.ext().status(False))

    def check_device_status(self) -> None:
        code = self.device_status()
        if code:
            raise RuntimeError(f"himuon_b200: a device-side wait timed out on this rank (status code {code}); "
                               "gradients and parameters of this step are invalid")

    @torch.no_grad()
    def evaluate(self, batches, steps: int | None = None) -> float:
        """Mean loss over fixed evaluation batches (a list collected once, as the reference does,
        ``train_fsdp.py:147-166``), averaged over the ranks.  Runs under ``no_grad`` in eval mode: no gradient
        buffer, sink or optimizer state is touched, so a training step after it is unaffected."""
        if not isinstance(batches, (list, tuple)):          # an iterator: draw `steps` batches from it
            batches = [next(batches) for _ in range(int(steps or 0))]
        elif steps is not None:
            batches = batches[:steps]
        was_training = self.model.training
        self.model.eval()
        tot = torch.zeros((), device=self.device, dtype=torch.float32)
        try:
            for hb in batches:
                batch = self._to_device(hb)
                tot += self.model(batch["input_ids"], labels=batch["labels"]).loss.float()
        finally:
            self.model.train(was_training)
        tot /= max(1, len(batches))
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
            tot /= dist.get_world_size()
        return float(tot.item())


# ------------------------------------------------------------------------------------------- main loop
def run_training(args, mode: str) -> dict:
    args = merge_kv_args(args)
    seed_everything(args.seed)
    distributed = mode in ("ddp", "fsdp")
    rank, world_size, local_rank = 0, 1, 0
    if distributed:
        local_rank = int(os.environ.get("LOCAL_RANK", 0))
        use_cuda = torch.cuda.is_available() and (args.device or "cuda").startswith("cuda")
        if not dist.is_initialized():
            dist.init_process_group("nccl" if use_cuda else "gloo")
        rank, world_size = dist.get_rank(), dist.get_world_size()
        device = torch.device(f"cuda:{local_rank}") if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(device)
    else:
        device = torch.device(args.device) if args.device else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, None: torch.bfloat16 if device.type == "cuda" else torch.float32}[args.dtype]

    tag = {"single": "", "ddp": "ddp_", "fsdp": "fsdp2_"}[mode]
    default_lr = args.lr if args.lr is not None else {"adamw": 1e-3}.get(args.optimizer.lower(), None)
    run_name = args.run_name or f"{args.model}_{tag}{args.optimizer}_lr{default_lr}_{datetime.now().strftime('%Y%m%d_%H%M%S')}"
    is_main = rank == 0
    if args.wandb and is_main:
        from .logger import WandbLogger
        logger = WandbLogger(vars(args), run_name)
    elif is_main:
        from .logger import LoguruLogger
        logger = LoguruLogger(run_name)
    else:
        logger = None

    def log(msg):
        if logger is not None:
            logger.info(msg)

    model, tokenizer = get_model_and_tokenizer(args.model)
    if getattr(args, "gradient_checkpointing", False):
        model.gradient_checkpointing_enable()
    model.config.use_cache = False
    model = model.to(device=device, dtype=dtype)
    n_params, n_str = count_model_parameters(model)
    log(f"Model {args.model}: {n_str}")

    engine, banks = None, None
    if mode == "ddp":
        from .parallel.ddp import DataParallelEngine
        engine = DataParallelEngine(model, nvls=bool(getattr(args, "nvls", False)),
                                    overlap=bool(getattr(args, "ddp_overlap", False)))
    elif mode == "fsdp":
        from .parallel.fsdp import ShardedEngine
        # Banks (whole matrices sharded on the layer axis) serve every optimizer that updates a stacked (n, H, W)
        # parameter correctly: himuon, muon-fsdp, and adamw, which is element-wise.  The others (muon, himuon-legacy,
        # soap) need one 2-D parameter per matrix and run replicated.
        opt_name = args.optimizer.lower()
        use_banks = opt_name in ("himuon", "muon-fsdp", "adamw")
        if not use_banks:
            log(f"optimizer {opt_name!r} needs per-matrix parameters: parameters are replicated, not sharded")
        weights = "peer" if getattr(args, "peer_weights", False) else getattr(args, "fsdp_weights", "gathered")
        engine = ShardedEngine(model, use_banks=use_banks, cpu_offload=getattr(args, "cpu_offload", False),
                               weights=weights, grads=getattr(args, "fsdp_grads", "replicated"),
                               nvls=bool(getattr(args, "nvls", False)),
                               grad_prefetch=bool(getattr(args, "grad_prefetch", False)))
        banks = engine.banks

    tokens_per_step = args.batch_size * args.max_length * args.gradient_accumulation_steps * world_size
    if args.num_training_steps is None:
        args.num_training_steps = max(1, count_num_training_tokens(model) // tokens_per_step)
    vocab = model.config.vocab_size
    loader = build_dataloader(args, tokenizer, vocab, rank, world_size)
    eval_batches = None
    if args.eval_interval:        # fixed evaluation set, collected once
        eval_iter = iter(build_dataloader(args, tokenizer, vocab, rank, world_size, eval_split=True))
        eval_batches = [next(eval_iter) for _ in range(args.eval_steps)]

    optimizer = get_optimizer(args.optimizer, model, args)
    if mode == "fsdp":
        scheduler = wsd_schedule(optimizer, args.num_warmup_steps, 0, args.num_decay_steps, args.min_lr_ratio)
    else:
        scheduler = cosine_with_warmup(optimizer, args.num_warmup_steps, args.num_training_steps)
    if mode == "fsdp":
        engine.attach_optimizer(optimizer)
    if logger is not None:
        logger.log_optimizer_source(optimizer)
    apply_reconfigure = make_apply_reconfigure(optimizer, parse_reconfigure_schedule(args.reconfigure_schedule), log)
    apply_reconfigure(0)

    trainer = Trainer(model, optimizer, scheduler, engine, args.gradient_accumulation_steps, device,
                      graph_microbatch=bool(getattr(args, "cuda_graph_step", False)),
                      phase_timing=bool(getattr(args, "time_stats", False)))
    trainer.zero_set_to_none = not args.cuda_graph if hasattr(optimizer, "reconfigure") else True
    if trainer.graph_microbatch:
        trainer.zero_set_to_none = False       # captured graphs write into the gradient tensors that exist at capture
    budget = TimeBudget(args.time_budget)
    eos = getattr(tokenizer, "eos_token_id", None)
    global_step, tokens_seen, micro = 0, 0, []
    t_step = time.perf_counter()
    last = {}
    model.train()
    for batch in loader:
        tokens_seen += int((batch["labels"] != eos).sum()) if eos is not None else batch["labels"].numel()
        micro.append(batch)
        if len(micro) < args.gradient_accumulation_steps:
            continue
        loss = trainer.train_step(micro)
        micro = []
        global_step += 1
        apply_reconfigure(global_step)
        tok = torch.tensor([tokens_seen], dtype=torch.int64, device=device)
        if distributed and world_size > 1:
            dist.all_reduce(tok, op=dist.ReduceOp.SUM)
        metrics = {"step": global_step, "lr": optimizer.param_groups[0]["lr"], "loss": trainer.read_loss(loss),
                   "tokens": int(tok.item())}
        if getattr(args, "time_stats", False):
            if device.type == "cuda":
                torch.cuda.synchronize()
            now = time.perf_counter()
            metrics["step_time"] = now - t_step
            metrics["tokens_per_sec"] = tokens_per_step / max(1e-9, now - t_step)
            t_step = now
            for name, ms in trainer.phases.summary().items():       # device time per phase, max over ranks
                metrics[f"ms_{name}"] = round(ms, 3)
            trainer.phases.reset()
        if args.eval_interval and global_step % args.eval_interval == 0:
            metrics["eval_loss"] = trainer.evaluate(eval_batches)
        if logger is not None:
            logger.log_metrics(metrics)
        last = metrics
        stop = global_step >= args.num_training_steps or budget.is_expired()
        if distributed and world_size > 1:
            # one small collective per step carries rank 0's stop decision and every rank's kernel status, so a
            # rank whose bounded wait ran out makes all ranks raise together instead of training on garbage
            flag = torch.tensor([int(stop) if is_main else 0, trainer.device_status()], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            stop, bad = bool(flag[0].item()), int(flag[1].item())
            if bad:
                raise RuntimeError(f"himuon_b200: a device-side wait timed out on some rank (status code {bad}); stopping")
        if stop:
            log("Stopping training")
            break

    if args.save_checkpoint:
        out_dir = os.path.join("checkpoints", f"{run_name}_step{global_step}")
        if mode == "fsdp":
            state = engine.full_state_dict()      # gathered and un-banked on rank 0
            if is_main:
                model.save_pretrained(out_dir, state_dict=state)
        elif is_main:
            model.save_pretrained(out_dir)
        if is_main and hasattr(tokenizer, "save_pretrained"):
            tokenizer.save_pretrained(out_dir)
        log(f"Saved checkpoint to {out_dir}")
    if distributed:
        if engine is not None:
            engine.close()
        dist.barrier()
        dist.destroy_process_group()
    return last
