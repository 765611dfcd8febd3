"""Data-parallel engine: replicated parameters, gradients averaged by the fused peer-memory all-reduce.

Every trainable parameter's ``.grad`` is a view into one flat region of the symmetric heap (per dtype), so the
weight-gradient GEMMs accumulate straight into the communication buffer and no copy precedes the collective.
Accumulation micro-steps do no communication (the reference's ``no_sync()``, ``train_ddp.py:158-161``).  After the
synchronising micro-step each dtype region is reduced by one full-grid launch (the default), or, with
``overlap=True``, the reduction overlaps the backward pass the way the DDP reducer's buckets do (``train_ddp.py:90``):
the decoder layers' matrices are laid out layer by layer, a bucket is a run of consecutive layers, and as soon as the
backward pass has left a bucket's first layer its all-reduce starts on a side stream with a small grid, beside the
remaining backward GEMMs; what is left when backward ends (embeddings, norm weights, whose gradients are folded in
at the very end) is reduced by one more launch.
Replaces ``torch.nn.parallel.DistributedDataParallel`` and its bucketed NCCL all-reduce.
"""

from __future__ import annotations

import re
from contextlib import contextmanager

import torch
import torch.distributed as dist

from .fence import LayerFence
from .symm import SymmetricHeap, _world

_LAYER_RE = re.compile(r"(?:^|\.)layers\.(\d+)\.")


class DataParallelEngine:
    def __init__(self, model: torch.nn.Module, timeout_s: float = 120.0, broadcast_params: bool = True,
                 overlap: bool = False, bucket_layers: int = 4, comm_blocks: int = 16, nvls: bool = False):
        """``overlap``: start each bucket's all-reduce from inside the backward pass (side stream) instead of one
        full-grid launch per region after it.  Off by default: on B200 / NVLink 5 the single launch measured faster at
        every size tried (Qwen3-0.6B, 1.19 GB of gradients: equal on 2 GPUs, 1.4 % faster on 4, 1.8 % on 8), because
        the all-reduce takes 3 ms at full grid while the small-grid bucket launches slow the power-limited backward
        GEMMs by as much as they hide;
        ``bucket_layers``: decoder layers per bucket; ``comm_blocks``: grid cap of the overlapped all-reduce launches
        (they share the SMs with the backward GEMMs); ``nvls``: bind the gradient heap to an NVLink multicast object
        and reduce / broadcast through the switch (``multimem``) instead of peer loads and stores."""
        self.model = model
        self.rank, self.world = _world()
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.device = named[0][1].device
        self.cuda = self.device.type == "cuda"
        self.bucket_layers = max(1, int(bucket_layers))
        self.comm_blocks = int(comm_blocks)
        self._pad = 16 * max(1, self.world)     # elements: keeps every region a multiple of 16 B x world

        # Matrices of decoder layer i (complete as soon as the backward pass has left layer i) come first, layer by
        # layer; everything else (embeddings, head, norm weights with their deferred gradients) follows.
        by_dtype: dict[torch.dtype, dict] = {}
        n_layers = 0
        for name, p in named:
            m = _LAYER_RE.search(name)
            rec = by_dtype.setdefault(p.dtype, {"layers": {}, "rest": []})
            if m is not None and p.ndim >= 2:
                rec["layers"].setdefault(int(m.group(1)), []).append(p)
                n_layers = max(n_layers, int(m.group(1)) + 1)
            else:
                rec["rest"].append(p)
        self.n_layers = n_layers
        self.n_buckets = -(-n_layers // self.bucket_layers) if n_layers else 0
        total = 0
        for dt, rec in by_dtype.items():
            esz = torch.empty((), dtype=dt).element_size()
            n = sum(self._padded(sum(p.numel() for li in self._bucket_range(k) for p in rec["layers"].get(li, [])))
                    for k in range(self.n_buckets))
            n += self._padded(sum(p.numel() for p in rec["rest"]))
            total += n * esz + 4096
        self.heap = SymmetricHeap(total, self.device, timeout_s, multicast=nvls)
        self._algo = 3 if self.heap.has_multicast else 0
        self.regions = []          # (flat tensor, heap offset) per dtype: zeroing and whole-region reduction
        self.buckets: list[list] = [[] for _ in range(self.n_buckets)]   # per bucket: (slice, heap offset) per dtype
        self.rest = []             # (slice, heap offset) per dtype
        for dt, rec in by_dtype.items():
            esz = torch.empty((), dtype=dt).element_size()
            sizes = [self._padded(sum(p.numel() for li in self._bucket_range(k) for p in rec["layers"].get(li, [])))
                     for k in range(self.n_buckets)]
            rest_n = self._padded(sum(p.numel() for p in rec["rest"]))
            flat, offset = self.heap.alloc((sum(sizes) + rest_n,), dt)
            flat.zero_()
            cursor = 0
            for k in range(self.n_buckets):
                start = cursor
                for li in self._bucket_range(k):
                    for p in rec["layers"].get(li, []):
                        p.grad = flat[cursor:cursor + p.numel()].view(p.shape)
                        cursor += p.numel()
                cursor = start + sizes[k]
                if sizes[k]:
                    self.buckets[k].append((flat[start:start + sizes[k]], offset + start * esz))
            start = cursor
            for p in rec["rest"]:
                p.grad = flat[cursor:cursor + p.numel()].view(p.shape)
                cursor += p.numel()
            if rest_n:
                self.rest.append((flat[start:start + rest_n], offset + start * esz))
            self.regions.append((flat, offset))
        if broadcast_params and self.world > 1:
            for p in model.parameters():
                dist.broadcast(p.data, src=0)
        self._sync = True
        self.overlap = bool(overlap) and self.world > 1 and self.n_buckets > 0
        # forward+backward graphs of the synchronising micro-step contain the bucket all-reduces: it needs its own graph
        self.graph_key_sync = self.overlap
        self._side = torch.cuda.Stream(self.device) if (self.cuda and self.overlap) else None
        self._launched: set[int] = set()
        self._side_done = None
        self.overlapped_launches = 0
        object.__setattr__(model, "_layer_hooks", self if self.overlap else None)

    def _region_algo(self, flat) -> int:
        """Through the switch when the heap has a multicast mapping, except for small, latency-bound regions."""
        if self._algo == 3 and flat.numel() * flat.element_size() > (256 << 10):
            return 3
        return 0

    def _bucket_range(self, k: int):
        return range(k * self.bucket_layers, min(self.n_layers, (k + 1) * self.bucket_layers))

    def _padded(self, n: int) -> int:
        return -(-n // self._pad) * self._pad

    # ------------------------------------------------------------------ layer-loop hooks
    def pre_layer(self, i: int, h, delta):
        """Before decoder layer ``i``: the first layer of a bucket marks, in the autograd graph of a synchronising
        micro-step, the point where the bucket's gradients are complete."""
        if i == 0:
            self._launched.clear()
        if self._sync and i % self.bucket_layers == 0 and torch.is_grad_enabled() and h.requires_grad:
            h, delta = LayerFence.apply(self, "start", i // self.bucket_layers, h, delta)
        return h, delta

    def post_layer(self, i: int, h, delta):
        return h, delta

    def _on_backward_boundary(self, kind: str, k: int):
        """The backward pass has left bucket ``k``: average it over the ranks beside the rest of backward."""
        if k in self._launched:
            return
        self._launched.add(k)
        self.overlapped_launches += 1
        if not self.cuda:
            for flat, offset in self.buckets[k]:
                self.heap.allreduce_(flat, offset, 1.0 / self.world, algo=self._region_algo(flat))
            return
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(self._side):
            self._side.wait_event(ready)
            for flat, offset in self.buckets[k]:
                self.heap.allreduce_(flat, offset, 1.0 / self.world, max_blocks=self.comm_blocks, algo=self._algo)
            done = torch.cuda.Event()
            done.record(self._side)
        if k == 0:
            # Bucket 0 is the last one the backward pass leaves.  The compute stream joins the side stream here, so
            # that one rank never has collectives in flight on two streams and a CUDA-graph capture of this
            # micro-step ends with every forked stream joined.
            main.wait_event(done)
            self._side_done = None
        else:
            self._side_done = done

    # ---- CUDA-graph replays run none of the Python above: the trainer saves and restores what it would have set
    def graph_capture_state(self):
        return frozenset(self._launched)

    def graph_replay_state(self, state) -> None:
        self._launched = set(state)
        self._side_done = None

    @contextmanager
    def no_sync(self):
        """Accumulation micro-step: no reduction is started from its backward pass."""
        prev, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = prev

    def finish_backward(self):
        """Average whatever the backward pass has not reduced already."""
        if self._side_done is not None:
            torch.cuda.current_stream(self.device).wait_event(self._side_done)
            self._side_done = None
        if not self._launched:                       # nothing was overlapped: one launch per dtype region
            for flat, offset in self.regions:
                self.heap.allreduce_(flat, offset, 1.0 / self.world, algo=self._region_algo(flat))
            return
        for k in range(self.n_buckets):
            if k not in self._launched:
                for flat, offset in self.buckets[k]:
                    self.heap.allreduce_(flat, offset, 1.0 / self.world, algo=self._region_algo(flat))
        for flat, offset in self.rest:
            self.heap.allreduce_(flat, offset, 1.0 / self.world, algo=self._region_algo(flat))
        self._launched.clear()

    def zero_grad(self, set_to_none: bool = False):
        """Gradients live in the communication buffer, so they are zeroed in place, never dropped."""
        for flat, _ in self.regions:
            flat.zero_()

    def close(self):
        for p in self.model.parameters():
            p.grad = None
        object.__setattr__(self.model, "_layer_hooks", None)
        self.regions, self.buckets, self.rest = [], [], []
        self.heap.close()
