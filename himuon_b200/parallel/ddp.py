"""Data-parallel engine: replicated parameters, gradients averaged by one fused all-reduce kernel.

Every trainable parameter's ``.grad`` is a view into one flat region of the symmetric heap (per
dtype), so the weight-gradient GEMMs accumulate straight into the communication buffer and the
whole model is reduced by a single launch of the two-shot peer-memory all-reduce (average fused),
issued once per optimizer step; accumulation micro-steps do no communication (the reference's
``no_sync()``, ``train_ddp.py:158-161``).  Replaces ``torch.nn.parallel.DistributedDataParallel``
(``train_ddp.py:90``) and its bucketed NCCL all-reduce.
"""

from __future__ import annotations

from contextlib import contextmanager

import torch
import torch.distributed as dist

from .symm import SymmetricHeap, _world


class DataParallelEngine:
    def __init__(self, model: torch.nn.Module, timeout_s: float = 120.0, broadcast_params: bool = True):
        self.model = model
        self.rank, self.world = _world()
        params = [p for p in model.parameters() if p.requires_grad]
        self.device = params[0].device
        by_dtype: dict[torch.dtype, list] = {}
        for p in params:
            by_dtype.setdefault(p.dtype, []).append(p)
        self._pad = 16 * max(1, self.world)     # elements: keeps every region a multiple of 16 B x world
        total = sum(self._padded(sum(p.numel() for p in ps)) * torch.empty((), dtype=dt).element_size() + 2048
                    for dt, ps in by_dtype.items())
        self.heap = SymmetricHeap(total, self.device, timeout_s)
        self.regions = []
        for dt, ps in by_dtype.items():
            n = self._padded(sum(p.numel() for p in ps))
            flat, offset = self.heap.alloc((n,), dt)
            flat.zero_()
            cursor = 0
            for p in ps:
                p.grad = flat[cursor:cursor + p.numel()].view(p.shape)
                cursor += p.numel()
            self.regions.append((flat, offset))
        if broadcast_params and self.world > 1:
            for p in model.parameters():
                dist.broadcast(p.data, src=0)
        self._sync = True

    def _padded(self, n: int) -> int:
        return -(-n // self._pad) * self._pad

    @contextmanager
    def no_sync(self):
        """Accumulation micro-step: nothing to do, reduction only happens in ``finish_backward``."""
        prev, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = prev

    def finish_backward(self):
        """Average the accumulated gradients over the ranks (one kernel per dtype region)."""
        for flat, offset in self.regions:
            self.heap.allreduce_(flat, offset, 1.0 / self.world)

    def zero_grad(self, set_to_none: bool = False):
        """Gradients live in the communication buffer, so they are zeroed in place, never dropped."""
        for flat, _ in self.regions:
            flat.zero_()

    def close(self):
        for p in self.model.parameters():
            p.grad = None
        self.regions = []
        self.heap.close()
