"""A marker in the autograd graph at a boundary of the decoder's layer loop.

The engines of this package act when the backward pass crosses such a boundary: the sharded engine rotates its weight
staging ring and reduces a finished layer group's gradients, the data-parallel engine starts the all-reduce of a
finished bucket while earlier layers are still being differentiated.  The reference gets the same effect from the
hooks inside PyTorch's DDP reducer and FSDP2 (``train_ddp.py:90``, ``train_fsdp.py:119-133``).
"""

from __future__ import annotations

import torch


class LayerFence(torch.autograd.Function):
    """Identity on the residual stream ``(h, delta)``.  ``owner._on_backward_boundary(kind, index)`` is called when
    the backward pass arrives here, i.e. after everything downstream of the boundary has been differentiated and
    before anything upstream of it."""

    @staticmethod
    def forward(ctx, owner, kind, index, h, delta):
        ctx.owner, ctx.kind, ctx.index = owner, kind, index
        ctx.set_materialize_grads(False)
        if delta is None:
            return h.view_as(h), None
        return h.view_as(h), delta.view_as(delta)

    @staticmethod
    def backward(ctx, gh, gd):
        ctx.owner._on_backward_boundary(ctx.kind, ctx.index)
        return None, None, None, gh, gd
