"""Differentiable ops of the decoder and the optimizers.

On a CUDA device with bf16 tensors every op launches the hand-written sm_100a kernels of
``himuon_b200/csrc`` (and raises if the extension is missing); anywhere else (CPU, fp32) the
pure-PyTorch implementations of :mod:`himuon_b200.ops.reference` run and autograd
differentiates them.  A launch counter records how many of the library's own kernels were
issued (``launch_count()``), which the benchmark reports.
"""

from __future__ import annotations

import math

import weakref

import torch

from . import reference as ref
from .. import _ext

_LAUNCHES = 0


def launch_count() -> int:
    return _LAUNCHES


def _count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def add_launches(n: int) -> None:
    """Accounts for kernels launched by replaying a captured CUDA graph (the Python wrappers do not run then)."""
    _count(n)


def use_kernels(t: torch.Tensor) -> bool:
    """True when ``t`` runs on the sm_100a kernel path (CUDA + bf16)."""
    return t.is_cuda and t.dtype == torch.bfloat16


_WARNED: set = set()


def _warn_torch_path(op: str, why: str) -> None:
    """Says once per (op, reason) that a bf16 CUDA tensor is taking the plain PyTorch implementation of an op."""
    if (op, why) not in _WARNED:
        _WARNED.add((op, why))
        import warnings
        warnings.warn(f"himuon_b200.ops.{op}: {why}; running the PyTorch implementation instead of the sm_100a kernel",
                      stacklevel=3)


def check_status() -> None:
    """Raise if any kernel's bounded wait ran out since the last check (synchronises)."""
    code = _ext.ext().status(True)
    if code:
        raise RuntimeError(f"himuon_b200: a device-side wait timed out (status code {code}); results are invalid")


# ------------------------------------------------------------------------------------------- GEMM
def gemm(a, b, *, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, aux=None, out=None,
         out_dtype=None, round_acc=False, max_ctas=0, symmetric=False):
    """``alpha * op(a) @ op(b) + beta * aux`` for 2-D or batched 3-D operands (no autograd).  ``symmetric``: the caller
    guarantees a symmetric result (``X X^T``; ``c A A + b A`` with ``A`` symmetric), which lets the kernel compute one
    triangle of tiles and mirror it."""
    if use_kernels(a):
        M = a.shape[-1] if trans_a else a.shape[-2]
        N = b.shape[-2] if trans_b else b.shape[-1]
        if out is None:
            out = torch.empty(*a.shape[:-2], M, N, device=a.device, dtype=out_dtype or torch.bfloat16)
        if a.stride(-1) != 1:
            a = a.contiguous()
        if b.stride(-1) != 1:
            b = b.contiguous()
        _ext.ext().gemm(a, b, out, aux, trans_a, trans_b, float(alpha), float(beta), bool(round_acc), int(max_ctas),
                        bool(symmetric))
        _count()
        return out
    A = a.transpose(-2, -1) if trans_a else a
    B = b.transpose(-2, -1) if trans_b else b
    if a.dtype == torch.bfloat16:
        res = alpha * (A.float() @ B.float())
        if round_acc:
            res = res.bfloat16().float()
    else:
        res = alpha * (A @ B)
    if aux is not None and beta != 0.0:
        res = res + beta * aux.to(res.dtype)
    res = res.to(out_dtype or a.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


class GradSink:
    """Destination of a weight gradient that bypasses autograd accumulation.

    ``buffer`` is a persistent ``(H, W)`` view (for example one slot of a bank's gradient
    buffer).  The first write after ``reset()`` overwrites, later writes accumulate.
    """

    __slots__ = ("buffer", "fresh", "__weakref__")
    _log: "list | None" = None          # while a list: every sink written to is appended (CUDA-graph capture)

    def __init__(self, buffer: torch.Tensor):
        self.buffer = buffer
        self.fresh = True

    @classmethod
    def start_log(cls) -> None:
        cls._log = []

    @classmethod
    def stop_log(cls) -> list:
        """Weak references to the sinks written since ``start_log()``.  A replay of the graph captured meanwhile
        writes the same sinks without running any Python, so its caller marks them used afterwards."""
        seen, out = set(), []
        for s in cls._log or []:
            if id(s) not in seen:
                seen.add(id(s))
                out.append(weakref.ref(s))
        cls._log = None
        return out

    def mark_used(self) -> None:
        self.fresh = False
        if GradSink._log is not None:
            GradSink._log.append(self)

    def reset(self):
        self.fresh = True

    def add_wgrad(self, dy2d: torch.Tensor, x2d: torch.Tensor) -> None:
        gemm(dy2d, x2d, trans_a=True, out=self.buffer, aux=None if self.fresh else self.buffer,
             beta=0.0 if self.fresh else 1.0)
        self.mark_used()


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, sink, param, w_getter=None):
        x2 = x.reshape(-1, x.shape[-1])
        if w_getter is not None:
            # The weight lives in a staging buffer that is reused for other layers between this forward and its
            # backward: it is looked up again in backward instead of being saved (autograd would reject the reuse).
            w = w_getter()
            ctx.save_for_backward(x2)
        else:
            ctx.save_for_backward(x2, w)
        y = gemm(x2, w, trans_b=True)
        ctx.w_getter = w_getter
        ctx.sink = sink
        ctx.param = param
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        if ctx.w_getter is not None:
            (x2,), w = ctx.saved_tensors, ctx.w_getter()
        else:
            x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1 or dy2.stride(0) % 8 or dy2.data_ptr() % 16:
            dy2 = dy2.contiguous()            # column slices of a wider buffer are consumed in place
        dx = gemm(dy2, w).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.sink is not None:
            ctx.sink.add_wgrad(dy2, x2)
        elif ctx.needs_input_grad[1]:
            p = ctx.param
            if p is not None and p.grad is not None and p.grad.dtype in (torch.bfloat16, torch.float32) \
                    and p.grad.is_contiguous():
                # accumulate straight into the existing gradient (no temporary, no extra add kernel)
                gemm(dy2, x2, trans_a=True, out=p.grad, aux=p.grad, beta=1.0)
            else:
                dw = gemm(dy2, x2, trans_a=True)
        return dx, dw, None, None, None


def linear(x: torch.Tensor, w: torch.Tensor | None, sink: GradSink | None = None, w_getter=None) -> torch.Tensor:
    """``x @ w.T``.  With ``sink`` the weight gradient is written there instead of returned.  ``w_getter`` (with a
    sink): a callable returning the weight, called in forward and again in backward, for weights kept in a staging
    buffer whose contents come and go between the two passes; ``w`` is then ignored."""
    if w_getter is not None:
        assert sink is not None, "a staged weight has no autograd gradient: a sink must take it"
        if use_kernels(x) and x.dtype == torch.bfloat16:
            return _LinearFn.apply(x, None, sink, None, w_getter)
        return _SinkLinearRef.apply(x, None, sink, w_getter)
    if use_kernels(x) and w.dtype == torch.bfloat16:
        param = w if isinstance(w, torch.nn.Parameter) else None
        return _LinearFn.apply(x, w, sink, param)
    if sink is not None:
        return _SinkLinearRef.apply(x, w, sink)
    return torch.nn.functional.linear(x, w)


class _SinkLinearRef(torch.autograd.Function):
    """CPU / fp32 counterpart of the sink path (used by the bank engine off-GPU)."""

    @staticmethod
    def forward(ctx, x, w, sink, w_getter=None):
        if w_getter is not None:
            w = w_getter()
            ctx.save_for_backward(x)
        else:
            ctx.save_for_backward(x, w)
        ctx.w_getter = w_getter
        ctx.sink = sink
        return torch.nn.functional.linear(x, w)

    @staticmethod
    def backward(ctx, dy):
        if ctx.w_getter is not None:
            (x,), w = ctx.saved_tensors, ctx.w_getter()
        else:
            x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dw = (dy2.float().t() @ x2.float()).to(ctx.sink.buffer.dtype)
        if ctx.sink.fresh:
            ctx.sink.buffer.copy_(dw)
            ctx.sink.mark_used()
        else:
            ctx.sink.buffer.add_(dw)
        return (dy2 @ w).view(x.shape), None, None, None


# ------------------------------------------------------------------------------------------- deferred norm-weight grads
class _NormGradArena:
    """fp32 accumulators for the weight gradients of the norm layers.

    The norm backward kernels add their per-column sums straight into a slice of one persistent fp32 buffer; a
    callback queued on the autograd engine folds all pending slices into the parameters' ``.grad`` once, at the end
    of the backward pass (one cast, one multi-tensor add, one clear), instead of a zero-fill, a cast and an
    accumulation kernel per norm call.  Only used for leaf parameters (``defer_dw=True`` from the model code);
    ``torch.autograd.grad`` callers keep the immediate path.
    """

    CHUNK = 1 << 20

    def __init__(self, device):
        self.device = device
        self.chunks: list[torch.Tensor] = []
        self.used = self.CHUNK                      # forces the first allocation
        self.slots: dict[int, tuple] = {}           # id(param) -> (weakref, chunk index, offset, numel)
        self.pending: dict[int, None] = {}
        self.queued = False

    def buffer_for(self, w: torch.Tensor) -> torch.Tensor:
        slot = self.slots.get(id(w))
        if slot is None or slot[0]() is not w:
            n = (w.numel() + 3) // 4 * 4            # 16-byte aligned slices (four-wide atomics)
            if self.used + n > self.CHUNK:
                self.chunks.append(torch.zeros(max(self.CHUNK, n), device=self.device, dtype=torch.float32))
                self.used = 0
            slot = (weakref.ref(w), len(self.chunks) - 1, self.used, w.numel())
            self.used += n
            self.slots[id(w)] = slot
        self.pending[id(w)] = None
        if not self.queued:
            self.queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self.flush)
        return self.chunks[slot[1]][slot[2]: slot[2] + slot[3]]

    def flush(self) -> None:
        self.queued = False
        pending, self.pending = self.pending, {}
        by_chunk: dict[int, list] = {}
        for key in pending:
            ref_w, ci, off, n = self.slots[key]
            w = ref_w()
            if w is not None:
                by_chunk.setdefault(ci, []).append((w, off, n))
        for ci, items in by_chunk.items():
            chunk = self.chunks[ci]
            hi = max(off + n for _, off, n in items)
            casts: dict[torch.dtype, torch.Tensor] = {}
            grads, srcs = [], []
            for w, off, n in items:
                if w.dtype not in casts:
                    casts[w.dtype] = chunk[:hi].to(w.dtype)
                g = casts[w.dtype][off: off + n].view_as(w)
                if w.grad is None:
                    w.grad = g.clone()
                else:
                    grads.append(w.grad)
                    srcs.append(g)
            if grads:
                torch._foreach_add_(grads, srcs)
            chunk[:hi].zero_()


_NORM_ARENAS: dict = {}


def _norm_grad_buffer(w: torch.Tensor) -> torch.Tensor:
    arena = _NORM_ARENAS.get(w.device)
    if arena is None:
        arena = _NORM_ARENAS[w.device] = _NormGradArena(w.device)
    return arena.buffer_for(w)


def _deferrable(w, defer_dw: bool) -> bool:
    return bool(defer_dw) and w is not None and w.is_leaf and w.requires_grad


# ------------------------------------------------------------------------------------------- norms / rope
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, defer_dw=False):
        ctx.defer_dw = defer_dw
        # the parameter object itself: under activation checkpointing saved_tensors hands back a detached copy
        ctx.w_param = w if defer_dw else None
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
        _ext.ext().rmsnorm_fwd(x2, w, y, rstd, float(eps))
        _count()
        ctx.save_for_backward(x2, w, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = torch.empty_like(x2)
        if ctx.defer_dw:
            _ext.ext().rmsnorm_bwd(dy2, x2, w, rstd, dx, _norm_grad_buffer(ctx.w_param))
            _count(2)
            return dx.view(dy.shape), None, None, None
        dw = torch.zeros(w.numel(), device=w.device, dtype=torch.float32)
        _ext.ext().rmsnorm_bwd(dy2, x2, w, rstd, dx, dw)
        _count(2)
        return dx.view(dy.shape), dw.to(w.dtype), None, None


def rmsnorm(x, w, eps: float, defer_dw: bool = False):
    """``defer_dw``: accumulate the weight gradient in fp32 and add it to ``w.grad`` once at the end of the backward
    pass (for leaf parameters trained with ``backward()``; ``torch.autograd.grad`` on ``w`` needs ``False``)."""
    if use_kernels(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _RMSNormFn.apply(x, w, eps, _deferrable(w, defer_dw))
    return ref.rmsnorm(x, w, eps)


class _AddRMSNormFn(torch.autograd.Function):
    """``h = x + delta; y = rmsnorm(h)`` in one kernel; returns ``(h, y)``.  Backward folds the gradient that
    arrives on ``h`` (the residual path) into the norm's input gradient, which is the gradient of both inputs."""

    @staticmethod
    def forward(ctx, x, delta, w, eps, defer_dw=False):
        ctx.defer_dw = defer_dw
        # the parameter object itself: under activation checkpointing saved_tensors hands back a detached copy
        ctx.w_param = w if defer_dw else None
        ctx.set_materialize_grads(False)      # an unused output arrives as None instead of a zero tensor
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        d2 = delta.reshape(-1, x.shape[-1]).contiguous()
        h = torch.empty_like(x2)
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
        _ext.ext().rmsnorm_fwd(x2, w, y, rstd, float(eps), d2, h)
        _count()
        ctx.save_for_backward(h, w, rstd)
        return h.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, g_h, g_y):
        h, w, rstd = ctx.saved_tensors
        if g_y is None:                       # the normalised output was not used
            return g_h, g_h, None, None, None
        dy2 = g_y.reshape(-1, g_y.shape[-1]).contiguous()
        res = g_h.reshape(-1, g_h.shape[-1]).contiguous() if g_h is not None else None
        dx = torch.empty_like(h)
        if ctx.defer_dw:
            _ext.ext().rmsnorm_bwd(dy2, h, w, rstd, dx, _norm_grad_buffer(ctx.w_param), res)
            _count(2)
            dx = dx.view(g_y.shape)
            return dx, dx, None, None, None
        dw = torch.zeros(w.numel(), device=w.device, dtype=torch.float32)
        _ext.ext().rmsnorm_bwd(dy2, h, w, rstd, dx, dw, res)
        _count(2)
        dx = dx.view(g_y.shape)
        return dx, dx, dw.to(w.dtype), None, None


def add_rmsnorm(x, delta, w, eps: float, defer_dw: bool = False):
    """Residual update followed by RMSNorm: returns ``(x + delta, rmsnorm(x + delta))``; ``delta=None`` skips the add."""
    if delta is None:
        return x, rmsnorm(x, w, eps, defer_dw)
    if use_kernels(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and delta.shape == x.shape:
        return _AddRMSNormFn.apply(x, delta, w, eps, _deferrable(w, defer_dw))
    h = x + delta
    return h, ref.rmsnorm(h, w, eps)


class _HeadNormRopeFn(torch.autograd.Function):
    """Per-head RMSNorm (optional) + RoPE on a ``(tokens, heads*128)`` view."""

    @staticmethod
    def forward(ctx, x, w, cos_sin, heads, seq_len, eps, defer_dw=False, inplace_grad=False):
        ctx.defer_dw = defer_dw
        # the parameter object itself: under activation checkpointing saved_tensors hands back a detached copy
        ctx.w_param = w if defer_dw else None
        ctx.inplace_grad = inplace_grad
        y = torch.empty(x.shape[0], heads * 128, device=x.device, dtype=x.dtype)
        rstd = torch.empty(x.shape[0] * heads, device=x.device, dtype=torch.float32) if w is not None else None
        _ext.ext().headnorm_rope_fwd(x, w, y, rstd, cos_sin, heads, seq_len, float(eps))
        _count()
        ctx.save_for_backward(x, w, rstd, cos_sin)
        ctx.heads, ctx.seq_len = heads, seq_len
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd, cos_sin = ctx.saved_tensors
        if dy.stride(-1) != 1:
            dy = dy.contiguous()
        # Each head vector is read completely before it is written, so the input gradient may take the place of the
        # incoming one (asked for by callers that know dy has no other reader, e.g. a slice of attention's dq|dk|dv).
        inplace = ctx.inplace_grad and dy.stride(0) % 8 == 0 and dy.data_ptr() % 16 == 0
        dx = dy if inplace else torch.empty(dy.shape[0], ctx.heads * 128, device=dy.device, dtype=dy.dtype)
        if w is not None and ctx.defer_dw:
            _ext.ext().headnorm_rope_bwd(dy, x, w, rstd, dx, _norm_grad_buffer(ctx.w_param), cos_sin, ctx.heads, ctx.seq_len)
            _count(2)
            return dx, None, None, None, None, None, None, None
        dw = torch.zeros(128, device=dy.device, dtype=torch.float32) if w is not None else None
        _ext.ext().headnorm_rope_bwd(dy, x if w is not None else None, w, rstd, dx, dw, cos_sin, ctx.heads, ctx.seq_len)
        _count(2 if w is not None else 1)
        return dx, (dw.to(w.dtype) if w is not None else None), None, None, None, None, None, None


def head_norm_rope(x2d, w, cos_sin, heads: int, seq_len: int, head_dim: int, eps: float, defer_dw: bool = False,
                   inplace_grad: bool = False):
    """``x2d``: ``(B*S, heads*head_dim)`` (may be a column slice).  Returns the same layout.  ``inplace_grad``: the
    backward pass may overwrite the gradient it receives with the gradient it returns."""
    if use_kernels(x2d) and head_dim == 128:
        return _HeadNormRopeFn.apply(x2d, w, cos_sin, heads, seq_len, eps, _deferrable(w, defer_dw), inplace_grad)
    if use_kernels(x2d):
        _warn_torch_path("head_norm_rope", f"head_dim {head_dim} (the kernel is written for 128)")
    T = x2d.shape[0]
    x = x2d.reshape(T // seq_len, seq_len, heads, head_dim)
    if w is not None:
        x = ref.rmsnorm(x, w, eps)
    return ref.apply_rope(x, cos_sin).reshape(T, heads * head_dim)


class _SplitColsFn(torch.autograd.Function):
    """``x[:, :n0], x[:, n0:]`` whose backward hands the two gradients back as one tensor without a zero fill and an
    add: when they already are the adjacent column blocks of one buffer (attention's ``dq|dk|dv``) that view is
    returned as is, otherwise they are copied into a fresh buffer."""

    @staticmethod
    def forward(ctx, x, n0):
        ctx.n0 = n0
        ctx.cols = x.shape[1]
        return x[:, :n0], x[:, n0:]

    @staticmethod
    def backward(ctx, g0, g1):
        n0, n1 = ctx.n0, ctx.cols - ctx.n0
        if g0 is None and g1 is None:
            return None, None
        if (g0 is not None and g1 is not None and g0.stride(1) == 1 and g1.stride(1) == 1
                and g0.untyped_storage().data_ptr() == g1.untyped_storage().data_ptr()
                and g0.stride(0) == g1.stride(0) and g1.storage_offset() == g0.storage_offset() + n0
                and g0.stride(0) >= n0 + n1):
            return torch.as_strided(g0, (g0.shape[0], n0 + n1), (g0.stride(0), 1), g0.storage_offset()), None
        ref_t = g0 if g0 is not None else g1
        out = torch.empty(ref_t.shape[0], n0 + n1, device=ref_t.device, dtype=ref_t.dtype)
        if g0 is not None:
            out[:, :n0].copy_(g0)
        else:
            out[:, :n0].zero_()
        if g1 is not None:
            out[:, n0:].copy_(g1)
        else:
            out[:, n0:].zero_()
        return out, None


def split_cols(x2d: torch.Tensor, n0: int):
    """Column split of a 2-D tensor into ``(x[:, :n0], x[:, n0:])`` with a copy-free backward where possible."""
    return _SplitColsFn.apply(x2d, n0)


# ------------------------------------------------------------------------------------------- attention
class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, B, S, Hq, Hkv, scale):
        o = torch.empty(q.shape[0], Hq * 128, device=q.device, dtype=q.dtype)
        lse = torch.empty(B * Hq * S, device=q.device, dtype=torch.float32)
        _ext.ext().flash_attn_fwd(q, k, v, o, lse, B, S, Hq, Hkv, float(scale))
        _count()
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.dims = (B, S, Hq, Hkv, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        B, S, Hq, Hkv, scale = ctx.dims
        if do.stride(-1) != 1 or do.stride(0) % 8:
            do = do.contiguous()
        # dq | dk | dv share one buffer so the fused QKV projection sees a single contiguous gradient
        dqkv = torch.empty(q.shape[0], (Hq + 2 * Hkv) * 128, device=q.device, dtype=q.dtype)
        dq = dqkv[:, : Hq * 128]
        dk = dqkv[:, Hq * 128: (Hq + Hkv) * 128]
        dv = dqkv[:, (Hq + Hkv) * 128:]
        delta = torch.empty(B * Hq * S, device=q.device, dtype=torch.float32)
        part = torch.empty(2, q.shape[0], Hq * 128, device=q.device, dtype=q.dtype) if Hq > Hkv else None
        _ext.ext().flash_attn_bwd(do, q, k, v, o, lse, dq, dk, dv, delta, part, B, S, Hq, Hkv, float(scale))
        _count(4 if part is not None else 2)
        return dq, dk, dv, None, None, None, None, None


def attention(q2d, k2d, v2d, B: int, S: int, Hq: int, Hkv: int, head_dim: int, scale: float | None = None):
    """Causal GQA attention on ``(B*S, heads*head_dim)`` views; returns ``(B*S, Hq*head_dim)``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if use_kernels(q2d) and head_dim == 128:
        return _FlashAttnFn.apply(q2d, k2d, v2d, B, S, Hq, Hkv, scale)
    if use_kernels(q2d) and head_dim < 128 and head_dim % 8 == 0:
        # Smaller heads (64 in Llama-3.2-1B and llama_220m) run the same tcgen05 kernels zero-padded to 128: zeros in
        # q and k add nothing to the scores, zeros in v give zero output columns, which are cut off again.  Twice the
        # tensor work of a native 64-wide kernel, but no S x S score matrix in memory; autograd differentiates the
        # padding and the slice.
        T = q2d.shape[0]
        pad = 128 - head_dim

        def widen(x, heads):
            return torch.nn.functional.pad(x.reshape(T, heads, head_dim), (0, pad)).reshape(T, heads * 128)

        o = _FlashAttnFn.apply(widen(q2d, Hq), widen(k2d, Hkv), widen(v2d, Hkv), B, S, Hq, Hkv, scale)
        return o.reshape(T, Hq, 128)[:, :, :head_dim].reshape(T, Hq * head_dim)
    if use_kernels(q2d):
        _warn_torch_path("attention", f"head_dim {head_dim} (the kernels take 128, or a multiple of 8 below it)")
    q = q2d.reshape(B, S, Hq, head_dim)
    k = k2d.reshape(B, S, Hkv, head_dim)
    v = v2d.reshape(B, S, Hkv, head_dim)
    return ref.attention(q, k, v, scale).reshape(B * S, Hq * head_dim)


# ------------------------------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        out = torch.empty(gate.shape, device=gate.device, dtype=gate.dtype)
        _ext.ext().swiglu_fwd(gate, up, out)
        _count()
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, dout):
        gate, up = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dgu = torch.empty(gate.shape[0], 2 * gate.shape[1], device=gate.device, dtype=gate.dtype)
        dgate, dup = dgu[:, : gate.shape[1]], dgu[:, gate.shape[1]:]
        _ext.ext().swiglu_bwd(dout, gate, up, dgate, dup)
        _count()
        return dgate, dup


class _SwiGLUPackedFn(torch.autograd.Function):
    """SwiGLU on a packed ``(tokens, 2*I)`` projection output ``[gate | up]``; the backward pass returns one
    packed gradient, so the fused gate/up GEMM sees a single contiguous ``dy``."""

    @staticmethod
    def forward(ctx, gu):
        I = gu.shape[1] // 2
        out = torch.empty(gu.shape[0], I, device=gu.device, dtype=gu.dtype)
        _ext.ext().swiglu_fwd(gu[:, :I], gu[:, I:], out)
        _count()
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        I = gu.shape[1] // 2
        if dout.stride(-1) != 1 or dout.stride(0) % 8:
            dout = dout.contiguous()
        dgu = torch.empty_like(gu)
        _ext.ext().swiglu_bwd(dout, gu[:, :I], gu[:, I:], dgu[:, :I], dgu[:, I:])
        _count()
        return dgu


def swiglu_packed(gu):
    """``silu(gu[:, :I]) * gu[:, I:]`` for a packed gate/up projection output."""
    I = gu.shape[1] // 2
    if use_kernels(gu) and gu.dim() == 2 and I % 8 == 0 and gu.is_contiguous():
        return _SwiGLUPackedFn.apply(gu)
    return ref.swiglu(gu[:, :I], gu[:, I:])


def swiglu(gate, up):
    """``silu(gate) * up`` on 2-D ``(tokens, I)`` views (either may be a column slice)."""
    if use_kernels(gate) and gate.dim() == 2 and gate.shape[1] % 8 == 0 and gate.stride(0) % 8 == 0 \
            and up.stride(0) % 8 == 0:
        return _SwiGLUFn.apply(gate, up)
    return ref.swiglu(gate, up)


# ------------------------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).contiguous()
        out = torch.empty(flat.numel(), table.shape[1], device=table.device, dtype=table.dtype)
        _ext.ext().embedding_fwd(flat, table, out)
        _count()
        ctx.save_for_backward(flat)
        ctx.table = table
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dout):
        (flat,) = ctx.saved_tensors
        table = ctx.table
        d2 = dout.reshape(-1, dout.shape[-1]).contiguous()
        if isinstance(table, torch.nn.Parameter) and table.grad is not None and table.grad.is_contiguous() \
                and table.grad.dtype in (torch.bfloat16, torch.float32):
            _ext.ext().embedding_bwd(flat, d2, table.grad)
            _count()
            return None, None
        dt = torch.zeros(table.shape, device=table.device, dtype=table.dtype)
        _ext.ext().embedding_bwd(flat, d2, dt)
        _count(2)
        return None, dt


def embedding(ids, table):
    if use_kernels(table) and table.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, table)
    return torch.nn.functional.embedding(ids, table)


# ------------------------------------------------------------------------------------------- lm_head + CE
class _LinearCrossEntropyFn(torch.autograd.Function):
    """Token-chunked ``lm_head`` + softmax cross-entropy; logits never exist for more than one chunk.

    The forward pass already produces ``dh`` and ``dW`` (scaled by ``loss_scale / n_valid``, read on
    the device); the backward pass only rescales by ``g / loss_scale``.
    """

    @staticmethod
    def forward(ctx, h, w, labels, ignore_index, chunk, sink, param, loss_scale, grad_on):
        e = _ext.ext()
        T, H = h.shape
        V = w.shape[0]
        labels = labels.contiguous()
        inv = 1.0 / (labels != ignore_index).sum().clamp(min=1).float()
        loss_sum = torch.zeros((), device=h.device, dtype=torch.float32)
        count = torch.zeros((), device=h.device, dtype=torch.float32)
        # Gradients are produced here, in the forward pass, only when a backward pass will follow: grad mode on and
        # the hidden states part of a graph.  Under no_grad (evaluation) nothing may touch ``.grad`` or a sink.
        need_grad = bool(grad_on) and (h.requires_grad or w.requires_grad or sink is not None)
        dh = torch.empty_like(h) if need_grad else None
        direct = loss_scale is not None
        scale = float(loss_scale) if direct else 1.0
        target, fresh = None, True
        if need_grad:
            if direct and sink is not None:
                target, fresh = sink.buffer, sink.fresh
            elif direct and param is not None and param.grad is not None and param.grad.is_contiguous():
                target, fresh = param.grad, False
            else:
                direct = False
                scale = 1.0
                target, fresh = torch.empty(V, H, device=h.device, dtype=w.dtype), True
        logits = torch.empty(min(chunk, T), V, device=h.device, dtype=torch.bfloat16)
        for t0 in range(0, T, chunk):
            t1 = min(T, t0 + chunk)
            lg = logits[: t1 - t0]
            e.gemm(h[t0:t1], w, lg, None, False, True, 1.0, 0.0, False, 0)
            e.cross_entropy(lg, labels[t0:t1], loss_sum, count, None, scale, inv, int(ignore_index))
            _count(2)
            if need_grad:
                e.gemm(lg, w, dh[t0:t1], None, False, False, 1.0, 0.0, False, 0)
                e.gemm(lg, h[t0:t1], target, None if fresh else target, True, False, 1.0, 0.0 if fresh else 1.0, False, 0)
                fresh = False
                _count(2)
        if need_grad and direct and sink is not None:
            sink.mark_used()
        ctx.direct = direct
        ctx.scale = scale
        if need_grad:
            ctx.save_for_backward(dh, *([] if direct else [target]))
        ctx.has_grad = need_grad
        return loss_sum * inv

    @staticmethod
    def backward(ctx, g):
        if not ctx.has_grad:
            return (None,) * 9
        saved = ctx.saved_tensors
        dh = saved[0] * (g / ctx.scale).to(saved[0].dtype)
        dw = None if ctx.direct else saved[1] * g.to(saved[1].dtype)
        return dh, dw, None, None, None, None, None, None, None


def linear_cross_entropy(h2d, w, labels, ignore_index: int = -100, chunk: int = 4096, sink: GradSink | None = None,
                         loss_scale: float | None = None):
    """Mean cross-entropy of ``h2d @ w.T`` against ``labels`` (``ignore_index`` rows skipped).

    ``loss_scale`` is the factor the caller multiplies the returned loss by before ``backward()``
    (``1/grad_accumulation``).  When given, the weight gradient is accumulated in place (into
    ``sink`` or an existing ``w.grad``) during the forward pass, already scaled; without it the
    gradient flows back through autograd.  The returned loss is always the unscaled mean.
    """
    if use_kernels(h2d) and w.dtype == torch.bfloat16:
        param = w if isinstance(w, torch.nn.Parameter) else None
        # autograd.Function.forward always runs with grad mode off, so the caller's mode is passed in
        return _LinearCrossEntropyFn.apply(h2d.contiguous(), w, labels, ignore_index, chunk, sink, param, loss_scale,
                                           torch.is_grad_enabled())
    return ref.linear_cross_entropy(h2d, w, labels, ignore_index)
