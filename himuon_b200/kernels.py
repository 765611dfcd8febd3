"""Public kernel callables: ``XXT``, ``ba_plus_cAA``, ``fused_bmm_add``, ``ns5_smem``.

Same call signatures and numerics contract as the reference's Triton kernel package
(``src/himuon/triton_kernels/__init__.py:21-27``; wrappers ``XXT.py:78-108``, ``ba_plus_cAA.py:92-124``,
``fused_bmm_add.py:99-135``, ``ns5_smem.py:195-263``), so its kernel microbenchmarks and kernel tests can call
them unchanged.  On a CUDA device with bf16 operands each is one launch of this library's tcgen05 kernels:

* ``XXT`` / ``ba_plus_cAA`` - the batched GEMM in its symmetric-output mode: only the tiles on or below the
  diagonal are computed, each off-diagonal tile is also stored transposed (the reference's triangle-and-mirror);
* ``fused_bmm_add`` - the batched GEMM with the ``round(acc) + a * X`` epilogue;
* ``ns5_smem`` - the tile-resident fused Newton-Schulz kernel (whole tile in shared memory, accumulators in
  tensor memory); tile shapes outside its domain run the batched three-GEMM iteration instead of failing.

Anything else (CPU tensors, fp16 / fp32 operands) is computed with plain PyTorch ops of the same rounding points.
The reference raises ``RuntimeError`` from every symbol when Triton cannot be imported; here the callables always
work, and on a CUDA machine without the compiled extension they raise from the extension loader.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ops
from .ops import ns as _ns
from .ops import reference as _ref

__all__ = ("XXT", "ba_plus_cAA", "fused_bmm_add", "ns5_smem")


def _kernel_path(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


def _as3d(t: torch.Tensor):
    return (t.unsqueeze(0), True) if t.ndim == 2 else (t, False)


def _pad8(t: torch.Tensor, rows: bool = True, cols: bool = True) -> torch.Tensor:
    """Zero-pad the last two dims up to multiples of 8 (the 16-byte granularity of the TMA boxes) and make the
    result contiguous; zero rows / columns change none of the products below."""
    pr = (-t.shape[-2]) % 8 if rows else 0
    pc = (-t.shape[-1]) % 8 if cols else 0
    if pr or pc:
        t = F.pad(t, (0, pc, 0, pr))
    return t.contiguous()


def _store(out: torch.Tensor, res: torch.Tensor, squeeze: bool) -> torch.Tensor:
    if squeeze:
        res = res[0]
    if res.data_ptr() != out.data_ptr() or res.shape != out.shape:
        out.copy_(res[..., : out.shape[-2], : out.shape[-1]])
    return out


def XXT(A: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = A @ A^T`` for ``A`` of shape ``(M, K)`` or ``(B, M, K)``; ``out`` is ``(.., M, M)``."""
    assert A.ndim in (2, 3), "XXT expects a 2-D or 3-D input"
    M = A.shape[-2]
    assert out.shape[-2] == M and out.shape[-1] == M, "Output matrix has incorrect shape"
    if not _kernel_path(A, out):
        out.copy_((A.float() @ A.float().transpose(-2, -1)).to(out.dtype))
        return out
    A3, sq = _as3d(A)
    O3, _ = _as3d(out)
    Ap = _pad8(A3)
    direct = O3.is_contiguous() and Ap.shape[-2] == M
    dst = O3 if direct else torch.empty(Ap.shape[0], Ap.shape[-2], Ap.shape[-2], device=A.device, dtype=out.dtype)
    ops.gemm(Ap, Ap, trans_b=True, out=dst, symmetric=True)
    return out if direct else _store(out, dst, sq)


def ba_plus_cAA(A: torch.Tensor, alpha: float, beta: float, out: torch.Tensor) -> torch.Tensor:
    """``out = alpha * (A @ A^T) + beta * A`` for square symmetric ``A`` (``(M, M)`` or ``(B, M, M)``)."""
    assert A.ndim in (2, 3), "ba_plus_cAA expects a 2-D or 3-D input"
    M, K = A.shape[-2:]
    assert M == K, "Input matrix must be square"
    assert out.shape[-2] == M and out.shape[-1] == M
    if not _kernel_path(A, out):
        Af = A.float()
        out.copy_((alpha * (Af @ Af.transpose(-2, -1)) + beta * Af).to(out.dtype))
        return out
    A3, sq = _as3d(A)
    O3, _ = _as3d(out)
    Ap = _pad8(A3)
    direct = O3.is_contiguous() and Ap.shape[-1] == M and O3.data_ptr() != Ap.data_ptr()
    dst = O3 if direct else torch.empty_like(Ap)
    ops.gemm(Ap, Ap, trans_b=True, alpha=alpha, beta=beta, aux=Ap, out=dst, symmetric=True)
    return out if direct else _store(out, dst, sq)


def fused_bmm_add(B: torch.Tensor, X: torch.Tensor, a: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = B @ X + a * X`` for ``B`` ``(Bt, M, M)`` and ``X`` ``(Bt, M, N)``.  The product is rounded to the
    output dtype before ``a * X`` is added (the reference kernel's rounding point, ``fused_bmm_add.py:74-88``)."""
    Bt, M, K = B.shape
    N = X.shape[-1]
    assert M == K, "fused_bmm_add requires M == K for epilogue B@X + a*X"
    if out is None:
        out = torch.empty_like(X)
    if not _kernel_path(B, X, out):
        acc = (B.float() @ X.float()).to(out.dtype)
        out.copy_((acc.float() + a * X.float()).to(out.dtype))
        return out
    Bp, Xp = _pad8(B), _pad8(X)
    direct = out.is_contiguous() and Xp.shape == X.shape and out.data_ptr() != Xp.data_ptr()
    dst = out if direct else torch.empty_like(Xp)
    ops.gemm(Bp, Xp, alpha=1.0, beta=a, aux=Xp, out=dst, round_acc=True)
    return out if direct else _store(out, dst, False)


def ns5_smem(X: torch.Tensor, *, persistent: bool = False, grid_size: int | None = None) -> torch.Tensor:
    """Five fused Newton-Schulz iterations per ``(M, N)`` tile of a bf16 ``(B, M, N)`` (or ``(M, N)``) tensor with
    ``M <= N``; returns a fresh tensor.  The sm_100a kernel is always persistent (one CTA pair per SM walking the
    tiles), so ``persistent`` and ``grid_size`` - launch-shape knobs of the Triton kernel - are accepted and have no
    effect on the result."""
    assert X.ndim in (2, 3), f"ns5_smem expects 2D or 3D, got {X.ndim}D"
    X3, sq = _as3d(X)
    _, M, N = X3.shape
    assert M <= N, f"ns5_smem expects M <= N, got ({M}, {N})"
    assert X.dtype == torch.bfloat16, f"ns5_smem is bf16-only, got {X.dtype}"
    assert X.is_contiguous(), "ns5_smem requires contiguous input"
    if not X.is_cuda:
        out = _ref.newton_schulz(X3, steps=5)
    else:
        out = _ns.newton_schulz(X3, steps=5)
    return out[0] if sq else out
