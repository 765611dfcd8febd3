"""Newton-Schulz dispatcher.

``newton_schulz(G, steps)`` is the op behind ``HiMuon.newton_schulz`` and Muon's
``zeropower_via_newtonschulz5`` (reference: ``src/himuon/optimizers/himuon.py:263-284``,
``muon.py:13-44``).  On a CUDA device it runs

* the tile-resident fused kernel (one CTA per tile, operands in shared memory, accumulators
  in TMEM) for tiles with at most 128 rows and 64..256 columns, and
* otherwise a batched three-GEMM iteration on the persistent tcgen05 GEMM with fused
  epilogues (``A = X X^T``; ``B = c A A + b A``; ``X = bf16(B X) + a X``; the two symmetric
  products compute only the tiles that touch the lower triangle and mirror them, as the
  reference's ``XXT`` / ``ba_plus_cAA`` kernels do), which handles any
  shape whose sides are multiples of 8, tall tiles included (no transpose copy: the GEMM
  reads either operand in either major).

Off-GPU the PyTorch reference with the same rounding points runs.
"""

from __future__ import annotations

import torch

from .. import _ext
from . import reference as ref
from . import _count, gemm

A_COEF, B_COEF, C_COEF = ref.NS_COEFFS


class NSWorkspace:
    """Reusable scratch for the three-GEMM path (keeps addresses stable for CUDA graphs)."""

    def __init__(self):
        self.bufs: dict[tuple, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}

    def get(self, B: int, m: int, n: int, device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        k = min(m, n)
        key = (m, n, str(device))
        cur = self.bufs.get(key)
        if cur is None or cur[0].shape[0] < B:
            cur = (
                torch.empty(B, k, k, device=device, dtype=torch.bfloat16),
                torch.empty(B, k, k, device=device, dtype=torch.bfloat16),
                torch.empty(B, m, n, device=device, dtype=torch.bfloat16),
            )
            self.bufs[key] = cur
        return cur[0][:B], cur[1][:B], cur[2][:B]

    def clear(self):
        self.bufs.clear()


def fused_supported(m: int, n: int) -> bool:
    lo, hi = min(m, n), max(m, n)
    return lo >= 1 and lo <= 128 and hi % 64 == 0 and 64 <= hi <= 256


def ns_inplace_cuda(X: torch.Tensor, steps: int = 5, eps: float = 1e-7, workspace: NSWorkspace | None = None,
                    normalize: bool = True) -> torch.Tensor:
    """Orthogonalise a contiguous bf16 ``(B, m, n)`` CUDA buffer in place and return it."""
    assert X.is_cuda and X.dtype == torch.bfloat16 and X.dim() == 3 and X.is_contiguous()
    e = _ext.ext()
    Bt, m, n = X.shape
    if Bt == 0:
        return X
    if m <= n and e.ns5_fused_supported(m, n) and normalize:
        e.ns5_fused(X, X, int(steps), float(eps))
        _count()
        return X
    if m % 8 or n % 8:
        raise ValueError(f"newton_schulz on CUDA needs tile sides that are multiples of 8, got ({m}, {n})")
    ws = workspace or NSWorkspace()
    A, Bm, Y = ws.get(Bt, m, n, X.device)
    cur, nxt = X, Y
    if normalize:
        # With an odd number of iterations the normalised copy goes to the scratch buffer, so that the ping-pong ends
        # in X and no copy back is needed.
        if steps % 2 == 1:
            e.ns_normalize(X, Bt, m * n, float(eps), Y)
            cur, nxt = Y, X
        else:
            e.ns_normalize(X, Bt, m * n, float(eps))
        _count()
    wide = m <= n
    for _ in range(steps):
        if wide:
            gemm(cur, cur, trans_b=True, out=A, symmetric=True)                   # A = X X^T        (m x m)
            gemm(A, A, trans_b=True, alpha=C_COEF, beta=B_COEF, aux=A, out=Bm, symmetric=True)  # B = c A A + b A
            gemm(Bm, cur, alpha=1.0, beta=A_COEF, aux=cur, out=nxt, round_acc=True)  # X' = B X + a X
        else:
            gemm(cur, cur, trans_a=True, out=A, symmetric=True)                   # A = X^T X        (n x n)
            gemm(A, A, trans_b=True, alpha=C_COEF, beta=B_COEF, aux=A, out=Bm, symmetric=True)
            gemm(cur, Bm, alpha=1.0, beta=A_COEF, aux=cur, out=nxt, round_acc=True)  # X' = X B + a X
        cur, nxt = nxt, cur
    if cur is not X:
        X.copy_(cur)
    return X


def newton_schulz(G: torch.Tensor, steps: int = 5, workspace: NSWorkspace | None = None) -> torch.Tensor:
    """Orthogonalise the last two dims of ``G`` (2-D or batched 3-D); returns ``G``'s dtype."""
    assert G.ndim >= 2
    if not G.is_cuda:
        return ref.newton_schulz(G, steps=steps)
    shape = G.shape
    X = G.reshape(-1, shape[-2], shape[-1]).to(torch.bfloat16)
    if X.data_ptr() == G.data_ptr() or not X.is_contiguous():
        X = X.contiguous() if not X.is_contiguous() else X.clone()
    m, n = X.shape[-2:]
    if m % 8 or n % 8:
        # pad to the TMA granularity; zero rows/columns do not change the iteration
        pm, pn = (-m) % 8, (-n) % 8
        Xp = torch.nn.functional.pad(X, (0, pn, 0, pm))
        out = ns_inplace_cuda(_pre_normalized(Xp), steps, workspace=workspace, normalize=False)[:, :m, :n]
    else:
        out = ns_inplace_cuda(X, steps, workspace=workspace)
    return out.reshape(shape).to(G.dtype)


def _pre_normalized(X: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    norm = X.float().norm(dim=(-2, -1), keepdim=True)
    return (X.float() / (norm + eps)).to(torch.bfloat16).contiguous()
