"""Plain PyTorch implementations of every op in :mod:`himuon_b200.ops`.

They are the numerical oracle for the CUDA kernels and the execution path on CPU
(unit-test tier, fp32 regression run).  Rounding points of the Newton-Schulz iteration
follow the reference's fused kernel (``src/himuon/triton_kernels/ns5_smem.py:84-101``):
fp32 Frobenius norm, then every product is rounded to the compute dtype.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(G: torch.Tensor, steps: int = 5, compute_dtype: torch.dtype = torch.bfloat16,
                  eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation of the last two dims of ``G``.

    Transposes tall matrices, normalises by the Frobenius norm (+eps), runs ``steps``
    iterations of ``X <- aX + (bA + cA^2)X`` with ``A = X X^T`` and returns the result in
    ``G``'s dtype (``src/himuon/optimizers/himuon.py:232-284``).
    """
    assert G.ndim >= 2
    a, b, c = NS_COEFFS
    wide = compute_dtype in (torch.float32, torch.float64)

    def mm(x, y):  # product with fp32 accumulation, rounded to the compute dtype
        return x @ y if wide else (x.float() @ y.float()).to(compute_dtype)

    X = G.to(compute_dtype)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.transpose(-2, -1)
    acc = torch.float64 if compute_dtype == torch.float64 else torch.float32
    norm = X.to(acc).norm(dim=(-2, -1), keepdim=True)
    X = (X.to(acc) / (norm + eps)).to(compute_dtype)
    for _ in range(steps):
        A = mm(X, X.transpose(-2, -1))
        Bm = (c * (A.to(acc) @ A.to(acc)) + b * A.to(acc)).to(compute_dtype)
        X = (mm(Bm, X).to(acc) + a * X.to(acc)).to(compute_dtype)
    if tall:
        X = X.transpose(-2, -1)
    return X.to(G.dtype)


def tile(t: torch.Tensor, tile_size) -> tuple[torch.Tensor, tuple[int, int, int, int]]:
    """``(H, W) -> (R, C, Th, Tw)`` with zero padding at the bottom/right (``himuon.py:289-300``)."""
    th, tw = tile_size
    h, w = t.shape
    pad_h = (th - h % th) % th
    pad_w = (tw - w % tw) % tw
    if pad_h or pad_w:
        t = F.pad(t, (0, pad_w, 0, pad_h))
    R, C = t.shape[0] // th, t.shape[1] // tw
    return t.view(R, th, C, tw).permute(0, 2, 1, 3).contiguous(), (h, w, pad_h, pad_w)


def untile(tiled: torch.Tensor, info) -> torch.Tensor:
    """Inverse of :func:`tile` including the crop (``himuon.py:303-311``)."""
    h, w, pad_h, pad_w = info
    R, C, th, tw = tiled.shape
    out = tiled.permute(0, 2, 1, 3).contiguous().view(R * th, C * tw)
    return out[:h, :w] if (pad_h or pad_w) else out


def rmsnorm(x, w, eps):
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return y * w


def rope_tables(seq_len: int, head_dim: int, theta: float, device=None) -> torch.Tensor:
    """``(seq_len, head_dim/2, 2)`` fp32 table of (cos, sin)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.arange(seq_len, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()


def apply_rope(x: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on ``(B, S, H, D)`` with positions ``0..S-1``."""
    D = x.size(-1)
    S = x.size(1)
    cos = torch.cat([cos_sin[:S, :, 0], cos_sin[:S, :, 0]], -1)[None, :, None, :]
    sin = torch.cat([cos_sin[:S, :, 1], cos_sin[:S, :, 1]], -1)[None, :, None, :]
    xf = x.float()
    rot = torch.cat([-xf[..., D // 2:], xf[..., : D // 2]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


def attention(q, k, v, scale=None):
    """Causal grouped-query attention on ``(B, S, H, D)`` tensors."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qh = q.transpose(1, 2)
    kh = k.transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    vh = v.transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale)
    return out.transpose(1, 2).contiguous()


def swiglu(gate, up):
    return F.silu(gate) * up


def linear_cross_entropy(h, w, labels, ignore_index=-100):
    """Mean token cross-entropy of ``h @ w.T`` in fp32 (HF ``ForCausalLMLoss`` after the shift)."""
    logits = (h @ w.t()).float()
    return F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction="mean")
