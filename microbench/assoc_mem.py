"""Stateless operator engine for the associative-memory probes (CPU capable).

The reference's ``microbench/assoc_mem.py:1-831`` studies how much of a Zipf-weighted set of key -> value
associations one optimizer step recovers when the gradient is replaced by its (tile-local) orthogonalisation, at
several arithmetic precisions.  This module provides the same building blocks: the quintic Newton-Schulz operator
at a chosen precision (fp64 / fp32 / bf16 / simulated fp8-e4m3), matrix tiling, the HiMuon operator, the synthetic
problem and the recovery metrics.
"""

from __future__ import annotations

import torch

from himuon_b200.ops import reference as ref

PRECISIONS = ("fp64_ref", "fp32", "bf16", "fp8e4m3_sim")


def _fp8_round(x: torch.Tensor) -> torch.Tensor:
    """Round-trip through float8_e4m3 with a per-tensor scale (simulates an fp8 matmul operand)."""
    amax = x.abs().max().clamp(min=1e-12)
    scale = 448.0 / amax
    return (x * scale).to(torch.float8_e4m3fn).to(x.dtype) / scale


def quintic_ns_operator(g: torch.Tensor, steps: int = 5, ns_precision: str = "fp32") -> torch.Tensor:
    """Newton-Schulz polar-factor approximation of the last two dims of ``g`` at the requested precision."""
    if ns_precision == "fp64_ref":
        return ref.newton_schulz(g.double(), steps, compute_dtype=torch.float64).to(g.dtype)
    if ns_precision == "fp32":
        return ref.newton_schulz(g.float(), steps, compute_dtype=torch.float32).to(g.dtype)
    if ns_precision == "bf16":
        return ref.newton_schulz(g.float(), steps, compute_dtype=torch.bfloat16).to(g.dtype)
    if ns_precision == "fp8e4m3_sim":
        a, b, c = ref.NS_COEFFS
        X = g.float()
        tall = X.size(-2) > X.size(-1)
        if tall:
            X = X.transpose(-2, -1)
        X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
        for _ in range(steps):
            Xq = _fp8_round(X)
            A = Xq @ Xq.transpose(-2, -1)
            Aq = _fp8_round(A)
            Bm = b * A + c * (Aq @ Aq)
            X = a * X + _fp8_round(Bm) @ Xq
        if tall:
            X = X.transpose(-2, -1)
        return X.to(g.dtype)
    raise ValueError(f"unknown ns_precision {ns_precision!r}; choose from {PRECISIONS}")


def tile_matrix(g: torch.Tensor, tile: int):
    return ref.tile(g, (tile, tile))


def untile_matrix(tiled: torch.Tensor, info):
    return ref.untile(tiled, info)


def himuon_operator(g: torch.Tensor, tile: int | None, steps: int = 5, ns_precision: str = "fp32") -> torch.Tensor:
    """Tile-local orthogonalisation (``tile=None`` or a tile covering the matrix gives plain Muon)."""
    if tile is None or tile >= max(g.shape):
        return quintic_ns_operator(g, steps, ns_precision)
    tiled, info = tile_matrix(g, tile)
    R, C = tiled.shape[:2]
    orth = quintic_ns_operator(tiled.reshape(R * C, tile, tile), steps, ns_precision).reshape(tiled.shape)
    return untile_matrix(orth, info)


def zipf_problem(d: int, n_items: int, alpha: float = 1.5, batch: int | None = None, seed: int = 0, device="cpu"):
    """Random unit keys / values and Zipf(alpha) frequencies; returns ``(keys, values, freqs, gradient)`` where the
    gradient of the linear associative memory at W = 0 is ``sum_i f_i v_i k_i^T`` (sampled when ``batch`` is given)."""
    g = torch.Generator().manual_seed(seed)
    keys = torch.nn.functional.normalize(torch.randn(n_items, d, generator=g), dim=1).to(device)
    vals = torch.nn.functional.normalize(torch.randn(n_items, d, generator=g), dim=1).to(device)
    freqs = torch.arange(1, n_items + 1, dtype=torch.float64).pow(-alpha)
    freqs = (freqs / freqs.sum()).float().to(device)
    if batch is None:
        weights = freqs
    else:
        idx = torch.multinomial(freqs.cpu(), batch, replacement=True, generator=g)
        weights = torch.bincount(idx, minlength=n_items).float().to(device) / batch
    grad = (vals * weights[:, None]).t() @ keys
    return keys, vals, freqs, grad


def recovered_items(update: torch.Tensor, keys: torch.Tensor, vals: torch.Tensor, margin: float = 0.0) -> int:
    """Items whose value is the arg-max read-out of ``update @ key`` among all stored values."""
    read = keys @ update.t()                    # (n, d): W k_i
    scores = read @ vals.t()                    # (n, n)
    correct = scores.argmax(dim=1) == torch.arange(keys.shape[0], device=keys.device)
    if margin > 0:
        top2 = scores.topk(2, dim=1).values
        correct &= (top2[:, 0] - top2[:, 1]) > margin
    return int(correct.sum())


def topk_recovery(update, keys, vals, ks=(1, 5, 10)):
    scores = (keys @ update.t()) @ vals.t()
    ranks = (scores > scores.diag()[:, None]).sum(dim=1)
    return {k: float((ranks < k).float().mean()) for k in ks}


def relative_operator_error(g: torch.Tensor, tile, steps: int, ns_precision: str) -> float:
    """``delta_F``: relative Frobenius distance of the operator at ``ns_precision`` from its fp64 evaluation."""
    ref64 = himuon_operator(g.double(), tile, steps, "fp64_ref")
    out = himuon_operator(g, tile, steps, ns_precision).double()
    return float((out - ref64).norm() / ref64.norm())
