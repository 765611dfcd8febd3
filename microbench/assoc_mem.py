"""Stateless operator engine for the associative-memory probes (CPU capable).

The reference's ``microbench/assoc_mem.py:1-831`` studies how much of a Zipf-weighted set of key -> value
associations one optimizer step recovers when the gradient is replaced by its (tile-local) orthogonalisation, at
several arithmetic precisions.  This module provides the same building blocks: the quintic Newton-Schulz operator
at a chosen precision (fp64 / fp32 / bf16 products / fp8-e4m3 products, simulated or on the GPU's fp8 tensor cores), matrix tiling
with square or rectangular tiles, the HiMuon operator, the synthetic problem in both of the reference's forms (the
compact ``zipf_problem`` and the ``sample_problem`` / ``build_gradient`` pair with population / minibatch and
approximate / exact-softmax gradients), and the recovery metrics (per item, by frequency rank, top-k curves,
operator gaps), plus result records for ``jsonl`` logs.
"""

from __future__ import annotations

import json
import math
import time
from dataclasses import asdict, dataclass
from pathlib import Path

import torch

from himuon_b200.ops import reference as ref

PRECISIONS = ("fp64_ref", "fp32", "bf16", "fp8e4m3_sim")
NS_PRECISIONS = PRECISIONS + ("fp8e4m3_native",)       # the last one needs a CUDA device with fp8 matmuls
RANK_FRACTIONS = (0.0, 0.01, 0.05, 0.10, 0.25, 0.50, 1.0)


def _precision_ops(ns_precision: str):
    """``(store, matmul)`` of a precision: ``store`` is applied to the input, to the normalised iterate and to every
    intermediate of the iteration (what a buffer of that precision would hold), ``matmul`` forms the products.

    * ``fp64_ref`` / ``fp32``: everything in that type;
    * ``bf16``: fp32 buffers, products of operands rounded to bf16 with fp32 accumulation (tensor-core semantics);
    * ``fp8e4m3_native``: fp32 buffers, products on the GPU's fp8 tensor cores (operands quantised per matrix);
    * ``fp8e4m3_sim``: the same arithmetic without fp8 hardware: both operands of every product are rounded through
      float8-e4m3 under a per-matrix scale and multiplied in fp32.  (The reference's simulated mode instead stores
      every *buffer* in fp8, which it does not use for its table; here the simulated mode tracks the native one, so
      that a machine without fp8 tensor cores reproduces the native column.)

    fp64 / fp32 / bf16 / native fp8 have the rounding points of the reference's engine
    (``microbench/assoc_mem.py:345-397``), so the operator gaps compare with its table."""
    if ns_precision == "fp64_ref":
        return (lambda t: t.double()), torch.matmul
    if ns_precision == "fp32":
        return (lambda t: t.float()), torch.matmul
    if ns_precision == "bf16":
        return (lambda t: t.float()), (lambda l, r: (l.to(torch.bfloat16) @ r.to(torch.bfloat16)).float())
    if ns_precision == "fp8e4m3_sim":
        return (lambda t: t.float()), (lambda l, r: _fp8_round_each(l) @ _fp8_round_each(r))
    if ns_precision == "fp8e4m3_native":
        return (lambda t: t.float()), _fp8_matmul_batched
    raise ValueError(f"unknown ns_precision {ns_precision!r}; choose from {NS_PRECISIONS}")


def _fp8_round_each(x: torch.Tensor) -> torch.Tensor:
    """Round-trip through float8-e4m3 with one scale per matrix of a (possibly batched) tensor."""
    x = x.float()
    amax = x.abs().amax(dim=(-2, -1), keepdim=True).clamp(min=1e-12)
    scale = 448.0 / amax
    return (x * scale).to(torch.float8_e4m3fn).float() / scale


def _fp8_matmul_batched(left: torch.Tensor, right: torch.Tensor) -> torch.Tensor:
    if left.ndim == 2:
        return fp8_matmul(left, right)
    return torch.stack([fp8_matmul(a, b) for a, b in zip(left.reshape(-1, *left.shape[-2:]), right.reshape(-1, *right.shape[-2:]))]
                       ).reshape(*left.shape[:-1], right.shape[-1])


def quintic_ns_operator(g: torch.Tensor, steps: int = 5, ns_precision: str = "fp32") -> torch.Tensor:
    """Newton-Schulz polar-factor approximation of the last two dims of ``g`` (2-D or batched) with every buffer and
    product held at the requested precision; returns ``g``'s dtype."""
    store, mm = _precision_ops(ns_precision)
    a, b, c = ref.NS_COEFFS
    X = store(g)
    tall = X.size(-2) > X.size(-1)
    if tall:
        X = X.transpose(-2, -1)
    X = store(X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7))
    for _ in range(steps):
        A = store(mm(X, X.transpose(-2, -1)))
        Bm = store(b * A + c * mm(A, A))
        X = store(a * X + mm(Bm, X))
    if tall:
        X = X.transpose(-2, -1)
    return X.to(g.dtype)


def fp8_matmul(left: torch.Tensor, right: torch.Tensor) -> torch.Tensor:
    """``left @ right`` with both operands quantised to float8-e4m3 under a per-tensor scale and multiplied by the
    GPU's fp8 tensor cores (``torch._scaled_mm``), fp32 result.  2-D CUDA operands whose sides are multiples of 16."""
    if not (left.is_cuda and right.is_cuda):
        raise RuntimeError("fp8e4m3_native needs CUDA tensors")
    if not hasattr(torch, "_scaled_mm") or not hasattr(torch, "float8_e4m3fn"):
        raise RuntimeError("fp8e4m3_native needs torch._scaled_mm and torch.float8_e4m3fn")
    tiny = torch.finfo(torch.float32).tiny
    lf, rf = left.float(), right.float()
    ls = (lf.abs().max() / 448.0).clamp(min=tiny)
    rs = (rf.abs().max() / 448.0).clamp(min=tiny)
    l8 = (lf / ls).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).contiguous()
    r8 = (rf / rs).clamp(-448.0, 448.0).t().contiguous().to(torch.float8_e4m3fn).t()      # column-major, as the op wants
    return torch._scaled_mm(l8, r8, scale_a=ls, scale_b=rs, out_dtype=torch.float32)


def _tile_hw(tile) -> tuple[int, int]:
    return (int(tile), int(tile)) if isinstance(tile, int) else (int(tile[0]), int(tile[1]))


def tile_matrix(g: torch.Tensor, tile):
    """``tile``: an int or a ``(tile_h, tile_w)`` pair."""
    return ref.tile(g, _tile_hw(tile))


def untile_matrix(tiled: torch.Tensor, info):
    return ref.untile(tiled, info)


def himuon_operator(g: torch.Tensor, tile: int | None, steps: int = 5, ns_precision: str = "fp32") -> torch.Tensor:
    """Tile-local orthogonalisation (``tile=None`` or a tile covering the matrix gives plain Muon)."""
    if tile is None:
        return quintic_ns_operator(g, steps, ns_precision)
    th, tw = _tile_hw(tile)
    if g.numel() <= th * tw:                     # the optimizer's own rule: small matrices are orthogonalised whole
        return quintic_ns_operator(g, steps, ns_precision)
    tiled, info = tile_matrix(g, (th, tw))
    R, C = tiled.shape[:2]
    orth = quintic_ns_operator(tiled.reshape(R * C, th, tw), steps, ns_precision).reshape(tiled.shape)
    return untile_matrix(orth, info)


def apply_one_step(g: torch.Tensor, optimizer: str, eta: float, ns_steps: int = 5, tile=256, ns_precision: str = "fp32"):
    """``eta * update`` for ``sgd`` (the gradient), ``muon`` (full-matrix NS) or ``himuon`` (tile-local NS)."""
    if optimizer == "sgd":
        return eta * g.float()
    if optimizer == "muon":
        return eta * quintic_ns_operator(g, ns_steps, ns_precision).float()
    if optimizer == "himuon":
        return eta * himuon_operator(g, tile, ns_steps, ns_precision).float()
    raise ValueError(f"unknown optimizer {optimizer!r}")


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


# ------------------------------------------------------------------------------------------- full problem model
@dataclass(frozen=True)
class ProblemSpec:
    d: int
    num_items: int
    frequency_mode: str
    alpha: float
    seed: int
    device: str
    dtype: str


@dataclass
class ProblemInstance:
    """``u`` / ``v``: the ``(num_items, d)`` item embeddings on the output / input side, ``p``: item frequencies."""
    spec: ProblemSpec
    u: torch.Tensor
    v: torch.Tensor
    p: torch.Tensor
    mean_u: torch.Tensor

    @property
    def d(self) -> int:
        return self.spec.d

    @property
    def num_items(self) -> int:
        return self.spec.num_items


def make_frequencies(num_items: int, mode: str = "power_law", alpha: float = 1.5, device="cpu", dtype=torch.float32):
    if mode == "uniform":
        return torch.full((num_items,), 1.0 / num_items, device=device, dtype=dtype)
    if mode == "power_law":
        w = torch.arange(1, num_items + 1, device=device, dtype=dtype).pow(-alpha)
        return w / w.sum()
    raise ValueError(f"unknown frequency mode {mode!r}")


def sample_problem(d: int, num_items: int | None = None, frequency_mode: str = "power_law", alpha: float = 1.5,
                   seed: int = 0, device: str = "cpu", dtype=torch.float32) -> ProblemInstance:
    """Gaussian embeddings of variance 1/d; by default ``max(512, 4 d)`` items."""
    n = int(num_items) if num_items is not None else max(512, 4 * d)
    gen = torch.Generator(device=device).manual_seed(seed)
    u = torch.randn(n, d, generator=gen, device=device, dtype=dtype) / math.sqrt(d)
    v = torch.randn(n, d, generator=gen, device=device, dtype=dtype) / math.sqrt(d)
    p = make_frequencies(n, frequency_mode, alpha, device, dtype)
    spec = ProblemSpec(d, n, frequency_mode, alpha, seed, str(device), str(dtype).replace("torch.", ""))
    return ProblemInstance(spec, u, v, p, u.mean(dim=0))


def estimate_peak_memory_bytes(d: int, num_items: int, score_chunk: int = 256, tile=None, n_weights: int = 1) -> int:
    """Coarse upper bound of the tensor memory one configuration needs (fp32 working precision)."""
    chunk = min(score_chunk, num_items)
    problem = (2 * num_items * d + 2 * num_items + d) * 4
    scores = (num_items * chunk + 2 * chunk * d + 2 * num_items) * 4
    if tile is None:
        op = 2 * d * d * 4
    else:
        th, tw = _tile_hw(tile)
        op = 2 * (-(-d // th) * th) * (-(-d // tw) * tw) * 4
    return problem + scores + op + (1 + n_weights) * d * d * 4


def assert_memory_budget(budget_gib: float, **kw) -> float:
    need = estimate_peak_memory_bytes(**kw) / float(1 << 30)
    if need > budget_gib:
        raise MemoryError(f"configuration needs about {need:.2f} GiB, budget is {budget_gib:.2f} GiB: {kw}")
    return need


def sample_empirical_frequencies(p: torch.Tensor, batch_size: int, seed: int) -> torch.Tensor:
    gen = torch.Generator(device=p.device).manual_seed(seed)
    idx = torch.multinomial(p, batch_size, replacement=True, generator=gen)
    return torch.bincount(idx, minlength=p.numel()).to(p.dtype) / batch_size


def build_gradient(problem: ProblemInstance, gradient_mode: str, batch_size: int | None = None, seed: int | None = None,
                   weight: torch.Tensor | None = None, score_chunk: int = 256):
    """Descent direction ``sum_i f_i (u_i - E[u]) v_i^T`` of the softmax retrieval loss.

    ``approx_*`` drops the expectation, ``true_*`` uses the uniform mean at ``W = 0`` or, when ``weight`` is given,
    the softmax expectation under the current ``W``; ``*_population`` weights by the true frequencies,
    ``*_minibatch`` by the empirical frequencies of ``batch_size`` draws."""
    if gradient_mode not in ("approx_population", "true_population", "approx_minibatch", "true_minibatch"):
        raise ValueError(f"unknown gradient mode {gradient_mode!r}")
    if gradient_mode.endswith("minibatch"):
        if batch_size is None or seed is None:
            raise ValueError(f"{gradient_mode} needs batch_size and seed")
        freqs = sample_empirical_frequencies(problem.p, batch_size, seed)
    else:
        freqs = problem.p
    exact = gradient_mode.startswith("true_")
    if exact and weight is not None:
        u, v, w = problem.u.float(), problem.v.float(), weight.float()
        grad = torch.zeros(problem.d, problem.d, device=w.device)
        for s0 in range(0, problem.num_items, score_chunk):
            vc = v[s0:s0 + score_chunk]
            logits = u @ (vc @ w.t()).t()                         # (items, chunk): score of every item for each query
            probs = torch.softmax(logits - logits.max(dim=0, keepdim=True).values, dim=0)
            centred = u[s0:s0 + score_chunk] - probs.t() @ u
            grad += (freqs[s0:s0 + score_chunk, None].float() * centred).t() @ vc
    else:
        centred = problem.u - problem.mean_u if exact else problem.u
        grad = (freqs[:, None] * centred).t() @ problem.v
    nz = freqs[freqs > 0]
    meta = {"gradient_mode": gradient_mode, "batch_size": batch_size, "gradient_seed": seed,
            "gradient_depends_on_weight": bool(exact and weight is not None), "effective_support": int(nz.numel()),
            "freq_max": float(freqs.max()), "freq_min_nonzero": float(nz.min())}
    return grad, meta


def evaluate_recovery(problem: ProblemInstance, weight: torch.Tensor, score_chunk: int = 256):
    """Per item: recovered iff ``u_i^T W v_i`` beats every other item's score for query ``v_i``; also the margin."""
    u, v, w = problem.u.float(), problem.v.float(), weight.float()
    n = problem.num_items
    ok = torch.zeros(n, dtype=torch.bool)
    margin = torch.empty(n)
    for s0 in range(0, n, score_chunk):
        s1 = min(n, s0 + score_chunk)
        scores = u @ (v[s0:s1] @ w.t()).t()                       # (n, chunk)
        cols = torch.arange(s1 - s0, device=scores.device)
        rows = torch.arange(s0, s1, device=scores.device)
        own = scores[rows, cols].clone()
        scores[rows, cols] = float("-inf")
        best_other = scores.max(dim=0).values
        ok[s0:s1] = (own > best_other).cpu()
        margin[s0:s1] = (own - best_other).cpu()
    return ok, margin


def frequency_rank_summary(problem: ProblemInstance, recovered: torch.Tensor, fractions=RANK_FRACTIONS) -> dict:
    """Recovery by frequency rank: for each band of ranks (and each prefix) the share of items and of probability
    mass that was recovered."""
    fr = tuple(float(f) for f in fractions)
    if not fr or fr[0] != 0.0 or fr[-1] != 1.0:
        raise ValueError("fractions must start at 0.0 and end at 1.0")
    p = problem.p.float().cpu()
    order = torch.argsort(p, descending=True)
    ps, rs = p[order], recovered.float().cpu()[order]
    n = p.numel()
    bounds, prev = [0], 0
    for f in fr[1:]:
        prev = min(n, max(prev, math.ceil(f * n)))
        bounds.append(prev)
    bins, prefixes = [], []
    for (f0, f1), (b0, b1) in zip(zip(fr[:-1], fr[1:]), zip(bounds[:-1], bounds[1:])):
        if b1 > b0:
            bins.append({"label": f"{100 * f0:g}%-{100 * f1:g}%", "start": b0, "end": b1, "items": b1 - b0,
                         "recovered_fraction": float(rs[b0:b1].mean()), "probability_mass": float(ps[b0:b1].sum()),
                         "recovered_probability_mass": float((ps[b0:b1] * rs[b0:b1]).sum())})
        if b1 > 0:
            prefixes.append({"label": f"top {100 * f1:g}%", "items": b1, "recovered_fraction": float(rs[:b1].mean()),
                             "recovered_probability_mass": float((ps[:b1] * rs[:b1]).sum())})
    return {"recovered_probability_mass": float((ps * rs).sum()), "total_probability_mass": float(ps.sum()),
            "bins": bins, "prefixes": prefixes}


def topk_recovery_curve(problem: ProblemInstance, weight: torch.Tensor, max_k: int | None = None,
                        order: str = "frequency_desc", score_chunk: int = 256) -> dict:
    """Fraction of the ``k`` most frequent (or first ``k``) items recovered, for every ``k`` up to ``max_k``."""
    ok, _ = evaluate_recovery(problem, weight, score_chunk)
    if order == "frequency_desc":
        idx = torch.argsort(problem.p.float().cpu(), descending=True)
    elif order == "index":
        idx = torch.arange(problem.num_items)
    else:
        raise ValueError(f"unknown order {order!r}")
    lim = problem.num_items if max_k is None else min(problem.num_items, int(max_k))
    counts = torch.cumsum(ok.float()[idx][:lim], 0)
    frac = counts / torch.arange(1, lim + 1)
    return {"order": order, "max_k": lim, "k_values": list(range(1, lim + 1)),
            "topk_recovered_count": counts.tolist(), "topk_recovered_fraction": frac.tolist()}


def recovery_metrics(problem: ProblemInstance, weight: torch.Tensor, topk_values=(32, 128, 512), score_chunk: int = 256) -> dict:
    w = weight.float()
    ok, margin = evaluate_recovery(problem, w, score_chunk)
    n, k_ok = problem.num_items, int(ok.sum())
    fails = torch.nonzero(~ok)
    by_rank = frequency_rank_summary(problem, ok)
    sv = torch.linalg.svdvals(w)
    out = {"recovered_count": k_ok, "recovered_fraction": k_ok / n,
           "recovered_probability_mass": by_rank["recovered_probability_mass"],
           "first_failure_rank": None if fails.numel() == 0 else int(fails[0, 0]) + 1,
           "mean_margin_all": float(margin.mean()), "mean_margin_recovered": float(margin[ok].mean()) if k_ok else None,
           "weight_fro_norm": float(w.norm()), "weight_spectral_norm": float(sv[0]),
           "weight_top_singular_values": [float(x) for x in sv[:6]], "frequency_rank_summary": by_rank}
    freq_order = torch.argsort(problem.p.float().cpu(), descending=True)
    for name, seq in (("top", ok), ("freq_top", ok[freq_order])):
        for k in dict.fromkeys(int(k) for k in topk_values):
            kk = min(k, n)
            out[f"{name}_{k}_effective_k"] = kk
            out[f"{name}_{k}_recovered_count"] = int(seq[:kk].sum())
            out[f"{name}_{k}_recovered_fraction"] = float(seq[:kk].float().mean()) if kk else None
    return out


def operator_gap_metrics(reference: torch.Tensor, candidate: torch.Tensor) -> dict:
    r, c = reference.float(), candidate.float()
    denom = float(r.norm() * c.norm())
    gap = float((r - c).norm())
    return {"operator_cosine_similarity": float((r * c).sum()) / denom if denom > 0 else None,
            "operator_fro_gap": gap, "operator_relative_fro_gap": gap / (float(r.norm()) + 1e-12),
            "operator_spectral_norm_gap": abs(float(torch.linalg.matrix_norm(r, ord=2)) - float(torch.linalg.matrix_norm(c, ord=2)))}


def benchmark_operator_runtime(fn, *args, warmup: int = 3, iters: int = 10, **kw) -> dict:
    """Mean / min wall time of ``fn(*args, **kw)`` in milliseconds (device-synchronised when CUDA is in use)."""
    cuda = torch.cuda.is_available()
    for _ in range(warmup):
        fn(*args, **kw)
    times = []
    for _ in range(iters):
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn(*args, **kw)
        if cuda:
            torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3)
    return {"runtime_ms_mean": sum(times) / len(times), "runtime_ms_min": min(times), "runtime_iters": iters}


def make_result_record(problem: ProblemInstance, optimizer: str, eta: float, metrics: dict, **extra) -> dict:
    """One flat record per (problem, optimizer, setting) for the jsonl logs of the probes."""
    rec = {"timestamp": time.time(), **{f"problem_{k}": v for k, v in asdict(problem.spec).items()},
           "optimizer": optimizer, "eta": eta}
    rec.update(extra)
    rec.update(metrics)
    return rec


def write_jsonl(path, records, append: bool = True) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("a" if append else "w") as f:
        for r in records:
            f.write(json.dumps(r) + "\n")


def summarize_records(records: list[dict]) -> dict:
    """Mean recovered fraction and probability mass per optimizer over a list of records."""
    groups: dict[str, list[dict]] = {}
    for r in records:
        groups.setdefault(str(r.get("optimizer")), []).append(r)
    return {k: {"runs": len(v), "recovered_fraction_mean": sum(x["recovered_fraction"] for x in v) / len(v),
                "recovered_probability_mass_mean": sum(x["recovered_probability_mass"] for x in v) / len(v)}
            for k, v in groups.items()}
