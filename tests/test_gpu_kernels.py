"""Raw sm_100a kernels against plain PyTorch fp32 references (GPU tier).

Covers the tcgen05 GEMM in all four operand-major combinations, the fused tile-resident
NS5 kernel, the optimizer multi-tensor kernels, the HBM-bound model kernels and flash
attention forward/backward.  Mirrors the role of the reference's
tests/integration/test_kernels.py (kernels vs pure torch at bf16 tolerance).
"""

import math
import struct

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
    from himuon_b200._ext import ext

    return ext()


def _assert_status_clean():
    assert _ext().status(True) == 0, "a bounded device wait ran out (status word set)"


def _close(out, ref, atol, rtol):
    out = out.float()
    ref = ref.float()
    err = (out - ref).abs()
    tol = atol + rtol * ref.abs()
    # Every element is checked.  A few per hundred thousand may exceed the tolerance (rounding of a value that sits on
    # a bf16 boundary), none may exceed it four-fold, and no single row or column may collect the outliers: a wrong
    # boundary row or tile edge fails even when it is a vanishing share of the matrix.
    over = err > tol
    bad = over.float().mean().item()
    assert bad <= 1e-5, f"{bad:.4%} elements out of tolerance; max err {err.max().item():.4g}, ref max {ref.abs().max().item():.4g}"
    worst = (err / tol).max().item()
    assert worst <= 4.0, f"an element is {worst:.1f}x outside the tolerance (max err {err.max().item():.4g})"
    if over.dim() >= 2 and over.any():
        per_row = over.reshape(-1, over.shape[-1]).float().mean(dim=1).max().item()
        per_col = over.reshape(-1, over.shape[-2], over.shape[-1]).float().mean(dim=1).max().item()
        assert per_row <= 0.02 and per_col <= 0.02, f"outliers concentrate in one row/column ({per_row:.2%} / {per_col:.2%})"


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 512, 384), (128, 128, 64), (200, 328, 136), (1024, 2560, 1024), (520, 776, 2304),
                                   (2048, 2560, 4096)])
def test_gemm_majors(trans_a, trans_b, shape):
    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn((K, M) if trans_a else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((N, K) if trans_b else (K, N), device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _ext().gemm(a, b, out, None, trans_a, trans_b, 1.0, 0.0, False, 0)
    ref = (a.float().t() if trans_a else a.float()) @ (b.float().t() if trans_b else b.float())
    torch.cuda.synchronize()
    _assert_status_clean()
    _close(out, ref, atol=0.25, rtol=2e-2)


def test_gemm_batched_epilogue_and_fp32_accumulate():
    torch.manual_seed(1)
    B, M, N, K = 5, 256, 320, 192
    a = torch.randn(B, M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(B, N, K, device="cuda", dtype=torch.bfloat16)
    aux = torch.randn(B, M, N, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(aux)
    _ext().gemm(a, b, out, aux, False, True, 0.5, -1.5, False, 0)
    ref = 0.5 * torch.bmm(a.float(), b.float().transpose(1, 2)) - 1.5 * aux.float()
    _close(out, ref, atol=0.25, rtol=2e-2)
    # fp32 output accumulating into itself (weight-gradient accumulation)
    acc = torch.randn(B, M, N, device="cuda", dtype=torch.float32)
    ref2 = acc.clone() + torch.bmm(a.float(), b.float().transpose(1, 2))
    _ext().gemm(a, b, acc, acc, False, True, 1.0, 1.0, False, 0)
    torch.cuda.synchronize()
    _assert_status_clean()
    _close(acc, ref2, atol=1e-2, rtol=1e-3)


@pytest.mark.parametrize("M,N,K", [(2048, 2560, 2560), (2000, 2560, 9728), (2560, 2304, 2048), (11520, 2560, 4096)])
def test_gemm_pair_split_tail(M, N, K):
    """Shapes whose last wave of 256x256 tiles is mostly idle: the tail tiles are cut along K, summed in an fp32
    scratch by TMA reductions and finished by a second kernel.  Run twice (the scratch must come back zeroed), with
    the aux epilogue and with fp32 accumulation into the output."""
    torch.manual_seed(2)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    aux = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    for _ in range(2):
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        _ext().gemm(a, b, out, None, False, True, 1.0, 0.0, False, 0)
        _close(out, ref, atol=0.3, rtol=2e-2)
        out2 = torch.empty_like(out)
        _ext().gemm(a, b, out2, aux, False, True, 0.5, -1.5, False, 0)
        _close(out2, 0.5 * ref - 1.5 * aux.float(), atol=0.3, rtol=2e-2)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    ref2 = acc + ref
    _ext().gemm(a, b, acc, acc, False, True, 1.0, 1.0, False, 0)
    torch.cuda.synchronize()
    _assert_status_clean()
    _close(acc, ref2, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("M,N,K", [(2048, 2560, 2048), (4096, 2560, 2048), (2560, 9728, 2048), (2304, 2560, 4096),
                                   (19456, 2560, 2048)])
def test_gemm_pair_stream_k_accumulate(M, N, K):
    """fp32 `C += A^T B` (the weight-gradient GEMM) on shapes whose tile count does not fill the last wave: the work is
    dealt out as contiguous (tile, k-block) ranges and every partial tile is added into C by TMA reductions."""
    torch.manual_seed(3)
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    ref = acc.clone()
    prod = a.float().t() @ b.float()
    for i in range(2):
        _ext().gemm(a, b, acc, acc, True, False, 1.0, 1.0, False, 0)
        ref += prod
        _close(acc, ref, atol=2e-2, rtol=1e-3)
    torch.cuda.synchronize()
    _assert_status_clean()
    # bf16 accumulator (the banks' gradient buffers): every partial is rounded to bf16 and added in bf16
    acc16 = torch.randn(M, N, device="cuda", dtype=torch.float32).mul_(30).bfloat16()
    ref16 = acc16.float()
    for i in range(2):
        _ext().gemm(a, b, acc16, acc16, True, False, 1.0, 1.0, False, 0)
        ref16 = (ref16 + prod).bfloat16().float()
    torch.cuda.synchronize()
    _assert_status_clean()
    _close(acc16, ref16, atol=2.0, rtol=2e-2)


def _ns_ref(x, steps=5):
    a, b, c = 3.4445, -4.7750, 2.0315
    X = x.float()
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    X = X.bfloat16().float()
    for _ in range(steps):
        A = (X @ X.transpose(-2, -1)).bfloat16().float()
        Bm = (c * (A @ A) + b * A).bfloat16().float()
        X = ((Bm @ X).bfloat16().float() + a * X).bfloat16().float()
    return X


def _well_conditioned(B, m, n, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(B, m, n, generator=g)
    U, _, Vh = torch.linalg.svd(x, full_matrices=False)
    s = torch.linspace(0.8, 1.2, min(m, n))
    return (U * s) @ Vh


@pytest.mark.parametrize("m,n", [(128, 128), (64, 128), (64, 256), (32, 64), (128, 256)])
def test_ns5_fused(m, n):
    x = _well_conditioned(37, m, n).cuda().bfloat16()
    out = torch.empty_like(x)
    _ext().ns5_fused(x, out, 5, 1e-7)
    torch.cuda.synchronize()
    _assert_status_clean()
    _close(out, _ns_ref(x), atol=4e-2, rtol=4e-2)
    # an all-zero (padding) tile stays exactly zero
    z = torch.zeros(3, m, n, device="cuda", dtype=torch.bfloat16)
    oz = torch.empty_like(z)
    _ext().ns5_fused(z, oz, 5, 1e-7)
    assert oz.abs().max().item() == 0.0


def test_ns_normalize():
    x = torch.randn(9, 256, 512, device="cuda", dtype=torch.bfloat16)
    x[3].zero_()
    ref = x.float() / (x.float().norm(dim=(1, 2), keepdim=True) + 1e-7)
    _ext().ns_normalize(x, 9, 256 * 512, 1e-7)
    _close(x, ref, atol=1e-4, rtol=1e-2)
    assert x[3].abs().max().item() == 0.0


def test_momentum_tile_and_untile_apply():
    e = _ext()
    torch.manual_seed(0)
    Th = Tw = 128
    shapes = [(256, 384), (200, 300), (64, 64)]
    mu, lr, wd = 0.95, 0.02, 0.1
    grads = [torch.randn(s, device="cuda", dtype=torch.bfloat16) for s in shapes]
    moms = [torch.randn(s, device="cuda", dtype=torch.bfloat16) * 0.1 for s in shapes]
    params = [torch.randn(s, device="cuda", dtype=torch.bfloat16) for s in shapes]
    moms_ref = [m.clone() for m in moms]
    params_ref = [p.clone() for p in params]
    sz = e.sizeof_entries()
    assert sz[0] == 104 and sz[1] == 48 and sz[2] == 56
    mom_tab, app_tab = b"", b""
    tile_base, unit = 0, 0
    metas = []
    for g, m, p in zip(grads, moms, params):
        h, w = g.shape
        R, C = math.ceil(h / Th), math.ceil(w / Tw)
        mom_tab += struct.pack("<8QQq6i", g.data_ptr(), 0, 0, 0, 0, 0, 0, 0, m.data_ptr(), tile_base, h, w, R, C, unit, g.stride(0))
        app_tab += struct.pack("<Qq6ifi", p.data_ptr(), tile_base, h, w, R, C, unit, 0, 0.2 * math.sqrt(max(Th, Tw)), p.stride(0))
        metas.append((tile_base, R, C))
        tile_base += R * C
        unit += e.momentum_tile_units(R, C, Th)
    mom_dev = torch.frombuffer(bytearray(mom_tab), dtype=torch.uint8).cuda()
    app_dev = torch.frombuffer(bytearray(app_tab), dtype=torch.uint8).cuda()
    tiles = torch.full((tile_base, Th, Tw), 7.0, device="cuda", dtype=torch.bfloat16)
    e.momentum_tile(mom_dev, len(shapes), unit, Th, Tw, tiles, mu, True, 1.0, 1, False)
    for g, m_ref, m, (tb, R, C) in zip(grads, moms_ref, moms, metas):
        buf = m_ref.mul(mu).add(g)
        nes = g.add(buf, alpha=mu)
        _close(m, buf, atol=1e-2, rtol=1e-2)
        h, w = g.shape
        padded = torch.zeros(R * Th, C * Tw, device="cuda", dtype=torch.bfloat16)
        padded[:h, :w] = nes
        ref_tiles = padded.view(R, Th, C, Tw).permute(0, 2, 1, 3).reshape(R * C, Th, Tw)
        _close(tiles[tb:tb + R * C], ref_tiles, atol=2e-2, rtol=1e-2)
    hyper = torch.tensor([lr, wd], device="cuda", dtype=torch.float32)
    e.untile_apply(app_dev, len(shapes), unit, Th, Tw, tiles, hyper, False)
    for p_ref, p, (tb, R, C) in zip(params_ref, params, metas):
        h, w = p.shape
        u = tiles[tb:tb + R * C].view(R, C, Th, Tw).permute(0, 2, 1, 3).reshape(R * Th, C * Tw)[:h, :w]
        ref = p_ref.float() * (1 - lr * wd) - lr * 0.2 * math.sqrt(128) * u.float()
        _close(p, ref, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_adamw_multi(mode):
    e = _ext()
    torch.manual_seed(0)
    sizes = [5000, 17, 4096 * 3]
    lr, wd, b1, b2, eps = 1e-2, 0.1, 0.9, 0.95, 1e-8
    ps = [torch.randn(n, device="cuda") for n in sizes]
    gs = [torch.randn(n, device="cuda") for n in sizes]
    ms = [torch.zeros(n, device="cuda") for n in sizes]
    vs = [torch.zeros(n, device="cuda") for n in sizes]
    ref_p = [p.clone() for p in ps]
    tab, unit = b"", 0
    for p, g, m, v in zip(ps, gs, ms, vs):
        tab += struct.pack("<4Qqq2i", p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), unit, 0, 0)
        unit += (p.numel() + 4095) // 4096
    dev = torch.frombuffer(bytearray(tab), dtype=torch.uint8).cuda()
    hyper = torch.tensor([lr, wd, b1, b2, eps, 0, 0, 0], device="cuda", dtype=torch.float32)
    step = torch.zeros((), device="cuda", dtype=torch.float32)
    rm = [torch.zeros_like(p) for p in ps]
    rv = [torch.zeros_like(p) for p in ps]
    for t in range(1, 4):
        e.adamw_multi(dev, len(sizes), unit, hyper, step, mode, True, True)
        e.adamw_step_advance(step)
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
        for p, g, m, v in zip(ref_p, gs, rm, rv):
            m.lerp_(g, 1 - b1)
            v.lerp_(g * g, 1 - b2)
            if mode == 0:
                u = (m / bc1) / (v.sqrt() / math.sqrt(bc2) + eps)
                p.mul_(1 - lr * wd).sub_(lr * u)
            elif mode == 1:
                u = m / (eps + v.sqrt())
                p.mul_(1 - lr * wd).sub_(u * (lr / (bc1 / math.sqrt(bc2))))
            else:
                p.sub_(m / (v.sqrt() + eps) * (lr * math.sqrt(bc2) / bc1))
                p.sub_(p * (lr * wd))
    assert step.item() == 3.0
    for p, r in zip(ps, ref_p):
        _close(p, r, atol=1e-5, rtol=1e-4)


def test_rmsnorm_fwd_bwd():
    e = _ext()
    torch.manual_seed(0)
    rows, cols = 777, 2560
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).bfloat16()
    dy = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device="cuda")
    e.rmsnorm_fwd(x, w, y, rstd, 1e-6)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    yr.backward(dy.float())
    _close(y, yr, atol=2e-2, rtol=2e-2)
    dx = torch.empty_like(x)
    dw = torch.zeros(cols, device="cuda")
    e.rmsnorm_bwd(dy, x, w, rstd, dx, dw)
    _close(dx, xr.grad, atol=2e-2, rtol=2e-2)
    _close(dw, wr.grad, atol=0.3, rtol=2e-2)


def _rope_table(S, theta=1e6, D=128):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()  # (S, 64, 2)


def test_add_rmsnorm_fwd_bwd():
    """Fused residual add + RMSNorm: both outputs and the joined gradient against plain PyTorch in fp32."""
    from himuon_b200 import ops

    torch.manual_seed(5)
    T, H = 300, 2560
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    d = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_(True)
    h, y = ops.add_rmsnorm(x, d, w, 1e-6)
    gh = torch.randn_like(h)
    gy = torch.randn_like(y)
    gx, gd, gw = torch.autograd.grad((h, y), (x, d, w), (gh, gy))
    xr, dr, wr = x.detach().float().requires_grad_(True), d.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    # value rounded to bf16 like the kernel's h, gradient of the plain sum
    hr = (xr + dr) + ((xr + dr).bfloat16().float() - (xr + dr)).detach()
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    rgx, rgd, rgw = torch.autograd.grad((hr, yr), (xr, dr, wr), (gh.float(), gy.float()), retain_graph=True)
    _close(h, hr.detach(), atol=1e-2, rtol=1e-2)
    _close(y, yr.detach(), atol=3e-2, rtol=2e-2)
    _close(gx, rgx, atol=5e-2, rtol=3e-2)
    assert gd.data_ptr() == gx.data_ptr()                    # one gradient tensor serves both inputs
    _close(gw, rgw, atol=0.5, rtol=3e-2)
    # only the normalised output used (final norm of the model)
    h2, y2 = ops.add_rmsnorm(x, d, w, 1e-6)
    gx2, = torch.autograd.grad(y2, x, gy)
    rgx2, = torch.autograd.grad(yr, xr, gy.float())
    _close(gx2, rgx2, atol=5e-2, rtol=3e-2)


@pytest.mark.parametrize("use_norm", [True, False])
def test_headnorm_rope(use_norm):
    e = _ext()
    torch.manual_seed(0)
    B, S, H, D = 2, 96, 4, 128
    x = torch.randn(B * S, H * D, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
    dy = torch.randn_like(x)
    cs = _rope_table(S).cuda()
    y = torch.empty_like(x)
    rstd = torch.empty(B * S * H, device="cuda")
    e.headnorm_rope_fwd(x, w if use_norm else None, y, rstd if use_norm else None, cs, H, S, 1e-6)
    xr = x.float().view(B, S, H, D).requires_grad_(True)
    wr = w.float().requires_grad_(True)
    xn = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr if use_norm else xr
    cos = torch.cat([cs[..., 0], cs[..., 0]], -1)[None, :, None, :]
    sin = torch.cat([cs[..., 1], cs[..., 1]], -1)[None, :, None, :]
    rot = torch.cat([-xn[..., D // 2:], xn[..., :D // 2]], -1)
    yr = xn * cos + rot * sin
    yr.backward(dy.float().view(B, S, H, D))
    _close(y, yr.reshape(B * S, H * D), atol=3e-2, rtol=2e-2)
    dx = torch.empty_like(x)
    dw = torch.zeros(D, device="cuda")
    e.headnorm_rope_bwd(dy, x if use_norm else None, w if use_norm else None, rstd if use_norm else None, dx,
                        dw if use_norm else None, cs, H, S)
    _close(dx, xr.grad.reshape(B * S, H * D), atol=3e-2, rtol=2e-2)
    if use_norm:
        _close(dw, wr.grad, atol=0.3, rtol=2e-2)


def test_swiglu_embedding_ce():
    e = _ext()
    torch.manual_seed(0)
    T, I = 300, 1024
    g = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    u = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(g)
    e.swiglu_fwd(g, u, out)
    gr, ur = g.float().requires_grad_(True), u.float().requires_grad_(True)
    ref = torch.nn.functional.silu(gr) * ur
    ref.backward(d.float())
    _close(out, ref, atol=2e-2, rtol=2e-2)
    dg, du = torch.empty_like(g), torch.empty_like(g)
    e.swiglu_bwd(d, g, u, dg, du)
    _close(dg, gr.grad, atol=3e-2, rtol=2e-2)
    _close(du, ur.grad, atol=3e-2, rtol=2e-2)

    V, H = 1000, 256
    table = torch.randn(V, H, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, V, (T,), device="cuda")
    emb = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    e.embedding_fwd(ids, table, emb)
    assert torch.equal(emb, table[ids])
    dt = torch.zeros(V, H, device="cuda", dtype=torch.float32)
    demb = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    e.embedding_bwd(ids, demb, dt)
    ref_dt = torch.zeros(V, H, device="cuda").index_add_(0, ids, demb.float())
    _close(dt, ref_dt, atol=1e-3, rtol=1e-3)

    vocab = 5000
    logits = (torch.randn(T, vocab, device="cuda") * 3).bfloat16()
    labels = torch.randint(0, vocab, (T,), device="cuda")
    labels[::7] = -100
    lr_ = logits.float().requires_grad_(True)
    loss_ref = torch.nn.functional.cross_entropy(lr_, labels, ignore_index=-100, reduction="sum")
    loss_ref.backward()
    loss = torch.zeros((), device="cuda")
    cnt = torch.zeros((), device="cuda")
    work = logits.clone()
    e.cross_entropy(work, labels, loss, cnt, None, 1.0, None, -100)
    assert cnt.item() == (labels != -100).sum().item()
    assert abs(loss.item() - loss_ref.item()) / loss_ref.item() < 2e-3
    _close(work, lr_.grad, atol=2e-3, rtol=2e-2)


def _attn_ref(q, k, v, scale):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    kk = k.repeat_interleave(Hq // Hkv, dim=2)
    vv = v.repeat_interleave(Hq // Hkv, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
    mask = torch.ones(S, S, device=q.device, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = s.softmax(-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, vv)


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 2, 1), (2, 384, 4, 2), (1, 200, 2, 2), (1, 1024, 8, 2)])
def test_flash_attention_fwd_bwd(B, S, Hq, Hkv):
    e = _ext()
    torch.manual_seed(0)
    D = 128
    scale = 1.0 / math.sqrt(D)
    q = torch.randn(B * S, Hq * D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B * S, Hkv * D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B * S, Hkv * D, device="cuda", dtype=torch.bfloat16)
    o = torch.empty_like(q)
    lse = torch.empty(B * Hq * S, device="cuda")
    e.flash_attn_fwd(q, k, v, o, lse, B, S, Hq, Hkv, scale)
    torch.cuda.synchronize()
    _assert_status_clean()
    qr = q.float().view(B, S, Hq, D).requires_grad_(True)
    kr = k.float().view(B, S, Hkv, D).requires_grad_(True)
    vr = v.float().view(B, S, Hkv, D).requires_grad_(True)
    ref = _attn_ref(qr, kr, vr, scale)
    _close(o, ref.reshape(B * S, Hq * D), atol=2e-2, rtol=2e-2)
    do = torch.randn_like(q)
    ref.backward(do.float().view(B, S, Hq, D))
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty(B * Hq * S, device="cuda")
    e.flash_attn_bwd(do, q, k, v, o, lse, dq, dk, dv, delta, torch.empty(2, B * S, Hq * 128, device='cuda', dtype=torch.bfloat16) if Hq > Hkv else None, B, S, Hq, Hkv, scale)
    torch.cuda.synchronize()
    _assert_status_clean()
    _close(dq, qr.grad.reshape(B * S, Hq * D), atol=3e-2, rtol=3e-2)
    _close(dk, kr.grad.reshape(B * S, Hkv * D), atol=3e-2, rtol=3e-2)
    _close(dv, vr.grad.reshape(B * S, Hkv * D), atol=3e-2, rtol=3e-2)
