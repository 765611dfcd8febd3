"""HiMuon on the GPU kernels: NS dispatcher against the PyTorch oracle, smoke over dtype x tile, chunk-size
invariance, eager == graph, reconfigure invalidation, flat memory after capture, GPU == CPU optimizer step.
Mirrors the reference's tests/integration/test_himuon_{smoke,self_consistency,reconfigure,memory,dispatch}.py."""

import pytest
import torch

from helpers import make_linear_model, seed_grads

pytestmark = pytest.mark.gpu


def _well_conditioned(B, m, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, m, n, generator=g)
    U, _, Vh = torch.linalg.svd(x, full_matrices=False)
    return (U * torch.linspace(0.8, 1.2, min(m, n))) @ Vh


@pytest.mark.parametrize("shape", [(3, 512, 512), (2, 256, 512), (2, 512, 256), (5, 128, 128), (2, 768, 513),
                                   (1, 1024, 1024), (4, 64, 64), (2, 16, 1024)])
def test_newton_schulz_dispatcher_matches_oracle(shape):
    from himuon_b200 import ops
    from himuon_b200.ops import ns as ns_ops
    from himuon_b200.ops import reference as ref

    x = _well_conditioned(*shape).cuda().bfloat16()
    out = ns_ops.newton_schulz(x, 5)
    torch.cuda.synchronize()
    ops.check_status()
    want = ref.newton_schulz(x.cpu(), 5).float()
    err = (out.float().cpu() - want).abs()
    assert out.shape == x.shape and out.dtype == x.dtype
    assert (err > 4e-2 + 4e-2 * want.abs()).float().mean() < 1e-3, err.max()
    x2d = x[0]
    assert torch.allclose(ns_ops.newton_schulz(x2d, 5).float(), out[0].float(), atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tile", [128, 256, (128, 256), 1000000])
def test_smoke_finite_and_changed(dtype, tile):
    from himuon_b200.optimizers import HiMuon

    model = make_linear_model([(512, 512), (768, 513 if dtype == torch.float32 else 520), (64, 64), (256, 1024)], dtype, "cuda")
    opt = HiMuon(model.parameters(), tile_size=tile, cuda_graph=False)
    before = [p.detach().clone() for p in model.parameters()]
    for s in range(2):
        seed_grads(model, s)
        opt.step()
    for p, b in zip(model.parameters(), before):
        assert torch.isfinite(p).all() and not torch.equal(p, b)


def test_device_tables_pass_the_host_side_bounds_check():
    """With the table checks on, HiMuon (tiled, padded and whole-matrix parameters plus an AdamW-fallback group) and the
    AdamW class build their device tables and step; the checks walk every entry against the live tensors."""
    from himuon_b200.optimizers import AdamW, HiMuon, _tablecheck

    _tablecheck.enable(True)
    try:
        model = make_linear_model([(512, 512), (768, 520), (64, 64), (256, 1024)], torch.bfloat16, "cuda")
        bias = torch.nn.Parameter(torch.zeros(96, device="cuda", dtype=torch.bfloat16))
        bias.grad = torch.ones_like(bias)
        opt = HiMuon([{"params": list(model.parameters())}, {"params": [bias], "use_muon": False, "lr": 1e-3}],
                     tile_size=(128, 256), cuda_graph=False)
        seed_grads(model, 0)
        opt.step()
        adam = AdamW(list(model.parameters()) + [bias], lr=1e-3)
        adam.step()
        torch.cuda.synchronize()
        assert all(torch.isfinite(p).all() for p in model.parameters())
    finally:
        _tablecheck.enable(False)


def _run(b_hw=None, cuda_graph=False, steps=5, dtype=torch.bfloat16):
    from himuon_b200.optimizers import HiMuon

    torch.manual_seed(0)
    model = make_linear_model([(512, 768), (300, 520), (128, 128)], dtype).to("cuda")   # CPU init: same weights as the CPU run
    bias = torch.nn.Parameter(torch.zeros(64, device="cuda", dtype=dtype))
    opt = HiMuon([{"params": list(model.parameters())}, {"params": [bias], "use_muon": False, "lr": 1e-3}],
                 tile_size=128, b_hw=b_hw, cuda_graph=cuda_graph, cuda_graph_warmup=2)
    seed_grads(model, 0)
    bias.grad = torch.zeros_like(bias)
    for s in range(steps):
        seed_grads(model, s)                      # in place: addresses stay stable for the graph
        bias.grad.copy_(torch.full_like(bias, 0.1 * (s + 1)))
        opt.step()
    torch.cuda.synchronize()
    return [p.detach().float().cpu() for p in list(model.parameters()) + [bias]], opt


def test_chunk_size_invariance_and_eager_equals_graph():
    base, _ = _run()
    chunked, opt_c = _run(b_hw=5)
    assert opt_c.xlayer_plan()[0]["n_calls"] > 1
    graph, opt_g = _run(cuda_graph=True)
    assert opt_g._cuda_graph is not None and opt_g._graph_step_count == 5
    for a, b, c in zip(base, chunked, graph):
        assert torch.allclose(a, b, atol=1e-2, rtol=1e-2)
        assert torch.allclose(a, c, atol=1e-2, rtol=1e-2)


def test_gpu_step_matches_cpu_step():
    from himuon_b200.optimizers import HiMuon

    gpu, _ = _run(steps=3, dtype=torch.float32)
    torch.manual_seed(0)
    model = make_linear_model([(512, 768), (300, 520), (128, 128)])
    bias = torch.nn.Parameter(torch.zeros(64))
    opt = HiMuon([{"params": list(model.parameters())}, {"params": [bias], "use_muon": False, "lr": 1e-3}],
                 tile_size=128, cuda_graph=False)
    for s in range(3):
        seed_grads(model, s)
        bias.grad = torch.full_like(bias, 0.1 * (s + 1))
        opt.step()
    for a, p in zip(gpu, list(model.parameters()) + [bias]):
        assert torch.allclose(a, p.detach(), atol=3e-3, rtol=1e-2), (a - p.detach()).abs().max()


def test_reconfigure_in_graph_mode_recaptures():
    from himuon_b200.optimizers import HiMuon

    model = make_linear_model([(512, 512), (256, 512)], torch.bfloat16, "cuda")
    opt = HiMuon(model.parameters(), tile_size=256, cuda_graph=True, cuda_graph_warmup=1)
    seed_grads(model, 0)
    for s in range(3):
        seed_grads(model, s)
        opt.step()
    assert opt._cuda_graph is not None
    opt.reconfigure(tile_size=128)
    assert opt._cuda_graph is None and opt._cached_plan is None and opt._graph_step_count == 0
    for s in range(3):
        seed_grads(model, s)
        opt.step()
    assert opt._cuda_graph is not None and opt.xlayer_plan()[0]["bucket_key"][:2] == (128, 128)
    assert all(torch.isfinite(p).all() for p in model.parameters())


def test_memory_is_flat_after_capture():
    from himuon_b200.optimizers import HiMuon

    model = make_linear_model([(1024, 1024)] * 4, torch.bfloat16, "cuda")
    opt = HiMuon(model.parameters(), tile_size=512, cuda_graph=True, cuda_graph_warmup=2)
    seed_grads(model, 0)
    for s in range(4):
        seed_grads(model, s)
        opt.step()
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    for s in range(10):
        seed_grads(model, s)
        opt.step()
    torch.cuda.synchronize()
    assert abs(torch.cuda.memory_allocated() - base) <= 0.01 * base


def test_lr_schedule_takes_effect_without_recapture():
    from himuon_b200.optimizers import HiMuon

    model = make_linear_model([(256, 256)], torch.float32, "cuda")
    opt = HiMuon(model.parameters(), tile_size=128, cuda_graph=True, cuda_graph_warmup=1, weight_decay=0.0)
    seed_grads(model, 0)
    for s in range(3):
        opt.step()
    graph = opt._cuda_graph
    p = next(model.parameters())
    for g in opt.param_groups:
        g["lr"] = 0.0
    before = p.detach().clone()
    opt.step()
    torch.cuda.synchronize()
    assert opt._cuda_graph is graph and torch.equal(p, before)      # lr 0 -> no change, same captured graph


@pytest.mark.parametrize("which", ["adamw", "muon", "himuon"])
def test_resume_from_state_dict_continues_bias_correction(which):
    """load_state_dict replaces the moment tensors: the device entry tables must be rebuilt over the new ones and the
    Adam step counter must continue from the saved value instead of restarting at zero."""
    from himuon_b200.optimizers import AdamW, HiMuon, Muon

    def make():
        torch.manual_seed(0)
        model = make_linear_model([(256, 384), (128, 128)], dtype=torch.bfloat16, device="cuda")
        bias = torch.nn.Parameter(torch.zeros(64, device="cuda", dtype=torch.bfloat16))
        if which == "adamw":
            opt = AdamW(list(model.parameters()) + [bias], lr=1e-2, weight_decay=0.01)
        else:
            cls = Muon if which == "muon" else HiMuon
            kw = {} if which == "muon" else {"tile_size": 128, "cuda_graph": False}
            opt = cls([{"params": list(model.parameters())}, {"params": [bias], "use_muon": False, "lr": 1e-2}], lr=1e-2, **kw)
        return model, bias, opt

    def grads(model, bias, s):
        seed_grads(model, s)
        bias.grad = torch.full_like(bias, 0.1 * (s + 1))

    m1, b1, o1 = make()
    for s in range(3):
        grads(m1, b1, s)
        o1.step()
    import copy
    saved = copy.deepcopy(o1.state_dict())        # state_dict() hands out the live tensors; the next step mutates them
    snap = [p.detach().clone() for p in list(m1.parameters()) + [b1]]
    grads(m1, b1, 3)
    o1.step()
    m2, b2, o2 = make()
    with torch.no_grad():
        for p, v in zip(list(m2.parameters()) + [b2], snap):
            p.copy_(v)
    grads(m2, b2, 0)
    o2.step()                      # builds tables over fresh state, which the load below must invalidate
    with torch.no_grad():
        for p, v in zip(list(m2.parameters()) + [b2], snap):
            p.copy_(v)
    o2.load_state_dict(saved)
    grads(m2, b2, 3)
    o2.step()
    torch.cuda.synchronize()
    for a, b in zip(list(m1.parameters()) + [b1], list(m2.parameters()) + [b2]):
        assert torch.allclose(a.float(), b.float(), atol=2e-3, rtol=1e-2), (a.float() - b.float()).abs().max()


def _cosine(a, b):
    a, b = a.float().flatten().cpu(), b.float().flatten().cpu()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


@pytest.mark.parametrize("which", ["muon", "himuon-legacy"])
def test_baseline_optimizers_step_on_the_kernels_like_their_cpu_paths(which):
    """Muon and HiMuonLegacy (Newton-Schulz on tcgen05) take several steps on bf16 CUDA parameters; the updates must
    follow the same optimizer stepping fp32 copies of the same parameters and gradients on the CPU."""
    from himuon_b200 import ops
    from himuon_b200.optimizers import HiMuonLegacy, Muon

    shapes = [(256, 384), (128, 128), (320, 136)]

    def build(device, dtype):
        torch.manual_seed(0)
        model = make_linear_model(shapes, dtype=torch.float32)
        with torch.no_grad():
            for p in model.parameters():
                p.copy_(p.bfloat16().float())
        model = model.to(device=device, dtype=dtype)
        if which == "muon":
            opt = Muon([{"params": list(model.parameters())}], lr=0.02, weight_decay=0.1)
        else:
            opt = HiMuonLegacy([{"params": list(model.parameters())}], lr=0.02, weight_decay=0.1, tile_size=128)
        return model, opt

    gpu_model, gpu_opt = build("cuda", torch.bfloat16)
    cpu_model, cpu_opt = build("cpu", torch.float32)
    start = [p.detach().float().cpu().clone() for p in gpu_model.parameters()]
    before = ops.launch_count()
    for s in range(6):
        g = torch.Generator().manual_seed(100 + s)
        for pg, pc in zip(gpu_model.parameters(), cpu_model.parameters()):
            val = torch.randn(pc.shape, generator=g).bfloat16()
            pg.grad = val.cuda()
            pc.grad = val.float()
        gpu_opt.step()
        cpu_opt.step()
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.launch_count() - before >= 6, "the kernel path did not run"
    for p0, pg, pc in zip(start, gpu_model.parameters(), cpu_model.parameters()):
        dg, dc = pg.detach().float().cpu() - p0, pc.detach() - p0
        assert torch.isfinite(dg).all()
        c = _cosine(dg, dc)
        assert c > 0.97, (which, tuple(pc.shape), c)
        assert abs(float(dg.norm() / dc.norm()) - 1.0) < 0.1, (which, float(dg.norm()), float(dc.norm()))


def test_soap_kernels_match_fp32_torch():
    """`soap_moments` and `soap_ratio` against the same arithmetic in fp32 PyTorch."""
    from himuon_b200._ext import ext

    torch.manual_seed(0)
    n = 384 * 520
    g, gr, m, v = (torch.randn(n, device="cuda").bfloat16() for _ in range(4))
    v = v.abs()
    m0, v0 = m.clone(), v.clone()
    ext().soap_moments(g, gr, m, v, 0.95, 0.9)
    want_m = 0.95 * m0.float() + 0.05 * g.float()
    want_v = 0.9 * v0.float() + 0.1 * gr.float() ** 2
    assert torch.allclose(m.float(), want_m, atol=1e-2, rtol=1e-2) and torch.allclose(v.float(), want_v, atol=1e-2, rtol=1e-2)
    out = torch.empty_like(m)
    ext().soap_ratio(m, v, out, 1e-8)
    want = m.float() / (v.float().sqrt() + 1e-8)
    assert torch.allclose(out.float(), want, atol=1e-2, rtol=1e-2)
    ext().soap_ratio(m, v, m, 1e-8)                    # in place over its first input
    assert torch.equal(m, out)


def test_soap_kernel_path_follows_the_torch_path():
    """One SOAP step through the GEMM and the soap_* kernels against the same step through the optimizer's PyTorch
    ops, from identical state (bases, Gram statistics, moments) and with the same gradient, for three consecutive
    steps, one of which refreshes the eigenbases.  Longer independent runs are no oracle for this optimizer: the Adam
    ratio in the eigenbasis blows rounding differences up wherever the gradient has little signal, and the
    eigenbases of near-degenerate Gram matrices are ill-conditioned, so two correct implementations drift apart."""
    import copy

    from himuon_b200 import ops
    from himuon_b200.optimizers import SOAP

    shapes = [(256, 384), (128, 128), (320, 136)]
    kw = dict(lr=3e-3, precondition_frequency=3, weight_decay=0.01)
    torch.manual_seed(0)
    model = make_linear_model(shapes, dtype=torch.bfloat16, device="cuda")
    opt = SOAP(model.parameters(), **kw)
    opt._kernel_ok = lambda *a, **k: False                      # PyTorch ops only
    g = torch.Generator().manual_seed(11)
    for _ in range(5):
        for p in model.parameters():
            p.grad = torch.randn(p.shape, generator=g).bfloat16().cuda()
        opt.step()
    for nxt in range(3):
        twin = copy.deepcopy(model)
        opt_k = SOAP(twin.parameters(), **kw)
        for p, q in zip(model.parameters(), twin.parameters()):  # same state, dtype for dtype (no load_state_dict cast)
            opt_k.state[q] = copy.deepcopy(opt.state[p])
        grads = [torch.randn(p.shape, generator=g).bfloat16().cuda() for p in model.parameters()]
        before = [p.detach().float().clone() for p in model.parameters()]
        for p, q, gr in zip(model.parameters(), twin.parameters(), grads):
            p.grad, q.grad = gr.clone(), gr.clone()
        n0 = ops.launch_count()
        opt_k.step()
        assert ops.launch_count() - n0 >= 10 * len(shapes), "the kernel path did not run"
        opt.step()
        torch.cuda.synchronize()
        for p, q, b in zip(model.parameters(), twin.parameters(), before):
            d_ref, d_ker = p.detach().float() - b, q.detach().float() - b
            assert torch.isfinite(d_ker).all()
            c = _cosine(d_ker, d_ref)
            assert c > 0.995, (nxt, tuple(p.shape), c)
            assert abs(float(d_ker.norm() / d_ref.norm()) - 1.0) < 0.02, (nxt, tuple(p.shape))
            gg_r, gg_k = opt.state[p]["GG"], opt_k.state[q]["GG"]
            for a, bb in zip(gg_r, gg_k):                        # Gram EMA in the GEMM epilogue vs lerp_
                assert float((a - bb).norm() / a.norm()) < 1e-3
    ops.check_status()
