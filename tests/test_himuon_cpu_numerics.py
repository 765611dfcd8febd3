"""HiMuon numerics on the PyTorch path (CPU): oracle agreement, chunk-size invariance, bank == per-matrix,
routing rules.  These are the checks the reference can only run on a GPU
(tests/integration/test_himuon_self_consistency.py, test_himuon_fsdp_parity.py, test_himuon_dispatch.py)."""

import math

import torch

from himuon_b200.ops import reference as ref
from himuon_b200.optimizers import HiMuon, Muon
from helpers import make_linear_model, seed_grads


def _polar(x):
    U, _, Vh = torch.linalg.svd(x.double(), full_matrices=False)
    return (U @ Vh).float()


def test_ns_reference_approaches_polar_factor():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 32, 48, generator=g)
    U, _, Vh = torch.linalg.svd(x, full_matrices=False)
    x = (U * torch.linspace(0.8, 1.2, 32)) @ Vh
    for dt, tol in ((torch.float64, 0.35), (torch.float32, 0.35), (torch.bfloat16, 0.4)):
        y = ref.newton_schulz(x, 5, compute_dtype=dt).float()
        rel = (y - _polar(x)).norm() / _polar(x).norm()
        assert rel < tol, (dt, rel)
    tall = ref.newton_schulz(x.transpose(1, 2).contiguous(), 5, compute_dtype=torch.float32)
    wide = ref.newton_schulz(x, 5, compute_dtype=torch.float32)
    assert torch.allclose(tall.transpose(1, 2), wide, atol=1e-5)


def test_step_matches_hand_written_oracle():
    torch.manual_seed(0)
    model = make_linear_model([(40, 70)])
    p = next(model.parameters())
    p0 = p.detach().clone()
    opt = HiMuon(model.parameters(), lr=0.02, momentum=0.95, weight_decay=0.1, tile_size=32, cuda_graph=False)
    seed_grads(model, 1)
    g = p.grad.clone()
    opt.step()
    buf = g.clone()                       # first step: momentum buffer == grad
    upd = g + 0.95 * buf
    tiles, info = ref.tile(upd, (32, 32))
    orth = ref.newton_schulz(tiles.view(-1, 32, 32), 5).view(tiles.shape)
    u = ref.untile(orth, info)
    expect = p0 * (1 - 0.02 * 0.1) - 0.02 * 0.2 * math.sqrt(32) * u
    assert torch.allclose(p, expect, atol=1e-6)


def test_result_is_invariant_to_chunk_size():
    outs = []
    for b_hw in (1, 3, 64):
        torch.manual_seed(0)
        model = make_linear_model([(48, 80), (33, 65), (16, 16)])
        opt = HiMuon(model.parameters(), tile_size=16, b_hw=b_hw, cuda_graph=False)
        for s in range(2):
            seed_grads(model, s)
            opt.step()
        plan = opt.xlayer_plan()
        assert sum(plan[0]["chunk_sizes"]) == plan[0]["B_total"] and max(plan[0]["chunk_sizes"]) <= b_hw
        outs.append([p.detach().clone() for p in model.parameters()])
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.allclose(a, b, atol=1e-6)


def test_routing_small_params_take_full_matrix_path():
    model = make_linear_model([(64, 64), (16, 16), (8, 200)])
    opt = HiMuon(model.parameters(), tile_size=32, cuda_graph=False)
    seed_grads(model)
    opt.step()
    plan = opt.xlayer_plan()
    assert len(plan) == 1 and plan[0]["bucket_key"][:3] == (32, 32, False)
    ids = {id(p): p for p in model.parameters()}
    shapes = sorted(tuple(ids[i].shape) for i in plan[0]["param_ids"])
    assert shapes == [(8, 200), (64, 64)]                      # (16,16) has numel <= 32*32: full-matrix NS
    assert plan[0]["tile_count_per_param"] == [4, 7] and plan[0]["B_total"] == 11 and plan[0]["n_calls"] == len(plan[0]["chunk_sizes"])
    assert set(plan[0]) >= {"bucket_key", "param_ids", "tile_count_per_param", "B_total", "B_hw", "chunk_sizes", "n_calls"}
    assert balanced(HiMuon._balanced_chunks(10, 4)) == [4, 3, 3] and HiMuon._balanced_chunks(0, 4) == []


def balanced(x):
    return x


def _bank_vs_per_matrix(H, W, tile):
    torch.manual_seed(0)
    N = 4
    bank = torch.nn.Parameter(torch.randn(N, H, W) * 0.02)
    mats = [torch.nn.Parameter(bank.detach()[i].clone()) for i in range(N)]
    ob = HiMuon([bank], tile_size=tile, cuda_graph=False, lr=0.02)
    om = HiMuon(mats, tile_size=tile, cuda_graph=False, lr=0.02)
    for s in range(3):
        g = torch.randn(N, H, W, generator=torch.Generator().manual_seed(s))
        bank.grad = g.clone()
        for i, m in enumerate(mats):
            m.grad = g[i].clone()
        ob.step()
        om.step()
    for i, m in enumerate(mats):
        assert torch.allclose(bank.detach()[i], m.detach(), atol=1e-6), (H, W, tile)


def test_bank_update_equals_per_matrix_update_divisible_and_padded():
    _bank_vs_per_matrix(64, 96, 32)          # tiles divide the matrix
    _bank_vs_per_matrix(50, 75, 32)          # zero-padded tiles
    _bank_vs_per_matrix(24, 40, 64)          # tile covers the whole matrix


def test_pad_slots_of_a_bank_are_skipped_and_stay_zero():
    bank = torch.nn.Parameter(torch.zeros(3, 16, 16))
    bank._hm_skip_slots = {2}
    bank.grad = torch.randn(3, 16, 16)
    opt = HiMuon([bank], tile_size=8, cuda_graph=False)
    opt.step()
    assert bank.detach()[2].abs().max() == 0 and bank.detach()[0].abs().max() > 0
    assert opt.xlayer_plan()[0]["B_total"] == 8


def test_muon_full_matrix_step_and_fallback():
    torch.manual_seed(0)
    model = make_linear_model([(24, 40)])
    bias = torch.nn.Parameter(torch.zeros(5))
    opt = Muon([{"params": list(model.parameters())}, {"params": [bias], "use_muon": False, "lr": 1e-3, "weight_decay": 0.0}], lr=0.01)
    p = next(model.parameters())
    p0 = p.detach().clone()
    seed_grads(model, 3)
    bias.grad = torch.ones(5)
    g = p.grad.clone()
    opt.step()
    u = ref.newton_schulz(g + 0.95 * g, 5)
    expect = p0 * (1 - 0.01 * 0.1) - 0.01 * 0.2 * math.sqrt(40) * u
    assert torch.allclose(p, expect, atol=1e-6)
    assert (bias < 0).all()


def test_dispatch_plan_accounts_for_every_tile_in_each_split_regime():
    """Counterpart of the reference's dispatch tests (tests/integration/test_himuon_dispatch.py): the bucket plan
    holds every tile of every parameter exactly once and cuts a bucket into balanced chunks below, at and above the
    per-call cap."""
    shapes = [(64, 96), (64, 96), (40, 70), (128, 32)]
    tile = 32
    expected = [math.ceil(h / tile) * math.ceil(w / tile) for h, w in shapes]      # 6, 6, 6, 4
    total = sum(expected)
    for b_hw in (total + 5, total, total - 1, 7, 1):
        model = make_linear_model(shapes)
        opt = HiMuon(model.parameters(), tile_size=tile, b_hw=b_hw, cuda_graph=False)
        seed_grads(model)
        opt.step()
        plan = opt.xlayer_plan()
        assert len(plan) == 1
        b = plan[0]
        by_id = {id(p): tuple(p.shape) for p in model.parameters()}
        counts = {by_id[i]: [] for i in b["param_ids"]}
        for i, c in zip(b["param_ids"], b["tile_count_per_param"]):
            counts[by_id[i]].append(c)
        assert sorted(c for v in counts.values() for c in v) == sorted(expected)
        assert b["B_total"] == total and b["B_hw"] == b_hw
        assert sum(b["chunk_sizes"]) == total and max(b["chunk_sizes"]) <= b_hw
        assert b["n_calls"] == len(b["chunk_sizes"]) == math.ceil(total / b_hw)
        assert max(b["chunk_sizes"]) - min(b["chunk_sizes"]) <= 1                   # balanced, no tiny last chunk
