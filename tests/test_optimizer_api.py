"""Contract tests of the HiMuon public surface (CPU tier): signature, group schema, tile normalisation,
reconfigure, state_dict round trip, scheduler / zero_grad interplay - the counterpart of the reference's
tests/unit/test_optimizer_api.py."""

import inspect

import pytest
import torch

from himuon_b200.optimizers import HiMuon, HiMuonLegacy
from helpers import make_linear_model, seed_grads

EXPECTED_SIGNATURE = {
    "lr": 0.02, "momentum": 0.95, "nesterov": True, "weight_decay": 0.1, "tile_size": 512, "ns_steps": 5,
    "use_muon": True, "lr_adjust": "tile", "adamw_betas": (0.95, 0.95), "adamw_eps": 1e-8, "b_hw": None,
    "cuda_graph": True, "cuda_graph_warmup": 3,
}
GROUP_KEYS = {"lr", "momentum", "nesterov", "weight_decay", "tile_size", "ns_steps", "use_muon", "adamw_betas", "adamw_eps"}


def _opt(**kw):
    model = make_linear_model([(32, 48), (16, 16)])
    return model, HiMuon(model.parameters(), **kw)


def test_signature_is_locked():
    params = inspect.signature(HiMuon.__init__).parameters
    names = [n for n in params if n not in ("self", "params")]
    assert names == list(EXPECTED_SIGNATURE)
    for n, default in EXPECTED_SIGNATURE.items():
        assert params[n].default == default


def test_is_optimizer_with_group_schema():
    _, opt = _opt()
    assert isinstance(opt, torch.optim.Optimizer)
    for g in opt.param_groups:
        assert GROUP_KEYS <= set(g)
        for k in ("lr_adjust", "b_hw", "cuda_graph", "cuda_graph_warmup"):
            assert k not in g
    assert opt.lr_adjust == "tile"


@pytest.mark.parametrize("given,expected", [(128, (128, 128)), ((64, 256), (64, 256)), ([32, 16], (32, 16))])
def test_tile_size_normalisation(given, expected):
    _, opt = _opt(tile_size=given)
    assert opt.param_groups[0]["tile_size"] == expected


def test_bad_tile_and_lr_adjust_rejected():
    with pytest.raises(AssertionError):
        _opt(tile_size=(1, 2, 3))
    with pytest.raises(AssertionError):
        _opt(tile_size=0)
    with pytest.raises(ValueError):
        _opt(lr_adjust="banana")


def test_reconfigure_updates_all_groups_and_ignores_unknown():
    model = make_linear_model([(32, 48), (16, 16)])
    ps = list(model.parameters())
    opt = HiMuon([{"params": [ps[0]]}, {"params": [ps[1]], "use_muon": False, "lr": 1e-3}], tile_size=64)
    opt.reconfigure(tile_size=16, ns_steps=3, momentum=0.9, not_a_key=1, lr_adjust="none")
    for g in opt.param_groups:
        assert g["tile_size"] == (16, 16) and g["ns_steps"] == 3 and g["momentum"] == 0.9
        assert "not_a_key" not in g
    assert opt.lr_adjust == "tile"          # instance attribute, not a group key: silently ignored
    assert opt.param_groups[1]["lr"] == 1e-3


def test_reconfigure_invalidates_plan_and_buffers():
    model, opt = _opt(tile_size=16, cuda_graph=False)
    assert opt.xlayer_plan() == []
    seed_grads(model)
    opt.step()
    plan = opt.xlayer_plan()
    assert plan and plan[0]["bucket_key"][:3] == (16, 16, False)
    opt.reconfigure(tile_size=8)
    assert opt.xlayer_plan() == [] and opt._cached_plan is None and opt._cuda_graph is None
    assert opt._graph_step_count == 0 and opt._pending_updates == [] and opt._concat_buffers == {}
    opt.step()
    assert opt.xlayer_plan()[0]["bucket_key"][:2] == (8, 8)


def test_state_dict_round_trip():
    model, opt = _opt(tile_size=16, cuda_graph=False)
    seed_grads(model)
    opt.step()
    sd = opt.state_dict()
    model2 = make_linear_model([(32, 48), (16, 16)])
    opt2 = HiMuon(model2.parameters(), tile_size=16, cuda_graph=False)
    opt2.load_state_dict(sd)
    for (_, s1), (_, s2) in zip(opt.state.items(), opt2.state.items()):
        assert torch.equal(s1["momentum_buffer"], s2["momentum_buffer"])
    assert opt2.param_groups[0]["tile_size"] == (16, 16)


def test_works_with_scheduler_and_zero_grad_modes():
    from himuon_b200.trainer import cosine_with_warmup

    model, opt = _opt(tile_size=16, cuda_graph=False)
    sched = cosine_with_warmup(opt, 2, 10)
    for set_to_none in (True, False):
        seed_grads(model)
        before = [p.detach().clone() for p in model.parameters()]
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=set_to_none)
        for p, b in zip(model.parameters(), before):
            assert torch.isfinite(p).all()
            assert (p.grad is None) == set_to_none
    assert opt.param_groups[0]["lr"] > 0


def test_static_helpers_tile_untile_and_ns():
    t = torch.arange(35 * 50, dtype=torch.float32).view(35, 50)
    tiled, info = HiMuon._tile(t, (16, 32))
    assert tiled.shape == (3, 2, 16, 32) and info == (35, 50, 13, 14)
    assert torch.equal(HiMuon._untile(tiled, info), t)
    x = torch.randn(4, 16, 24)
    y = HiMuon.newton_schulz(x, 5)
    assert y.shape == x.shape and y.dtype == x.dtype and torch.isfinite(y).all()
    assert HiMuon.newton_schulz(torch.zeros(2, 8, 8), 5).abs().max() == 0


def test_legacy_variant_shares_surface():
    model = make_linear_model([(32, 48)])
    opt = HiMuonLegacy(model.parameters(), tile_size=16)
    assert GROUP_KEYS <= set(opt.param_groups[0])
    opt.reconfigure(tile_size=(8, 16))
    assert opt.param_groups[0]["tile_size"] == (8, 16)
    seed_grads(model)
    opt.step()
    assert all(torch.isfinite(p).all() for p in model.parameters())
