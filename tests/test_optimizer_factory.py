"""Factory grouping rules (counterpart of the reference's tests/unit/test_optimizer_factory.py)."""

import argparse

import pytest
import torch

from himuon_b200.optim import get_optimizer, get_optimizer_kwargs
from himuon_b200.optimizers import SOAP, AdamW, HiMuon, HiMuonLegacy, Muon, MuonFsdp
from helpers import TinyCausalLM


@pytest.mark.parametrize("name,cls", [("himuon", HiMuon), ("HiMuon", HiMuon), ("muon", Muon), ("muon-fsdp", MuonFsdp),
                                      ("himuon-legacy", HiMuonLegacy)])
def test_muon_family_three_groups(name, cls):
    model = TinyCausalLM()
    opt = get_optimizer(name, model, argparse.Namespace(lr=0.02, weight_decay=0.05, unrelated=3))
    assert isinstance(opt, cls)
    g_muon, g_1d, g_head = opt.param_groups
    assert g_muon["use_muon"] is True and g_muon["weight_decay"] == 0.05 and g_muon["lr"] == 0.02
    assert [tuple(p.shape) for p in g_muon["params"]] == [(16, 16)]          # only mlp.weight
    assert g_1d["use_muon"] is False and g_1d["lr"] == 1e-3 and g_1d["weight_decay"] == 0.0
    assert all(p.ndim < 2 for p in g_1d["params"]) and len(g_1d["params"]) == 3
    assert g_head["use_muon"] is False and g_head["lr"] == 1e-3 and g_head["weight_decay"] == 0.05
    assert {tuple(p.shape) for p in g_head["params"]} == {(32, 16)}
    n_grouped = sum(len(g["params"]) for g in opt.param_groups)
    assert n_grouped == len(list(model.parameters()))


@pytest.mark.parametrize("name,cls", [("adamw", AdamW), ("soap", SOAP)])
def test_decay_split_two_groups(name, cls):
    model = TinyCausalLM()
    opt = get_optimizer(name, model, argparse.Namespace(lr=1e-3, weight_decay=None))
    assert isinstance(opt, cls)
    decay, no_decay = opt.param_groups
    assert decay["weight_decay"] == 0.1 and no_decay["weight_decay"] == 0.0
    assert all(p.dim() >= 2 for p in decay["params"]) and all(p.dim() < 2 for p in no_decay["params"])


def test_kwargs_filtered_by_signature_and_none_dropped():
    ns = argparse.Namespace(lr=0.5, tile_size=256, weight_decay=None, batch_size=7, ns_steps=3)
    kw = get_optimizer_kwargs(HiMuon, ns)
    assert kw == {"lr": 0.5, "tile_size": 256, "ns_steps": 3}
    assert get_optimizer_kwargs(HiMuon, None) == {}
    assert get_optimizer_kwargs(HiMuon, {"lr": 1.0, "zzz": 2}) == {"lr": 1.0}


def test_unknown_optimizer_raises():
    with pytest.raises(ValueError):
        get_optimizer("sgd-with-feelings", TinyCausalLM(), None)


def test_bank_parameters_land_in_the_muon_group():
    model = TinyCausalLM()
    model.q_bank = torch.nn.Parameter(torch.zeros(4, 8, 8))
    opt = get_optimizer("himuon", model, None)
    assert any(p.ndim == 3 for p in opt.param_groups[0]["params"])
