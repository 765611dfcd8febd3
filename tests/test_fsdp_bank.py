"""Parameter-bank contracts on a synthetic decoder (counterpart of the reference's tests/unit/test_fsdp_bank.py)."""

import pytest
import torch
import torch.nn.functional as F

from himuon_b200.fsdp_bank import (BankSpec, Llama3BankScheme, Qwen3BankScheme, release_pre_shard_refs,
                                   unbank_state_dict, wrap_with_banks)
from himuon_b200.models import CausalLM, DecoderConfig


def _model(layers=3, model_type="qwen3"):
    torch.manual_seed(0)
    cfg = DecoderConfig(model_type=model_type, vocab_size=64, hidden_size=32, intermediate_size=48,
                        num_hidden_layers=layers, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                        tie_word_embeddings=False, max_position_embeddings=64)
    return CausalLM(cfg)


@pytest.mark.parametrize("scheme_cls,mt", [(Qwen3BankScheme, "qwen3"), (Llama3BankScheme, "llama")])
def test_five_banks_shapes_and_padding(scheme_cls, mt):
    model = _model(3, mt)
    specs = scheme_cls().collect(model, world_size=4)
    assert [s.name for s in specs] == ["q_bank", "kv_bank", "o_bank", "gate_up_bank", "down_bank"]
    by = {s.name: s for s in specs}
    assert by["q_bank"].matrix_shape == (32, 32) and by["kv_bank"].matrix_shape == (16, 32)
    assert by["gate_up_bank"].matrix_shape == (48, 32) and by["down_bank"].matrix_shape == (32, 48)
    assert by["q_bank"].n_padded == 4 and by["q_bank"].n_logical == 3 and by["q_bank"].n_pad_rows == 1
    assert by["kv_bank"].n_padded == 8 and by["kv_bank"].n_logical == 6
    assert by["kv_bank"].source_param_names[:2] == ["model.layers.0.self_attn.k_proj.weight",
                                                    "model.layers.0.self_attn.v_proj.weight"]
    assert by["gate_up_bank"].source_param_names[2:4] == ["model.layers.1.mlp.gate_proj.weight",
                                                          "model.layers.1.mlp.up_proj.weight"]


def test_wrap_copies_slots_deletes_weights_and_keeps_forward():
    model = _model(3)
    ids = torch.randint(0, 64, (2, 16))
    ref_logits = model(ids).logits.detach().clone()
    originals = {n: p.detach().clone() for n, p in model.named_parameters()}
    model, banks = wrap_with_banks(model, Qwen3BankScheme(), world_size=2)
    names = dict(model.named_parameters())
    for bank_name in Qwen3BankScheme.BANK_NAMES:
        assert bank_name in names and names[bank_name].ndim == 3
    assert not any("q_proj.weight" in n or "down_proj.weight" in n for n in names)
    by = {b.spec.name: b for b in banks}
    for i in range(3):
        assert torch.equal(by["q_bank"].parameter[i], originals[f"model.layers.{i}.self_attn.q_proj.weight"])
        assert torch.equal(by["kv_bank"].parameter[2 * i + 1], originals[f"model.layers.{i}.self_attn.v_proj.weight"])
        assert torch.equal(by["gate_up_bank"].parameter[2 * i], originals[f"model.layers.{i}.mlp.gate_proj.weight"])
    assert by["q_bank"].parameter[3].abs().max() == 0          # pad slot
    assert model.model.layers[1].self_attn.k_proj._bank_idx == 2
    assert model.model.layers[1].self_attn.k_proj._bank_name == "kv_bank"
    assert torch.allclose(model(ids).logits, ref_logits, atol=1e-6)
    lin = model.model.layers[0].mlp.down_proj
    x = torch.randn(5, 48)
    assert torch.equal(lin(x), F.linear(x, by["down_bank"].parameter[0]))


def test_bank_gradient_flows_into_slots_only():
    model, banks = wrap_with_banks(_model(3), Qwen3BankScheme(), world_size=4)
    ids = torch.randint(0, 64, (2, 16))
    model(ids, labels=ids).loss.backward()
    g = model.q_bank.grad
    assert g is not None and g[:3].abs().sum() > 0 and g[3].abs().max() == 0


def test_unbank_state_dict_is_the_inverse():
    model = _model(2)
    original = {k: v.clone() for k, v in model.state_dict().items()}
    model, banks = wrap_with_banks(model, Qwen3BankScheme(), world_size=3)
    restored = unbank_state_dict(model.state_dict(), banks)
    assert set(restored) == set(original)
    for k in original:
        assert torch.equal(restored[k], original[k])
    broken = {k: v for k, v in model.state_dict().items() if k != "o_bank"}
    with pytest.raises(KeyError):
        unbank_state_dict(broken, banks)


def test_release_pre_shard_refs():
    model, banks = wrap_with_banks(_model(2), Qwen3BankScheme(), world_size=2)
    release_pre_shard_refs(banks)
    for b in banks:
        assert b.parameter is None and isinstance(b.spec, BankSpec) and b.name_to_idx
