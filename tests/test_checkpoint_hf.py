"""Checkpoint format: what `save_pretrained` writes must load into Hugging Face `transformers` models and give the
same logits, for plain and for bank-sharded (un-banked at save time) models - the reference saves through HF's own
`save_pretrained` (train.py:166-170, train_fsdp.py:285-297)."""

import json
import os

import pytest
import torch

from himuon_b200.fsdp_bank import Qwen3BankScheme, unbank_state_dict, wrap_with_banks
from himuon_b200.models import CausalLM, DecoderConfig

transformers = pytest.importorskip("transformers")


def _cfg(model_type, tie):
    return DecoderConfig(model_type=model_type, vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=8, rms_norm_eps=1e-6, rope_theta=10000.0,
                         tie_word_embeddings=tie, max_position_embeddings=64)


@pytest.mark.parametrize("model_type,tie", [("qwen3", True), ("llama", False)])
def test_hf_transformers_loads_our_checkpoint(tmp_path, model_type, tie):
    torch.manual_seed(0)
    model = CausalLM(_cfg(model_type, tie)).eval()
    out_dir = str(tmp_path / "ckpt")
    model.save_pretrained(out_dir)
    with open(os.path.join(out_dir, "config.json")) as f:
        cfg = json.load(f)
    assert cfg["model_type"] == model_type and cfg["architectures"][0].endswith("ForCausalLM")
    hf = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32).eval()
    ids = torch.randint(0, 96, (2, 16))
    with torch.no_grad():
        ours = model(ids).logits
        theirs = hf(input_ids=ids).logits
    assert torch.allclose(ours, theirs, atol=2e-4, rtol=1e-3), (ours - theirs).abs().max()
    back = CausalLM.from_pretrained(out_dir)
    with torch.no_grad():
        assert torch.allclose(back(ids).logits, ours, atol=1e-6)


def test_banked_model_saves_unbanked_hf_keys(tmp_path):
    torch.manual_seed(0)
    model = CausalLM(_cfg("qwen3", True)).eval()
    ids = torch.randint(0, 96, (2, 16))
    with torch.no_grad():
        want = model(ids).logits
    expected_keys = set(model.state_dict())
    model, banks = wrap_with_banks(model, Qwen3BankScheme(), world_size=4)
    state = unbank_state_dict(model.state_dict(), banks)
    assert set(state) == expected_keys and any(k.startswith("model.layers.1.mlp.down_proj") for k in state)
    out_dir = str(tmp_path / "ckpt")
    model.save_pretrained(out_dir, state_dict=state)
    hf = transformers.AutoModelForCausalLM.from_pretrained(out_dir, torch_dtype=torch.float32).eval()
    with torch.no_grad():
        assert torch.allclose(hf(input_ids=ids).logits, want, atol=2e-4, rtol=1e-3)
