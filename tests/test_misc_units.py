"""Dataset schema, model helpers, utils and logger format (counterparts of the reference's
tests/unit/test_dataset.py, test_model.py, test_utils.py)."""

import argparse
import time
import warnings

import pytest
import torch

from himuon_b200.dataset import SyntheticTokenDataset, ToyDataset
from himuon_b200.logger import format_metrics
from himuon_b200.model import count_model_parameters, count_num_training_tokens, get_model_and_tokenizer
from himuon_b200.models import MODEL_CONFIGS, get_config
from himuon_b200.utils import TimeBudget, merge_kv_args, parse_kv_args, seed_everything
from helpers import FakeTokenizer, TextStream


def test_toy_dataset_schema_and_padding():
    tok = FakeTokenizer()
    ds = ToyDataset(TextStream(["hello", "a much longer piece of text than the limit"]), tok, max_length=16)
    items = list(ds)
    assert tok.pad_token == tok.eos_token
    for it in items:
        assert set(it) == {"input_ids", "attention_mask", "labels"}
        assert it["input_ids"].shape == (16,) and torch.equal(it["labels"], it["input_ids"])
        assert it["labels"] is not it["input_ids"]
    assert items[0]["input_ids"][5:].eq(tok.eos_token_id).all()      # padded with eos, labels not masked
    assert items[0]["attention_mask"].sum() == 5


def test_toy_dataset_requires_eos():
    tok = FakeTokenizer()
    tok.eos_token_id = None
    with pytest.raises(ValueError):
        ToyDataset(TextStream([]), tok)


def test_synthetic_dataset_is_sharded_and_reproducible():
    a = list(SyntheticTokenDataset(100, 8, seed=3, rank=0, world_size=2, num_examples=3))
    b = list(SyntheticTokenDataset(100, 8, seed=3, rank=1, world_size=2, num_examples=3))
    a2 = list(SyntheticTokenDataset(100, 8, seed=3, rank=0, world_size=2, num_examples=3))
    assert all(torch.equal(x["input_ids"], y["input_ids"]) for x, y in zip(a, a2))
    assert not torch.equal(a[0]["input_ids"], b[0]["input_ids"])
    assert a[0]["input_ids"].max() < 100 and a[0]["input_ids"].dtype == torch.long


def test_param_count_helpers():
    class M(torch.nn.Module):
        def __init__(self, n):
            super().__init__()
            self.w = torch.nn.Parameter(torch.empty(n, device="meta"))

    assert count_model_parameters(M(10))[1] == "10 trainable parameters"
    assert count_model_parameters(M(2_500_000))[1] == "2.50M trainable parameters"
    n, s = count_model_parameters(M(3_000_000_000))
    assert s == "3.00B trainable parameters" and count_num_training_tokens(M(1000), 0.5) == 10000


def test_model_table_and_loader():
    assert get_config("qwen3-4b").hidden_size == 2560 and get_config("Qwen3-4B").num_hidden_layers == 36
    assert MODEL_CONFIGS["Llama-3.1-8B"].intermediate_size == 14336 and MODEL_CONFIGS["Llama-3.1-8B"].rope_theta == 500000.0
    with pytest.raises(ValueError):
        get_model_and_tokenizer("gpt-17")
    model, tok = get_model_and_tokenizer("tiny-qwen3")
    assert model.lm_head.weight is model.model.embed_tokens.weight and tok.eos_token_id is not None
    names = [n for n, _ in model.named_parameters()]
    assert "model.layers.0.self_attn.q_norm.weight" in names and "model.layers.1.mlp.down_proj.weight" in names


def test_kv_args_and_merge():
    assert parse_kv_args(["a=1", "b=(2, 3)", "c=foo", "d=0.5", "e=x=y"]) == {"a": 1, "b": (2, 3), "c": "foo", "d": 0.5, "e": "x=y"}
    ns = argparse.Namespace(lr=0.1, kwargs=["lr=0.2", "tile_size=64"], other=None)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        merge_kv_args(ns)
    assert ns.lr == 0.2 and ns.tile_size == 64 and len(w) == 1


def test_time_budget_and_seed():
    assert not TimeBudget(None).is_expired() and repr(TimeBudget(None)) == "inf"
    b = TimeBudget(1e-7)
    time.sleep(0.01)
    assert b.is_expired()
    seed_everything(7)
    x = torch.rand(3)
    seed_everything(7)
    assert torch.equal(x, torch.rand(3))


def test_metric_line_format():
    line = format_metrics({"step": 3, "lr": 0.0125, "loss": 2.34567, "tokens": 1234567, "eval_loss": 1.5})
    assert line == "Step: 3 LR: 0.012500 Training loss: 2.3457, Tokens: 1,234,567, Eval loss: 1.5000"


def test_symmetric_heap_guard_zones_catch_an_overrun():
    import torch

    from himuon_b200.parallel.symm import SymmetricHeap

    heap = SymmetricHeap(1 << 16, torch.device("cpu"), canaries=True)
    a, off_a = heap.alloc((100,), torch.float32)
    b, off_b = heap.alloc((64,), torch.bfloat16)
    assert off_b >= off_a + 400 + SymmetricHeap.CANARY_BYTES
    a.fill_(1.0)
    b.fill_(2.0)
    assert heap.check_canaries() == []
    # a write that runs past the end of the first region lands in its guard zone
    heap.view(0, off_a, (104,), torch.float32)[100:].fill_(3.0)
    assert heap.check_canaries() == [off_a + 400]
    plain = SymmetricHeap(1 << 12, torch.device("cpu"))
    plain.alloc((8,), torch.float32)
    assert plain.check_canaries() == []


def test_phase_timer_is_inert_without_cuda_and_ranges_nest():
    from himuon_b200.utils import PhaseTimer, nvtx_range

    t = PhaseTimer(enabled=True)            # no CUDA here: stays disabled, costs nothing
    with t.phase("forward_backward"):
        with nvtx_range("inner"):
            pass
    with t.phase("optimizer"):
        pass
    import torch
    if not torch.cuda.is_available():
        assert t.enabled is False and t.summary() == {}
    t.reset()
    assert t.summary() == {}
