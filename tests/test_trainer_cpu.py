"""Host-side behaviour of the Trainer: evaluation must not disturb training state, and a kernel status word that
reports an expired wait must stop training with an error."""

import argparse

import pytest
import torch

from himuon_b200.models import CausalLM, DecoderConfig
from himuon_b200.optim import get_optimizer
from himuon_b200.trainer import Trainer


def _cfg():
    return DecoderConfig(model_type="qwen3", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                         num_attention_heads=2, num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4,
                         tie_word_embeddings=True, max_position_embeddings=64)


def _batches(n, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, 64, (2, 16), generator=g)
        out.append({"input_ids": ids, "labels": ids})
    return out


def _trainer(zero_to_none):
    torch.manual_seed(0)
    model = CausalLM(_cfg())
    opt = get_optimizer("adamw", model, argparse.Namespace(lr=1e-2, weight_decay=0.0))
    tr = Trainer(model, opt, None, None, 2, torch.device("cpu"))
    tr.zero_set_to_none = zero_to_none
    return model, tr


@pytest.mark.parametrize("zero_to_none", [True, False])
def test_evaluate_between_steps_leaves_gradients_and_the_next_step_untouched(zero_to_none):
    train = _batches(4, seed=1)
    evalb = _batches(3, seed=2)
    model_a, tr_a = _trainer(zero_to_none)
    model_b, tr_b = _trainer(zero_to_none)
    tr_a.train_step(train[:2])
    tr_b.train_step(train[:2])
    grads_before = {n: (None if p.grad is None else p.grad.clone()) for n, p in model_a.named_parameters()}
    e1 = tr_a.evaluate(evalb)
    e2 = tr_a.evaluate(iter(evalb), steps=3)          # the iterator form draws the same three batches
    assert e1 == e2 and model_a.training
    for n, p in model_a.named_parameters():
        g = grads_before[n]
        assert (p.grad is None) == (g is None), n
        if g is not None:
            assert torch.equal(p.grad, g), n
    la = tr_a.read_loss(tr_a.train_step(train[2:]))
    lb = tr_b.read_loss(tr_b.train_step(train[2:]))
    assert la == lb
    for (n, a), (_, b) in zip(model_a.named_parameters(), model_b.named_parameters()):
        assert torch.equal(a, b), n


def test_loss_scale_is_only_forwarded_when_a_backward_pass_follows(monkeypatch):
    from himuon_b200 import ops
    seen = []
    real = ops.linear_cross_entropy

    def spy(*a, **k):
        seen.append(k.get("loss_scale"))
        return real(*a, **k)

    monkeypatch.setattr(ops, "linear_cross_entropy", spy)
    model, tr = _trainer(True)
    b = _batches(1, seed=3)[0]
    model.train()
    model(b["input_ids"], labels=b["labels"])
    with torch.no_grad():
        model(b["input_ids"], labels=b["labels"])
    model.eval()
    model(b["input_ids"], labels=b["labels"])
    assert seen == [0.5, None, None]


def test_an_expired_device_wait_stops_training(monkeypatch):
    model, tr = _trainer(True)
    loss = tr.train_step(_batches(2, seed=4))
    assert tr.device_status() == 0
    tr.read_loss(loss)
    monkeypatch.setattr(Trainer, "device_status", lambda self: 6)
    with pytest.raises(RuntimeError, match="status code 6"):
        tr.read_loss(loss)
