"""Host-side logic of the fused ops' autograd wrappers, run on the PyTorch fallback path (CPU tier):
the copy-free column split, the residual-add + RMSNorm pair, the deferred norm-weight gradient arena and the
Trainer's micro-batch graph switch (which must fall back to eager execution where no CUDA graph can be used)."""

import argparse

import torch

from himuon_b200 import ops
from himuon_b200.ops import reference as ref


def test_split_cols_backward_returns_the_shared_buffer_when_gradients_are_adjacent():
    x = torch.randn(6, 10, requires_grad=True)
    a, b = ops.split_cols(x, 4)
    assert a.shape == (6, 4) and b.shape == (6, 6)
    # gradients that are the two adjacent column blocks of one wider buffer (what attention's backward hands out)
    buf = torch.randn(6, 16)
    ga, gb = buf[:, 3:7], buf[:, 7:13]
    gx, = torch.autograd.grad((a, b), x, (ga, gb))
    assert gx.untyped_storage().data_ptr() == buf.untyped_storage().data_ptr()     # a view, no copy
    assert torch.equal(gx, buf[:, 3:13])


def test_split_cols_backward_copies_unrelated_gradients_and_handles_a_missing_one():
    x = torch.randn(5, 8, requires_grad=True)
    a, b = ops.split_cols(x, 3)
    ga, gb = torch.randn(5, 3), torch.randn(5, 5)
    gx, = torch.autograd.grad((a, b), x, (ga, gb), retain_graph=True)
    assert torch.equal(gx, torch.cat([ga, gb], dim=1))
    gx2, = torch.autograd.grad(b.sum(), x)                 # only the second half is used
    assert torch.equal(gx2[:, :3], torch.zeros(5, 3)) and torch.equal(gx2[:, 3:], torch.ones(5, 5))


def test_add_rmsnorm_fallback_matches_separate_ops():
    torch.manual_seed(0)
    x = torch.randn(7, 16, requires_grad=True)
    d = torch.randn(7, 16, requires_grad=True)
    w = torch.rand(16, requires_grad=True)
    h, y = ops.add_rmsnorm(x, d, w, 1e-6, defer_dw=True)    # defer_dw is a no-op on the fallback path
    (h.sum() + (y * y).sum()).backward()
    x2, d2, w2 = x.detach().clone().requires_grad_(True), d.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    h2 = x2 + d2
    y2 = ref.rmsnorm(h2, w2, 1e-6)
    (h2.sum() + (y2 * y2).sum()).backward()
    assert torch.allclose(h, h2) and torch.allclose(y, y2)
    for a, b in ((x.grad, x2.grad), (d.grad, d2.grad), (w.grad, w2.grad)):
        assert torch.allclose(a, b, atol=1e-6)
    h3, y3 = ops.add_rmsnorm(x.detach(), None, w.detach(), 1e-6)   # no pending delta: plain norm, stream unchanged
    assert h3.data_ptr() == x.data_ptr() and torch.allclose(y3, ref.rmsnorm(x.detach(), w.detach(), 1e-6))


class _ScaleWithDeferredGrad(torch.autograd.Function):
    """y = x * w whose weight gradient goes through the deferred arena, like the norm kernels do on CUDA."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return x * w

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        ops._norm_grad_buffer(w).add_((gy * x).sum(0).float())
        return gy * w, None


def test_norm_grad_arena_flushes_once_per_backward_and_accumulates_over_micro_batches():
    torch.manual_seed(1)
    w1 = torch.nn.Parameter(torch.rand(12).bfloat16())
    w2 = torch.nn.Parameter(torch.rand(5).bfloat16())
    xs = [torch.randn(3, 12).bfloat16() for _ in range(2)]
    expect1 = torch.zeros(12)
    expect2 = torch.zeros(5)
    for x in xs:                                             # two accumulation micro-steps
        y = _ScaleWithDeferredGrad.apply(_ScaleWithDeferredGrad.apply(x, w1), w1)     # the same weight used twice
        z = _ScaleWithDeferredGrad.apply(x[:, :5], w2)
        (y.float().sum() + z.float().sum()).backward()
        xf, wf = x.float(), w1.detach().float()
        expect1 += (2 * xf * wf).sum(0)                      # d/dw of x*w*w
        expect2 += x[:, :5].float().sum(0)
    assert w1.grad is not None and w1.grad.dtype == torch.bfloat16
    assert torch.allclose(w1.grad.float(), expect1, rtol=3e-2, atol=3e-2)
    assert torch.allclose(w2.grad.float(), expect2, rtol=3e-2, atol=3e-2)
    arena = ops._NORM_ARENAS[w1.device]
    assert not arena.pending and not arena.queued
    for chunk in arena.chunks:                               # accumulators are cleared after every flush
        assert float(chunk.abs().max()) == 0.0


def test_trainer_graph_switch_falls_back_to_eager_on_cpu():
    from himuon_b200.models import CausalLM, DecoderConfig
    from himuon_b200.optim import get_optimizer
    from himuon_b200.trainer import Trainer

    torch.manual_seed(0)
    cfg = DecoderConfig(model_type="qwen3", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                        num_attention_heads=2, num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4,
                        tie_word_embeddings=False, max_position_embeddings=64)
    model = CausalLM(cfg)
    opt = get_optimizer("adamw", model, argparse.Namespace(lr=1e-2, weight_decay=0.0))
    tr = Trainer(model, opt, None, None, 2, torch.device("cpu"), graph_microbatch=True, graph_warmup_steps=0)
    assert tr.graph_microbatch is False                     # CUDA graphs need a CUDA device
    ids = torch.randint(0, 64, (2, 16))
    losses = [tr.read_loss(tr.train_step([{"input_ids": ids, "labels": ids}] * 2)) for _ in range(5)]
    assert losses[-1] < losses[0]
    assert tr._mb_graphs == {} and tr.d2h_bytes == 5 * 4


def test_gradient_checkpointing_matches_plain_backward_on_the_fallback_path():
    from himuon_b200.models import CausalLM, DecoderConfig

    torch.manual_seed(0)
    cfg = DecoderConfig(model_type="qwen3", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                        num_attention_heads=2, num_key_value_heads=1, head_dim=16, rms_norm_eps=1e-6, rope_theta=1e4,
                        tie_word_embeddings=True, max_position_embeddings=64)
    plain = CausalLM(cfg)
    import copy
    ckpt = copy.deepcopy(plain)
    ckpt.gradient_checkpointing_enable()
    ids = torch.randint(0, 64, (2, 16))
    losses = []
    for m in (plain, ckpt):
        m.train()
        loss = m(ids, labels=ids).loss
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) < 1e-6
    for (n, a), (_, b) in zip(plain.named_parameters(), ckpt.named_parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-6), n
