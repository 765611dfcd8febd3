"""End-to-end checks of the decoder on the sm_100a kernels against the PyTorch reference ops."""

import argparse
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _small_cfg(model_type):
    from himuon_b200.models import DecoderConfig

    return DecoderConfig(model_type=model_type, vocab_size=2048, hidden_size=256, intermediate_size=512,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                         rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=(model_type == "qwen3"),
                         max_position_embeddings=512)


def _cos(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return torch.dot(a, b) / (a.norm() * b.norm() + 1e-12)


@pytest.mark.parametrize("model_type", ["qwen3", "llama"])
def test_model_loss_and_grads_match_reference(model_type):
    from himuon_b200 import ops
    from himuon_b200.models import CausalLM

    torch.manual_seed(0)
    ref_model = CausalLM(_small_cfg(model_type)).cuda().float()
    ker_model = copy.deepcopy(ref_model).bfloat16()
    # the fp32 copy uses the bf16-rounded weights so both see the same parameters
    with torch.no_grad():
        for pr, pk in zip(ref_model.parameters(), ker_model.parameters()):
            pr.copy_(pk.float())
    ids = torch.randint(0, 2048, (2, 256), device="cuda")
    before = ops.launch_count()
    out_k = ker_model(ids, labels=ids)
    out_k.loss.backward()
    assert ops.launch_count() - before > 30, "the kernel path did not run"
    out_r = ref_model(ids, labels=ids)
    out_r.loss.backward()
    torch.cuda.synchronize()
    ops.check_status()
    assert abs(out_k.loss.item() - out_r.loss.item()) < 3e-2, (out_k.loss.item(), out_r.loss.item())
    names = [n for n, _ in ref_model.named_parameters()]
    worst = []
    for n, pr, pk in zip(names, ref_model.parameters(), ker_model.parameters()):
        assert pk.grad is not None, n
        c = _cos(pr.grad, pk.grad).item()
        rel = abs(pk.grad.float().norm().item() / (pr.grad.norm().item() + 1e-12) - 1.0)
        worst.append((c, rel, n))
        # direction and size of every parameter's gradient: a bf16 forward/backward against the fp32 model
        assert c > 0.99, f"gradient of {n} diverges from the reference (cosine {c:.4f})"
        assert rel < 0.05, f"gradient norm of {n} is off by {rel:.3%}"
    print("lowest cosine", min(worst)[:3:2], "largest norm error", max(worst, key=lambda t: t[1])[1:])


def test_train_steps_himuon_graph_matches_eager():
    from himuon_b200.models import CausalLM
    from himuon_b200.optim import get_optimizer

    def run(cuda_graph):
        torch.manual_seed(0)
        model = CausalLM(_small_cfg("qwen3")).cuda().bfloat16()
        ns = argparse.Namespace(lr=1e-2, weight_decay=0.1, tile_size=128, cuda_graph=cuda_graph, cuda_graph_warmup=2)
        opt = get_optimizer("himuon", model, ns)
        g = torch.Generator(device="cuda").manual_seed(1)
        ids = torch.randint(0, 2048, (2, 128), device="cuda", generator=g)   # one fixed batch: the loss must fall
        losses = []
        for _ in range(6):
            loss = model(ids, labels=ids).loss
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=False)
            losses.append(loss.item())
        return losses, opt

    eager, _ = run(False)
    graph, opt = run(True)
    assert opt._cuda_graph is not None
    assert eager[-1] < eager[0]
    for a, b in zip(eager, graph):
        assert abs(a - b) < 5e-2, (eager, graph)


def test_trainer_microbatch_graph_matches_eager():
    """Forward+backward replayed from the two captured micro-batch graphs (first / accumulating) gives the same
    losses and the same parameters as the eager path, with the bank engine and the graph-captured optimizer."""
    from himuon_b200 import ops
    from himuon_b200.models import CausalLM
    from himuon_b200.optim import get_optimizer
    from himuon_b200.parallel.fsdp import ShardedEngine
    from himuon_b200.trainer import Trainer

    def run(graph_microbatch):
        torch.manual_seed(0)
        model = CausalLM(_small_cfg("qwen3")).cuda().bfloat16()
        engine = ShardedEngine(model, use_banks=True)
        ns = argparse.Namespace(lr=1e-2, weight_decay=0.1, tile_size=128, cuda_graph=True, cuda_graph_warmup=1)
        opt = get_optimizer("himuon", model, ns)
        engine.attach_optimizer(opt)
        tr = Trainer(model, opt, None, engine, 3, torch.device("cuda"), graph_microbatch=graph_microbatch,
                     graph_warmup_steps=2)
        tr.zero_set_to_none = False
        g = torch.Generator().manual_seed(1)
        losses, launches = [], []
        for _ in range(6):
            step = []
            for _ in range(3):
                ids = torch.randint(0, 2048, (2, 128), generator=g).pin_memory()
                step.append({"input_ids": ids, "labels": ids})
            n0 = ops.launch_count()
            losses.append(tr.read_loss(tr.train_step(step)))
            launches.append(ops.launch_count() - n0)
        params = {n: p.detach().float().clone() for n, p in model.named_parameters()}
        engine.close()
        return losses, params, launches, tr

    eager, p_eager, l_eager, _ = run(False)
    graph, p_graph, l_graph, tr = run(True)
    assert {k[0] for k in tr._mb_graphs} == {True, False}
    assert l_graph[-1] == l_eager[-1], (l_eager, l_graph)       # replays are counted like eager launches
    for a, b in zip(eager, graph):
        assert abs(a - b) < 5e-2, (eager, graph)
    for n in p_eager:
        c = _cos(p_eager[n], p_graph[n]).item()
        assert c > 0.999, (n, c)
    ops.check_status()


def test_gradient_checkpointing_gives_the_same_gradients_on_the_kernel_path():
    """Per-layer activation checkpointing (the CLI default of train_ddp.py / train_fsdp.py) recomputes each layer in
    backward: loss and every gradient, including the deferred norm-weight gradients, must match the plain run."""
    from himuon_b200.models import CausalLM

    torch.manual_seed(0)
    plain = CausalLM(_small_cfg("qwen3")).cuda().bfloat16()
    ckpt = copy.deepcopy(plain)
    ckpt.gradient_checkpointing_enable()
    ids = torch.randint(0, 2048, (2, 256), device="cuda")
    for m in (plain, ckpt):
        m.train()
        for _ in range(2):                                   # two accumulation micro-steps
            m(ids, labels=ids).loss.backward()
    torch.cuda.synchronize()
    for (n, a), (_, b) in zip(plain.named_parameters(), ckpt.named_parameters()):
        assert a.grad is not None and b.grad is not None, n
        c = _cos(a.grad, b.grad).item()
        assert c > 0.9999, (n, c)


def test_evaluate_between_train_steps_does_not_touch_gradients_on_the_kernel_path():
    """`Trainer.evaluate` runs the fused lm_head + cross-entropy under no_grad: no gradient buffer (they persist,
    zeroed in place, with the graph-captured optimizer) and no gradient sink may change, and the training step that
    follows must match a run without the evaluation."""
    from himuon_b200 import ops
    from himuon_b200.models import CausalLM
    from himuon_b200.optim import get_optimizer
    from himuon_b200.parallel.fsdp import ShardedEngine
    from himuon_b200.trainer import Trainer

    def batches(n, seed):
        g = torch.Generator().manual_seed(seed)
        out = []
        for _ in range(n):
            ids = torch.randint(0, 2048, (2, 128), generator=g).pin_memory()
            out.append({"input_ids": ids, "labels": ids})
        return out

    def run(with_eval):
        torch.manual_seed(0)
        model = CausalLM(_small_cfg("qwen3")).cuda().bfloat16()
        engine = ShardedEngine(model, use_banks=True)
        ns = argparse.Namespace(lr=1e-2, weight_decay=0.1, tile_size=128, cuda_graph=True, cuda_graph_warmup=1)
        opt = get_optimizer("himuon", model, ns)
        engine.attach_optimizer(opt)
        tr = Trainer(model, opt, None, engine, 2, torch.device("cuda"))
        tr.zero_set_to_none = False
        train = batches(6, 1)
        tr.train_step(train[0:2])
        tr.train_step(train[2:4])
        if with_eval:
            snap = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
            sinks = {k: st.grad_full.clone() for k, st in engine.state.items()}
            fresh = {k: [s.fresh for s in st.sinks] for k, st in engine.state.items()}
            ev = tr.evaluate(batches(3, 2))
            assert ev == ev and model.training
            for n, p in model.named_parameters():
                if n in snap:
                    assert torch.equal(p.grad, snap[n]), n
            for k, st in engine.state.items():
                assert torch.equal(st.grad_full, sinks[k]), k
                assert [s.fresh for s in st.sinks] == fresh[k], k
        loss = tr.read_loss(tr.train_step(train[4:6]))
        params = {n: p.detach().float().clone() for n, p in model.named_parameters()}
        engine.close()
        return loss, params

    l0, p0 = run(False)
    l1, p1 = run(True)
    assert abs(l0 - l1) < 1e-3, (l0, l1)
    for n in p0:
        c = _cos(p0[n], p1[n]).item()
        assert c > 0.9999, (n, c)          # norm-weight gradients are summed with atomics: runs differ in the last bits
    ops.check_status()


@pytest.mark.parametrize("opt_name", ["himuon", "adamw"])
def test_cpu_offload_keeps_optimizer_state_on_the_host_between_steps(opt_name):
    """--cpu-offload: momentum and Adam moments sit in pinned host memory while forward/backward run, come back for
    the optimizer step, and training matches the run without offloading."""
    from himuon_b200.models import CausalLM
    from himuon_b200.optim import get_optimizer
    from himuon_b200.parallel.fsdp import ShardedEngine
    from himuon_b200.trainer import Trainer

    def run(offload):
        torch.manual_seed(0)
        model = CausalLM(_small_cfg("qwen3")).cuda().bfloat16()
        engine = ShardedEngine(model, use_banks=True, cpu_offload=offload)
        ns = argparse.Namespace(lr=1e-2 if opt_name == "himuon" else 1e-3, weight_decay=0.1, tile_size=128,
                                cuda_graph=False)
        opt = get_optimizer(opt_name, model, ns)
        engine.attach_optimizer(opt)
        tr = Trainer(model, opt, None, engine, 2, torch.device("cuda"))
        g = torch.Generator().manual_seed(1)
        losses = []
        for _ in range(4):
            step = []
            for _ in range(2):
                ids = torch.randint(0, 2048, (2, 128), generator=g).pin_memory()
                step.append({"input_ids": ids, "labels": ids})
            losses.append(tr.read_loss(tr.train_step(step)))
            if offload:
                big = [v for st in opt.state.values() for v in st.values() if torch.is_tensor(v) and v.numel() > 1]
                assert big and all(v.device.type == "cpu" and v.is_pinned() for v in big)
                assert engine._offload.bytes_offloaded > 0
        params = {n: p.detach().float().clone() for n, p in model.named_parameters()}
        engine.close()
        if offload:       # close() brings the state back so it can be saved
            assert all(v.is_cuda for st in opt.state.values() for v in st.values() if torch.is_tensor(v))
        return losses, params

    l0, p0 = run(False)
    l1, p1 = run(True)
    for a, b in zip(l0, l1):
        assert abs(a - b) < 2e-2, (l0, l1)
    for n in p0:
        c = _cos(p0[n], p1[n]).item()
        assert c > 0.9999, (n, c)


def test_head_dim_64_models_run_attention_on_the_kernels():
    """Llama-3.2-1B / llama_220m have 64-wide heads: attention runs zero-padded on the 128-wide tcgen05 kernels (no
    S x S score matrix), the per-head norm / RoPE kernel is replaced by the PyTorch ops with a warning, and loss and
    gradients follow the fp32 model."""
    import warnings

    from himuon_b200 import ops
    from himuon_b200.models import CausalLM, DecoderConfig

    cfg = DecoderConfig(model_type="llama", vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0,
                        tie_word_embeddings=False, max_position_embeddings=512)
    torch.manual_seed(0)
    ref_model = CausalLM(cfg).cuda().float()
    ker_model = copy.deepcopy(ref_model).bfloat16()
    with torch.no_grad():
        for pr, pk in zip(ref_model.parameters(), ker_model.parameters()):
            pr.copy_(pk.float())
    ids = torch.randint(0, 2048, (2, 256), device="cuda")
    ops._WARNED.clear()
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        peak0 = torch.cuda.max_memory_allocated()
        out_k = ker_model(ids, labels=ids)
        out_k.loss.backward()
    assert any("head_norm_rope" in str(w.message) for w in caught)
    assert not any("ops.attention" in str(w.message) for w in caught), "attention left the kernel path"
    out_r = ref_model(ids, labels=ids)
    out_r.loss.backward()
    torch.cuda.synchronize()
    ops.check_status()
    assert abs(out_k.loss.item() - out_r.loss.item()) < 3e-2
    for (n, pr), pk in zip(ref_model.named_parameters(), ker_model.parameters()):
        c = _cos(pr.grad, pk.grad).item()
        assert c > 0.98, (n, c)
