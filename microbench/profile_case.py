"""Small single-kernel workloads for Nsight Compute captures and event timing:
``python -m microbench.profile_case <case>``.  Inputs exceed the 126 MB L2 but stay below 1 GB; each case launches its
kernel a handful of times and prints the CUDA-event time with achieved TFLOP/s or GB/s."""

from __future__ import annotations

import math
import sys

import torch

from himuon_b200._ext import ext
from himuon_b200.ops import ns as ns_ops


def _time(fn, n=5):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


def case_gemm():
    M, N, K = 8192, 8192, 2560
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: ext().gemm(a, b, c, None, False, True, 1.0, 0.0, False, 0))
    print(f"gemm {M}x{N}x{K} NT: {ms:.3f} ms, {2 * M * N * K / 1e9 / ms:.0f} TFLOP/s")


def case_gemm_wgrad():
    M, N, K = 9728, 2560, 8192
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: ext().gemm(a, b, c, c, True, False, 1.0, 1.0, False, 0))
    print(f"gemm wgrad {M}x{N}x{K} TN accumulate: {ms:.3f} ms, {2 * M * N * K / 1e9 / ms:.0f} TFLOP/s")


def case_ns512():
    x = torch.randn(512, 512, 512, device="cuda", dtype=torch.bfloat16)
    ws = ns_ops.NSWorkspace()
    ms = _time(lambda: ns_ops.ns_inplace_cuda(x.clone(), 5, workspace=ws), n=3)
    print(f"NS5 512 tiles of 512x512: {ms:.3f} ms, {512 * 15 * 2 * 512 ** 3 / 1e9 / ms:.0f} TFLOP/s")


def case_ns1024():
    x = torch.randn(96, 1024, 1024, device="cuda", dtype=torch.bfloat16)
    ws = ns_ops.NSWorkspace()
    ms = _time(lambda: ns_ops.ns_inplace_cuda(x.clone(), 5, workspace=ws), n=3)
    print(f"NS5 96 tiles of 1024x1024: {ms:.3f} ms, {96 * 15 * 2 * 1024 ** 3 / 1e9 / ms:.0f} TFLOP/s (full-product FLOPs)")


def case_ns_products():
    """The three products of one Newton-Schulz iteration on 512 tiles of 512x512, one launch each: the two symmetric
    ones with and without the symmetric-output mode."""
    from himuon_b200 import ops
    X = torch.randn(512, 512, 512, device="cuda", dtype=torch.bfloat16) / 23
    A, Bm, Y = torch.empty_like(X), torch.empty_like(X), torch.empty_like(X)
    fl = 512 * 2 * 512 ** 3 / 1e9
    for sym in (False, True):
        m1 = _time(lambda: ops.gemm(X, X, trans_b=True, out=A, symmetric=sym))
        m2 = _time(lambda: ops.gemm(A, A, trans_b=True, alpha=2.0315, beta=-4.775, aux=A, out=Bm, symmetric=sym))
        print(f"symmetric={sym}: X X^T {m1:.3f} ms ({fl / m1:.0f} TFLOP/s of full-product FLOPs) | c A A + b A {m2:.3f} ms ({fl / m2:.0f})")
    m3 = _time(lambda: ops.gemm(Bm, X, alpha=1.0, beta=3.4445, aux=X, out=Y, round_acc=True))
    print(f"B X + a X {m3:.3f} ms ({fl / m3:.0f} TFLOP/s)")


def case_ns128():
    x = torch.randn(8192, 128, 128, device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(x)
    ms = _time(lambda: ext().ns5_fused(x, y, 5, 1e-7))
    print(f"fused NS5 8192 tiles of 128x128: {ms:.3f} ms, {8192 * 15 * 2 * 128 ** 3 / 1e9 / ms:.0f} TFLOP/s")


def case_attn():
    B, S, Hq, Hkv = 4, 2048, 32, 8
    q = torch.randn(B * S, Hq * 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B * S, Hkv * 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    o, lse = torch.empty_like(q), torch.empty(B * Hq * S, device="cuda")
    sc = 1 / math.sqrt(128)
    fl = 4 * B * Hq * S * S * 128 / 2 / 1e9
    ms = _time(lambda: ext().flash_attn_fwd(q, k, v, o, lse, B, S, Hq, Hkv, sc))
    do, dq, dk, dv, delta = torch.randn_like(q), torch.empty_like(q), torch.empty_like(k), torch.empty_like(k), torch.empty_like(lse)
    part = torch.empty(2, B * S, Hq * 128, device="cuda", dtype=torch.bfloat16)
    msb = _time(lambda: ext().flash_attn_bwd(do, q, k, v, o, lse, dq, dk, dv, delta, part, B, S, Hq, Hkv, sc))
    print(f"attention B{B} S{S} H{Hq}/{Hkv}: fwd {ms:.3f} ms {fl / ms:.0f} TFLOP/s, bwd {msb:.3f} ms {2.5 * fl / msb:.0f} TFLOP/s")


def case_attn_train():
    """The attention shape of the headline training step: micro-batch 2 x sequence 1024, 32 query / 8 KV heads."""
    B, S, Hq, Hkv = 2, 1024, 32, 8
    q = torch.randn(B * S, Hq * 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B * S, Hkv * 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    o, lse = torch.empty_like(q), torch.empty(B * Hq * S, device="cuda")
    sc = 1 / math.sqrt(128)
    fl = 4 * B * Hq * S * S * 128 / 2 / 1e9
    ms = _time(lambda: ext().flash_attn_fwd(q, k, v, o, lse, B, S, Hq, Hkv, sc), n=20)
    do, dq, dk, dv, delta = torch.randn_like(q), torch.empty_like(q), torch.empty_like(k), torch.empty_like(k), torch.empty_like(lse)
    part = torch.empty(2, B * S, Hq * 128, device="cuda", dtype=torch.bfloat16)
    msb = _time(lambda: ext().flash_attn_bwd(do, q, k, v, o, lse, dq, dk, dv, delta, part, B, S, Hq, Hkv, sc), n=20)
    print(f"attention B{B} S{S} H{Hq}/{Hkv}: fwd {ms:.3f} ms {fl / ms:.0f} TFLOP/s, bwd {msb:.3f} ms {2.5 * fl / msb:.0f} TFLOP/s")


def case_optim():
    import struct
    e = ext()
    n, H, W, T = 64, 2560, 2560, 512
    g = torch.randn(n, H, W, device="cuda", dtype=torch.bfloat16)
    m = torch.zeros_like(g)
    p = torch.randn_like(g)
    R = C = H // T
    tab_m, tab_a, unit = bytearray(), bytearray(), 0
    for i in range(n):
        tab_m += struct.pack("<8QQq6i", g[i].data_ptr(), 0, 0, 0, 0, 0, 0, 0, m[i].data_ptr(), i * R * C, H, W, R, C, unit, W)
        tab_a += struct.pack("<Qq6ifi", p[i].data_ptr(), i * R * C, H, W, R, C, unit, 0, 4.5, W)
        unit += e.momentum_tile_units(R, C, T)
    tm, ta = torch.frombuffer(tab_m, dtype=torch.uint8).cuda(), torch.frombuffer(tab_a, dtype=torch.uint8).cuda()
    tiles = torch.empty(n * R * C, T, T, device="cuda", dtype=torch.bfloat16)
    hyper = torch.tensor([0.01, 0.1, 0, 0, 0, 0, 0, 0], device="cuda")
    gb = g.numel() * 2 / 1e9
    ms1 = _time(lambda: e.momentum_tile(tm, n, unit, T, T, tiles, 0.95, True, 1.0, 1, False))
    ms2 = _time(lambda: e.untile_apply(ta, n, unit, T, T, tiles, hyper, False))
    ms3 = _time(lambda: e.ns_normalize(tiles, n * R * C, T * T, 1e-7))
    print(f"momentum_tile {ms1:.3f} ms {4 * gb / ms1 * 1e3:.0f} GB/s | untile_apply {ms2:.3f} ms {3 * gb / ms2 * 1e3:.0f} GB/s | "
          f"ns_normalize {ms3:.3f} ms {3 * gb / ms3 * 1e3:.0f} GB/s")


def case_step():
    """One full training step (forward, backward, HiMuon step) of a small Qwen3-style model: every kernel of the
    library launches at least once."""
    import argparse

    from himuon_b200.models import CausalLM, DecoderConfig
    from himuon_b200.optim import get_optimizer

    torch.manual_seed(0)
    cfg = DecoderConfig(model_type="qwen3", vocab_size=32768, hidden_size=1024, intermediate_size=3072, num_hidden_layers=2,
                        num_attention_heads=8, num_key_value_heads=4, head_dim=128, tie_word_embeddings=True,
                        max_position_embeddings=2048)
    model = CausalLM(cfg).to("cuda", torch.bfloat16)
    opt = get_optimizer("himuon", model, argparse.Namespace(lr=0.01, weight_decay=0.1, tile_size=512, cuda_graph=False))
    ids = torch.randint(0, cfg.vocab_size, (4, 1024), device="cuda")
    for _ in range(2):
        loss = model(ids, labels=ids).loss
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=False)
    torch.cuda.synchronize()
    print(f"step case done, loss {loss.item():.3f}")


CASES = {"gemm": case_gemm, "gemm_wgrad": case_gemm_wgrad, "ns512": case_ns512, "ns1024": case_ns1024,
         "ns_products": case_ns_products, "ns128": case_ns128, "attn": case_attn, "attn_train": case_attn_train,
         "optim": case_optim, "step": case_step}

if __name__ == "__main__":
    for name in sys.argv[1:] or list(CASES):
        CASES[name]()
