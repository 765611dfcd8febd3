"""Loss-curve parity at equal seed: the reference stack (HF Qwen3 model + the reference's HiMuon with its Triton
kernels, from baseline/_ref) against this repository (own decoder + sm_100a kernels), same initial weights, same
batches, same hyper-parameters, single GPU, bf16.

    python baseline/loss_parity.py [--steps 40]

Prints both curves and the largest absolute difference.  The data is a fixed synthetic Markov-chain corpus so that the
loss actually falls (uniform-random tokens would stay at ln(vocab))."""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def batches(vocab, steps, batch, seq, device):
    g = torch.Generator().manual_seed(0)
    nxt = torch.randint(0, vocab, (vocab, 4), generator=g)
    out = []
    for _ in range(steps):
        ids = torch.empty(batch, seq, dtype=torch.long)
        ids[:, 0] = torch.randint(0, vocab, (batch,), generator=g)
        ch = torch.randint(0, 4, (batch, seq), generator=g)
        for t in range(1, seq):
            ids[:, t] = nxt[ids[:, t - 1], ch[:, t]]
        out.append(ids.to(device))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--tile", type=int, default=256)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    vocab, hidden, layers = 8192, 512, 4
    data = batches(vocab, args.steps, 8, 512, dev)
    opt_ns = argparse.Namespace(lr=0.02, weight_decay=0.1, tile_size=args.tile, cuda_graph=False)

    # ---- reference stack
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    from transformers import AutoConfig, AutoModelForCausalLM
    import himuon.optim as ref_optim

    torch.manual_seed(0)
    cfg = AutoConfig.for_model("qwen3", vocab_size=vocab, hidden_size=hidden, intermediate_size=1536, num_hidden_layers=layers,
                               num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
                               max_position_embeddings=2048, tie_word_embeddings=True, use_cache=False)
    hf = AutoModelForCausalLM.from_config(cfg).to(dev, torch.bfloat16)
    init = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    hf.train()
    ropt = ref_optim.get_optimizer("himuon", hf, opt_ns)
    ref_losses = []
    for ids in data:
        loss = hf(input_ids=ids, labels=ids).loss
        loss.backward()
        ropt.step()
        ropt.zero_grad(set_to_none=True)
        ref_losses.append(float(loss))
    del hf, ropt
    torch.cuda.empty_cache()

    # ---- this repository
    from himuon_b200.models import CausalLM, DecoderConfig
    from himuon_b200.optim import get_optimizer

    mcfg = DecoderConfig(model_type="qwen3", vocab_size=vocab, hidden_size=hidden, intermediate_size=1536, num_hidden_layers=layers,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
                         tie_word_embeddings=True, max_position_embeddings=2048)
    model = CausalLM(mcfg).to(dev, torch.bfloat16)
    missing = model.load_state_dict(init, strict=False)
    assert not [k for k in missing.missing_keys if "lm_head" not in k], missing
    model.train()
    opt = get_optimizer("himuon", model, opt_ns)
    our_losses = []
    for ids in data:
        loss = model(ids, labels=ids).loss
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        our_losses.append(float(loss))
    diffs = [abs(a - b) for a, b in zip(ref_losses, our_losses)]
    print(json.dumps({"steps": args.steps, "tile": args.tile, "reference": [round(x, 4) for x in ref_losses],
                      "ours": [round(x, 4) for x in our_losses], "max_abs_diff": max(diffs),
                      "mean_abs_diff": sum(diffs) / len(diffs)}))


if __name__ == "__main__":
    main()
