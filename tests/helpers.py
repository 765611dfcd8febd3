"""Small fakes shared by the CPU tests (a tiny LM with the Hugging Face parameter names, a character
tokenizer with the keyword surface ToyDataset uses, a text stream)."""

import torch
import torch.nn as nn


class TinyCausalLM(nn.Module):
    def __init__(self, vocab=32, hidden=16):
        super().__init__()
        self.embed_tokens = nn.Embedding(vocab, hidden)
        self.norm = nn.LayerNorm(hidden)
        self.mlp = nn.Linear(hidden, hidden, bias=True)
        self.lm_head = nn.Linear(hidden, vocab, bias=False)

    def forward(self, ids):
        return self.lm_head(self.mlp(self.norm(self.embed_tokens(ids))))


class FakeTokenizer:
    def __init__(self, vocab=64, eos=1):
        self.vocab, self.eos_token_id, self.eos_token, self.pad_token = vocab, eos, "<eos>", None

    def __call__(self, text, add_special_tokens=True, truncation=True, padding="max_length", max_length=16,
                 return_tensors="pt"):
        ids = [2 + (ord(c) % (self.vocab - 2)) for c in text][:max_length]
        n = len(ids)
        ids = ids + [self.eos_token_id] * (max_length - n)
        mask = [1] * n + [0] * (max_length - n)
        return {"input_ids": torch.tensor([ids]), "attention_mask": torch.tensor([mask])}


class TextStream:
    def __init__(self, texts):
        self.texts = texts

    def __iter__(self):
        for t in self.texts:
            yield {"text": t}


def make_linear_model(shapes, dtype=torch.float32, device="cpu"):
    return nn.ModuleList([nn.Linear(w, h, bias=False, dtype=dtype, device=device) for h, w in shapes])


def seed_grads(model, seed=0):
    g = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        val = torch.randn(p.shape, generator=g).to(p.device, p.dtype)
        if p.grad is None:
            p.grad = val
        else:
            p.grad.copy_(val)
