"""A dependency-free byte-level tokenizer with the call surface ``ToyDataset`` uses.

The reference loads the HF slow tokenizer of the chosen checkpoint from the Hub
(``src/himuon/model.py:17-19``); without network access text is tokenised as UTF-8 bytes
(ids 2..257) with ``eos_token_id`` taken from the model config, which is enough for offline
text runs and for tests.
"""

from __future__ import annotations

import torch


class ByteTokenizer:
    def __init__(self, vocab_size: int, eos_token_id: int = 1):
        self.vocab_size = vocab_size
        self.eos_token_id = eos_token_id
        self.eos_token = "<eos>"
        self.pad_token = None
        self.pad_token_id = None

    def __setattr__(self, key, value):
        super().__setattr__(key, value)
        if key == "pad_token" and value is not None:
            super().__setattr__("pad_token_id", self.eos_token_id)

    def __call__(self, text, add_special_tokens=True, truncation=True, padding="max_length", max_length=1024,
                 return_tensors="pt"):
        ids = [2 + b % max(1, self.vocab_size - 2) for b in text.encode("utf-8")]
        if truncation:
            ids = ids[:max_length]
        n = len(ids)
        pad = self.pad_token_id if self.pad_token_id is not None else self.eos_token_id
        if padding == "max_length":
            ids = ids + [pad] * (max_length - n)
        mask = [1] * n + [0] * (len(ids) - n)
        return {"input_ids": torch.tensor([ids], dtype=torch.long), "attention_mask": torch.tensor([mask], dtype=torch.long)}

    def save_pretrained(self, directory: str):
        import json
        import os

        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, "tokenizer_config.json"), "w") as f:
            json.dump({"tokenizer_class": "ByteTokenizer", "vocab_size": self.vocab_size,
                       "eos_token_id": self.eos_token_id}, f)
