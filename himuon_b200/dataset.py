"""Datasets: tokenised text stream (reference behaviour) and synthetic tokens.

``ToyDataset`` matches ``src/himuon/dataset.py:5-33``: each example is tokenised,
truncated and padded to ``max_length`` with the EOS token and ``labels`` is a copy
of ``input_ids`` (pad positions are *not* masked).  ``SyntheticTokenDataset``
yields uniform-random token ids of the same schema for offline runs.
"""

from __future__ import annotations

from typing import Any, Iterator

import torch
from torch.utils.data import IterableDataset


class ToyDataset(IterableDataset):
    def __init__(self, dataset, tokenizer: Any, max_length: int = 1024) -> None:
        self.dataset = dataset
        self.tokenizer = tokenizer
        self.max_length = max_length
        if self.tokenizer.eos_token_id is None:
            raise ValueError("Tokenizer must have an eos_token defined")
        self.tokenizer.pad_token = self.tokenizer.eos_token

    def __iter__(self) -> Iterator[dict]:
        for example in self.dataset:
            enc = self.tokenizer(
                example["text"],
                add_special_tokens=True,
                truncation=True,
                padding="max_length",
                max_length=self.max_length,
                return_tensors="pt",
            )
            ids = enc["input_ids"].squeeze(0)
            yield {
                "input_ids": ids,
                "attention_mask": enc["attention_mask"].squeeze(0),
                "labels": ids.detach().clone(),
            }


class SyntheticTokenDataset(IterableDataset):
    """Endless stream of i.i.d. uniform token ids, sharded by ``(rank, world_size)``.

    Example ``k`` of rank ``r`` is drawn from a generator seeded with
    ``seed + k * world_size + r`` so every rank sees a distinct, reproducible stream.
    """

    def __init__(self, vocab_size: int, max_length: int = 1024, seed: int = 0,
                 rank: int = 0, world_size: int = 1, num_examples: int | None = None):
        self.vocab_size = int(vocab_size)
        self.max_length = int(max_length)
        self.seed = int(seed)
        self.rank = int(rank)
        self.world_size = int(world_size)
        self.num_examples = num_examples

    def __iter__(self) -> Iterator[dict]:
        k = 0
        while self.num_examples is None or k < self.num_examples:
            gen = torch.Generator().manual_seed(self.seed + k * self.world_size + self.rank)
            ids = torch.randint(0, self.vocab_size, (self.max_length,), generator=gen, dtype=torch.long)
            yield {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()}
            k += 1
