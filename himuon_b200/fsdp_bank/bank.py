"""Data model of a parameter bank: same-shape per-layer matrices stacked to ``(n_padded, H, W)``
(``src/himuon/fsdp_bank/bank.py:19-70``)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch.nn as nn


@dataclass
class BankSpec:
    name: str
    matrix_shape: tuple[int, int]
    source_param_names: list[str]
    n_padded: int

    @property
    def n_logical(self) -> int:
        return len(self.source_param_names)

    @property
    def n_pad_rows(self) -> int:
        return self.n_padded - self.n_logical


@dataclass
class ParamBank:
    spec: BankSpec
    parameter: nn.Parameter | None
    name_to_idx: dict[str, int] = field(default_factory=dict)
