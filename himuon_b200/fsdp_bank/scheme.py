"""The protocol a model family implements to be banked (``src/himuon/fsdp_bank/scheme.py:17-46``)."""

from __future__ import annotations

from typing import Protocol, runtime_checkable

import torch.nn as nn

from .bank import BankSpec, ParamBank


@runtime_checkable
class BankScheme(Protocol):
    def collect(self, model: nn.Module, world_size: int) -> list[BankSpec]:
        """Describe the banks: names, matrix shape, source parameter names, padded length."""

    def install(self, model: nn.Module, banks: list[ParamBank]) -> nn.Module:
        """Attach the bank parameters to ``model`` and rewire every source Linear to read its slot."""
