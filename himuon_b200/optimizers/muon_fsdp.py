"""Muon on layer-sharded parameter banks.

Each rank owns whole ``(H, W)`` matrices of a bank (local shard ``(N_local, H, W)``), so the
batched Newton-Schulz over ``N_local`` needs no collective; the step scale comes from the
matrix shape ``(H, W)`` (``src/himuon/optimizers/muon_fsdp.py:54-201``).  Works on DTensor
parameters (local shards via ``to_local()``) and on this package's own sharded banks.
"""

from __future__ import annotations

from .himuon import _local
from .muon import Muon


class MuonFsdp(Muon):
    def _grad(self, p):
        return _local(p.grad)

    def _data(self, p):
        return _local(p.data)
