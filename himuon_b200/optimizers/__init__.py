"""Optimizers: HiMuon (tile-local NS), its legacy per-parameter variant, Muon, Muon on sharded
banks, AdamW and SOAP - the same set as ``src/himuon/optimizers/__init__.py`` upstream."""

from .adamw import AdamW
from .himuon import HiMuon
from .himuon_legacy import HiMuonLegacy
from .muon import Muon, zeropower_via_newtonschulz5
from .muon_fsdp import MuonFsdp
from .soap import SOAP

__all__ = ["AdamW", "HiMuon", "HiMuonLegacy", "Muon", "MuonFsdp", "SOAP", "zeropower_via_newtonschulz5"]
