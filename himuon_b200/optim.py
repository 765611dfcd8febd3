"""Optimizer factory: ``--optimizer`` name -> optimizer instance with the right param groups.

Grouping rules follow ``src/himuon/optim.py:7-197``:

* ``adamw`` / ``soap``: two groups - tensors with ``dim >= 2`` (weight decay from the kwargs, default
  0.1) and tensors with ``dim < 2`` (no decay);
* ``muon`` / ``muon-fsdp`` / ``himuon`` / ``himuon-legacy``: three groups - (1) matrices and banks whose
  name contains neither ``embed_tokens`` nor ``lm_head`` (``use_muon=True``), (2) 1-D tensors
  (``use_muon=False``, lr 1e-3, no decay), (3) 2-D embeddings / lm_head (``use_muon=False``, lr 1e-3).

Constructor kwargs are taken from the namespace / dict by signature introspection, ``None`` dropped.
"""

from __future__ import annotations

import inspect
from typing import Any

from torch.optim import Optimizer

from .optimizers import SOAP, AdamW, HiMuon, HiMuonLegacy, Muon, MuonFsdp

_DECAY_SPLIT = {"adamw": AdamW, "soap": SOAP}
_MUON_FAMILY = {"muon": Muon, "muon-fsdp": MuonFsdp, "himuon": HiMuon, "himuon-legacy": HiMuonLegacy}


def get_optimizer_kwargs(optimizer_class: type[Optimizer], kwargs: dict | Any | None = None) -> dict:
    """Entries of ``kwargs`` (dict or namespace) that ``optimizer_class.__init__`` accepts and are not ``None``."""
    if not kwargs:
        return {}
    values = kwargs if isinstance(kwargs, dict) else vars(kwargs)
    accepted = inspect.signature(optimizer_class).parameters.keys()
    return {k: v for k, v in values.items() if k in accepted and v is not None}


def get_optimizer(optimizer_name: str, model: Any, kwargs: dict | Any | None = None) -> Optimizer:
    name = optimizer_name.lower()
    if name in _DECAY_SPLIT:
        cls = _DECAY_SPLIT[name]
        kw = get_optimizer_kwargs(cls, kwargs)
        trainable = [p for p in model.parameters() if p.requires_grad]
        groups = [
            {"params": [p for p in trainable if p.dim() >= 2], "weight_decay": kw.get("weight_decay", 0.1)},
            {"params": [p for p in trainable if p.dim() < 2], "weight_decay": 0.0},
        ]
        return cls(groups, **kw)
    if name in _MUON_FAMILY:
        cls = _MUON_FAMILY[name]
        kw = get_optimizer_kwargs(cls, kwargs)
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]

        def is_head(n):
            return "embed_tokens" in n or "lm_head" in n

        groups = [
            {"params": [p for n, p in named if p.ndim >= 2 and not is_head(n)],
             "weight_decay": kw.get("weight_decay", 0.1), "use_muon": True},
            {"params": [p for n, p in named if p.ndim < 2],
             "lr": kw.get("adamw_lr", 1e-3), "weight_decay": 0.0, "use_muon": False},
            {"params": [p for n, p in named if p.ndim >= 2 and is_head(n)],
             "lr": kw.get("adamw_lr", 1e-3), "weight_decay": kw.get("weight_decay", 0.1), "use_muon": False},
        ]
        return cls(groups, **kw)
    raise ValueError(f"Optimizer {optimizer_name} not supported")
