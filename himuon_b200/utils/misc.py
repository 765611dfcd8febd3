"""Seeding, ``key=value`` CLI overrides and a wall-clock budget.

Behaviour follows ``src/himuon/utils.py:11-59`` of the reference: values of
``--kwargs k=v`` are parsed with ``ast.literal_eval`` and fall back to the raw
string; merging warns when a non-``None`` attribute is overridden.
"""

from __future__ import annotations

import ast
import os
import random
import time
import warnings
from datetime import timedelta

import numpy as np
import torch


def seed_everything(seed: int) -> None:
    """Seed python, numpy and torch (all devices) and make cuDNN deterministic."""
    random.seed(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False


def parse_kv_args(raw: list[str]) -> dict:
    """``['a=1', 'b=(2,3)', 'c=foo']`` -> ``{'a': 1, 'b': (2, 3), 'c': 'foo'}``."""
    out: dict = {}
    for item in raw:
        key, value = item.split("=", 1)
        try:
            value = ast.literal_eval(value)
        except (ValueError, SyntaxError):
            pass
        out[key] = value
    return out


def merge_kv_args(args, raw: list[str] | None = None):
    """Merge ``k=v`` pairs into an argparse namespace (in place) and return it."""
    if raw is None:
        raw = getattr(args, "kwargs", []) or []
    for key, value in parse_kv_args(raw).items():
        current = getattr(args, key, None)
        if current is not None:
            warnings.warn(f"'--kwargs {key}={value}' overrides existing arg '{key}={current}'")
        setattr(args, key, value)
    return args


class TimeBudget:
    """Wall-clock budget in hours; ``None``/0 means unlimited."""

    def __init__(self, hours: float | None = None):
        self.start_time = time.monotonic()
        self.deadline = self.start_time + hours * 3600 if hours else float("inf")

    def is_expired(self) -> bool:
        return time.monotonic() >= self.deadline

    def __repr__(self) -> str:
        remaining = self.deadline - time.monotonic()
        if remaining == float("inf"):
            return "inf"
        return str(timedelta(seconds=int(max(0.0, remaining))))
