"""Shared helper: run the multi-tensor AdamW kernel over a list of parameters."""

from __future__ import annotations

import struct

import torch


class AdamTable:
    """Device entry tables for ``adamw_multi`` keyed by (param dtype, state dtype); rebuilt when any
    parameter / gradient address changes."""

    def __init__(self):
        self.sig = None
        self.recs = []
        self.hyper_host = None
        self.hyper_dev = None
        self.step = None

    def build(self, items, n_groups, device):
        """``items``: list of (param_local, grad_local, m, v, group_idx)."""
        by: dict[tuple, dict] = {}
        for par, g, m, v, gi in items:
            rec = by.setdefault((par.dtype, g.dtype), {"tab": bytearray(), "n": 0, "units": 0})
            rec["tab"] += struct.pack("<4Qqq2i", par.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                      par.numel(), rec["units"], gi, 0)
            rec["n"] += 1
            rec["units"] += (par.numel() + 4095) // 4096
        self.recs = [
            {"tab": torch.frombuffer(r["tab"], dtype=torch.uint8).to(device), "n": r["n"], "units": r["units"],
             "param_fp32": k[0] == torch.float32, "state_fp32": k[1] == torch.float32}
            for k, r in by.items()
        ]
        if self.hyper_dev is None or self.hyper_dev.shape[0] != n_groups:
            self.hyper_host = torch.zeros(n_groups, 8, dtype=torch.float32).pin_memory()
            self.hyper_dev = torch.zeros(n_groups, 8, dtype=torch.float32, device=device)
        if self.step is None:
            self.step = torch.zeros((), dtype=torch.float32, device=device)

    def launch(self, mode: int):
        from .._ext import ext
        from ..ops import _count
        e = ext()
        self.hyper_dev.copy_(self.hyper_host, non_blocking=True)
        for r in self.recs:
            e.adamw_multi(r["tab"], r["n"], r["units"], self.hyper_dev, self.step, mode, r["param_fp32"], r["state_fp32"])
            _count()
        if self.recs:
            e.adamw_step_advance(self.step)
            _count()
