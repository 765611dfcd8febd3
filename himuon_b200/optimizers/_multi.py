"""Shared helper: run the multi-tensor AdamW kernel over a list of parameters."""

from __future__ import annotations

import struct

import torch

from . import _tablecheck


class PinnedHyper:
    """Per-group hyper-parameter rows (lr, wd, betas, eps) staged through pinned host memory.

    The device copy is refreshed by an asynchronous copy before every step, so the host row that copy reads must
    not be rewritten while it may still be in flight: the rows rotate through ``depth`` pinned buffers and each
    carries the event recorded after its last copy, which the host waits on before reusing the buffer.
    """

    def __init__(self, n_groups: int, device, depth: int = 2):
        self.dev = torch.zeros(n_groups, 8, dtype=torch.float32, device=device)
        pin = torch.device(device).type == "cuda"
        self._hosts = [torch.zeros(n_groups, 8, dtype=torch.float32) for _ in range(depth)]
        if pin:
            self._hosts = [h.pin_memory() for h in self._hosts]
        self._events = [None] * depth
        self._cur = 0
        self._cuda = pin

    @property
    def n_groups(self) -> int:
        return self.dev.shape[0]

    def begin(self) -> torch.Tensor:
        """The host rows to fill for the coming step (waits until the copy that last read them has finished)."""
        self._cur = (self._cur + 1) % len(self._hosts)
        ev = self._events[self._cur]
        if ev is not None:
            ev.synchronize()
        return self._hosts[self._cur]

    def commit(self) -> torch.Tensor:
        """Issue the host-to-device copy of the rows handed out by ``begin()``; returns the device table."""
        self.dev.copy_(self._hosts[self._cur], non_blocking=True)
        if self._cuda:
            ev = self._events[self._cur] or torch.cuda.Event()
            ev.record()
            self._events[self._cur] = ev
        return self.dev


class AdamTable:
    """Device entry tables for ``adamw_multi`` keyed by (param dtype, state dtype); rebuilt when any
    parameter / gradient address changes."""

    def __init__(self):
        self.sig = None
        self.recs = []
        self.hyper = None
        self.hyper_host = None          # the rows being filled for the coming step (see PinnedHyper.begin)
        self.hyper_dev = None
        self.step = None

    def build(self, items, n_groups, device, start_step: float = 0.0):
        """``items``: list of (param_local, grad_local, m, v, group_idx).  ``start_step``: number of steps already
        taken with these moments (a loaded state dict), so bias correction continues instead of restarting."""
        by: dict[tuple, dict] = {}
        for par, g, m, v, gi in items:
            rec = by.setdefault((par.dtype, g.dtype), {"tab": bytearray(), "n": 0, "units": 0, "live": []})
            rec["tab"] += struct.pack("<4Qqq2i", par.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                      par.numel(), rec["units"], gi, 0)
            rec["n"] += 1
            rec["units"] += (par.numel() + 4095) // 4096
            rec["live"] += [par, g, m, v]
        if _tablecheck.enabled():
            for (pdt, gdt), r in by.items():
                _tablecheck.check_adam_table(bytes(r["tab"]), r["n"], r["units"], n_groups, pdt.itemsize, gdt.itemsize,
                                             _tablecheck.Extents(r["live"]))
        self.recs = [
            {"tab": torch.frombuffer(r["tab"], dtype=torch.uint8).to(device), "n": r["n"], "units": r["units"],
             "param_fp32": k[0] == torch.float32, "state_fp32": k[1] == torch.float32}
            for k, r in by.items()
        ]
        if self.hyper is None or self.hyper.n_groups != n_groups:
            self.hyper = PinnedHyper(n_groups, device)
            self.hyper_dev = self.hyper.dev
        if self.step is None:
            self.step = torch.full((), float(start_step), dtype=torch.float32, device=device)

    def begin_hyper(self) -> torch.Tensor:
        self.hyper_host = self.hyper.begin()
        return self.hyper_host

    def launch(self, mode: int):
        from .._ext import ext
        from ..ops import _count
        e = ext()
        self.hyper.commit()
        for r in self.recs:
            e.adamw_multi(r["tab"], r["n"], r["units"], self.hyper_dev, self.step, mode, r["param_fp32"], r["state_fp32"])
            _count()
        if self.recs:
            e.adamw_step_advance(self.step)
            _count()
