"""Muon: full-matrix Newton-Schulz orthogonalised momentum with an AdamW fallback.

Semantics of ``src/himuon/optimizers/muon.py:13-195``: momentum (+Nesterov), five quintic NS
iterations on the whole matrix, Moonlight step scale ``0.2*sqrt(max(A, B))``; parameters with
``use_muon=False`` take Adam with ``u = m/(eps + sqrt(v))`` and step ``lr / (bc1/sqrt(bc2))``.
On CUDA the whole muon part of a step runs on the library's kernels: momentum + Nesterov, whole-matrix
Newton-Schulz (same-shape matrices batched) and the scaled, weight-decayed update are exactly HiMuon's step with a
tile that covers every matrix, so ``Muon`` drives a private :class:`HiMuon` over its muon groups (sharing the
per-parameter state dicts, so ``state_dict()`` still shows ``momentum_buffer``); the AdamW fallback is one multi-tensor
launch in Muon's own convention.  DTensor parameters and CPU tensors take the PyTorch ops.
"""

from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from ..ops import ns as ns_ops
from ._multi import AdamTable


def zeropower_via_newtonschulz5(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Orthogonalise ``G`` (2-D or batched) with the quintic Newton-Schulz iteration in bf16."""
    return ns_ops.newton_schulz(G, steps=steps)


class Muon(Optimizer):
    def __init__(self, params, lr=1e-3, weight_decay=0.1, momentum=0.95, nesterov=True, ns_steps=5,
                 use_muon=True, adamw_betas=(0.95, 0.95), adamw_eps=1e-8):
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        use_muon=use_muon, adamw_betas=adamw_betas, adamw_eps=adamw_eps)
        super().__init__(params, defaults)
        self._table = AdamTable()
        self._ws = ns_ops.NSWorkspace()
        self._kernel_muon = None        # private HiMuon over the muon groups (CUDA only), built on first use

    def _muon_on_kernels(self) -> bool:
        """True when every muon parameter with a gradient is a plain 2-D / 3-D bf16 or fp32 CUDA tensor."""
        seen = False
        for g in self.param_groups:
            if not g["use_muon"]:
                continue
            for p in g["params"]:
                if p.grad is None:
                    continue
                if hasattr(p, "to_local") or not p.is_cuda or p.ndim not in (2, 3) \
                        or p.dtype not in (torch.bfloat16, torch.float32) or p.grad.dtype != p.dtype:
                    return False
                seen = True
        return seen

    def _step_muon_kernels(self):
        from .himuon import HiMuon
        muon_groups = [g for g in self.param_groups if g["use_muon"]]
        keys = ("lr", "weight_decay", "momentum", "nesterov", "ns_steps")
        if self._kernel_muon is None or [id(p) for g in muon_groups for p in g["params"]] != self._kernel_muon_ids:
            inner = HiMuon([{"params": g["params"], **{k: g[k] for k in keys}} for g in muon_groups],
                           tile_size=10 ** 9, lr_adjust="tile", cuda_graph=False)
            for g in muon_groups:                         # the same per-parameter dicts: momentum buffers appear in ours
                for q in g["params"]:
                    inner.state[q] = self.state[q]
            self._kernel_muon = inner
            self._kernel_muon_ids = [id(p) for g in muon_groups for p in g["params"]]
        for src, dst in zip(muon_groups, self._kernel_muon.param_groups):
            for k in keys:
                dst[k] = src[k]
        self._kernel_muon.step()

    @staticmethod
    def adjust_lr_for_muon(lr, shape):
        a, b = shape[-2:]
        return lr * 0.2 * math.sqrt(max(a, b))

    # local-tensor hooks (overridden for sharded banks)
    def _grad(self, p):
        return p.grad

    def _data(self, p):
        return p.data

    def load_state_dict(self, state_dict):
        """Restores the state and drops the device entry table (it holds the addresses of the replaced moments)."""
        super().load_state_dict(state_dict)
        self._table = AdamTable()
        self._kernel_muon = None

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._muon_on_kernels():
            self._step_muon_kernels()
            self._step_adamw()
            return loss
        for group in self.param_groups:
            if not group["use_muon"]:
                continue
            by_shape: dict[tuple, list] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = self._grad(p)
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(g)
                buf = st["momentum_buffer"]
                buf.mul_(group["momentum"]).add_(g)
                upd = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                upd3 = upd if upd.ndim == 3 else upd.unsqueeze(0)
                by_shape.setdefault((tuple(upd3.shape[-2:]), upd.dtype), []).append((p, upd3))
            for (shape, _), items in by_shape.items():
                # same-shape matrices share one batched NS call
                stacked = torch.cat([u for _, u in items], 0) if len(items) > 1 else items[0][1]
                orth = ns_ops.newton_schulz(stacked, steps=group["ns_steps"], workspace=self._ws)
                lr, wd = group["lr"], group["weight_decay"]
                ofs = 0
                for p, u in items:
                    n = u.shape[0]
                    target = self._data(p)
                    if wd > 0.0:
                        target.mul_(1 - lr * wd)
                    target.add_(orth[ofs:ofs + n].view(target.shape).to(target.dtype),
                                alpha=-self.adjust_lr_for_muon(lr, shape))
                    ofs += n
        self._step_adamw()
        return loss

    def _step_adamw(self):
        groups = [(gi, g) for gi, g in enumerate(self.param_groups) if not g["use_muon"]]
        first = next((p for _, g in groups for p in g["params"] if p.grad is not None), None)
        if first is None:
            return
        if self._data(first).is_cuda:
            t = self._table
            sig = tuple((self._data(p).data_ptr(), self._grad(p).data_ptr(),
                         m.data_ptr() if torch.is_tensor(m := self.state[p].get("moment1")) else 0)
                        for _, g in groups for p in g["params"] if p.grad is not None)
            if t.sig != sig:
                items = []
                prior = 0
                for gi, group in groups:
                    for p in group["params"]:
                        if p.grad is None:
                            continue
                        g = self._grad(p)
                        st = self.state[p]
                        if "moment1" in st:             # restored by load_state_dict: keep the step count
                            prior = max(prior, int(st.get("step", 0)))
                        if "moment1" not in st:
                            st["step"] = 0
                            st["moment1"] = torch.zeros_like(g)
                            st["moment2"] = torch.zeros_like(g)
                        items.append((self._data(p), g, st["moment1"], st["moment2"], gi))
                t.build(items, len(self.param_groups), self._data(first).device, start_step=prior)
                t.sig = sig
            t.begin_hyper()
            for gi, group in groups:
                t.hyper_host[gi, 0] = group["lr"]
                t.hyper_host[gi, 1] = group["weight_decay"]
                t.hyper_host[gi, 2], t.hyper_host[gi, 3] = group["adamw_betas"]
                t.hyper_host[gi, 4] = group["adamw_eps"]
            t.launch(mode=1)
            for _, group in groups:
                for p in group["params"]:
                    if p.grad is not None:
                        self.state[p]["step"] += 1
            return
        for _, group in groups:
            b1, b2 = group["adamw_betas"]
            eps, lr, wd = group["adamw_eps"], group["lr"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = self._grad(p)
                st = self.state[p]
                if "step" not in st:
                    st["step"] = 0
                    st["moment1"] = torch.zeros_like(g)
                    st["moment2"] = torch.zeros_like(g)
                st["step"] += 1
                st["moment1"].lerp_(g, 1 - b1)
                st["moment2"].lerp_(g.square(), 1 - b2)
                u = st["moment1"] / (eps + st["moment2"].sqrt())
                scale = (1 - b1 ** st["step"]) / math.sqrt(1 - b2 ** st["step"])
                target = self._data(p)
                if wd > 0.0:
                    target.mul_(1 - lr * wd)
                target.add_(u.to(target.dtype), alpha=-lr / scale)
