"""Earlier HiMuon variant: per-parameter tiled Newton-Schulz, no cross-layer bucketing and no
CUDA graph (``src/himuon/optimizers/himuon_legacy.py:9-233``).  It exists as the comparison
point of the optimizer-step microbenchmark; numerics match HiMuon's tiled path."""

from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from ..ops import ns as ns_ops
from ..ops import reference as ref
from .himuon import HiMuon


class HiMuonLegacy(Optimizer):
    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, weight_decay=0.1, tile_size=512, ns_steps=5,
                 use_muon=True, lr_adjust="tile", adamw_betas=(0.95, 0.95), adamw_eps=1e-8):
        tile_size = HiMuon._normalize_defaults(tile_size)
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay, tile_size=tile_size,
                        ns_steps=ns_steps, use_muon=use_muon, adamw_betas=adamw_betas, adamw_eps=adamw_eps)
        super().__init__(params, defaults)
        if lr_adjust not in ("none", "tile"):
            raise ValueError(f"lr_adjust must be 'none' or 'tile', got {lr_adjust!r}")
        self.lr_adjust = lr_adjust

    def reconfigure(self, **updates):
        for group in self.param_groups:
            for k, v in updates.items():
                if k in group:
                    group[k] = v
            if "tile_size" in updates:
                group["tile_size"] = HiMuon._normalize_defaults(updates["tile_size"])
        self._invalidate_plan_cache()

    def _invalidate_plan_cache(self):
        """Nothing is cached per plan in this variant."""

    @staticmethod
    def newton_schulz(G, steps=5):
        return ns_ops.newton_schulz(G, steps=steps)

    def _scale(self, lr, block):
        return lr if self.lr_adjust == "none" else lr * 0.2 * math.sqrt(max(block[0], block[1]))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, wd = group["lr"], group["weight_decay"]
            if group["use_muon"]:
                th, tw = group["tile_size"]
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    g = p.grad
                    st = self.state[p]
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(g)
                    buf = st["momentum_buffer"]
                    buf.mul_(group["momentum"]).add_(g)
                    upd = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                    if upd.numel() <= th * tw:
                        u, block = self.newton_schulz(upd, group["ns_steps"]), tuple(upd.shape)
                    else:
                        tiled, info = ref.tile(upd, (th, tw))
                        R, C = tiled.shape[:2]
                        orth = self.newton_schulz(tiled.view(R * C, th, tw), group["ns_steps"]).view(R, C, th, tw)
                        u, block = ref.untile(orth, info), (th, tw)
                    if wd > 0.0:
                        p.mul_(1 - lr * wd)
                    p.add_(u.to(p.dtype), alpha=-self._scale(lr, block))
            else:
                b1, b2 = group["adamw_betas"]
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    g = p.grad
                    st = self.state[p]
                    if "step" not in st:
                        st["step"] = torch.zeros((), device=g.device)
                        st["moment1"] = torch.zeros_like(g)
                        st["moment2"] = torch.zeros_like(g)
                    st["step"].add_(1)
                    st["moment1"].lerp_(g, 1 - b1)
                    st["moment2"].lerp_(g.square(), 1 - b2)
                    bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                    u = (st["moment1"] / bc1) / (st["moment2"].sqrt() / bc2 ** 0.5 + group["adamw_eps"])
                    if wd > 0.0:
                        p.mul_(1 - lr * wd)
                    p.add_(u.to(p.dtype), alpha=-lr)
        return loss
