"""AdamW with decoupled weight decay applied after the Adam step.

Same convention as ``src/himuon/optimizers/adamw.py:13-118`` (HF-style): default betas
``(0.9, 0.95)``, ``p -= lr*sqrt(bc2)/bc1 * m/(sqrt(v)+eps)`` then ``p -= lr*wd*p``.  On CUDA all
parameters are updated by one multi-tensor kernel launch per dtype class.
"""

from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from ._multi import AdamTable


class AdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, correct_bias=True):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 <= betas[0] < 1.0 or not 0.0 <= betas[1] < 1.0:
            raise ValueError(f"Invalid betas: {betas}")
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, correct_bias=correct_bias)
        super().__init__(params, defaults)
        self._table = AdamTable()

    def _signature(self):
        # parameter, gradient and moment addresses: the device table is rebuilt when any of them moves
        return tuple((p.data_ptr(), p.grad.data_ptr(), m.data_ptr() if torch.is_tensor(m := self.state[p].get("exp_avg")) else 0)
                     for g in self.param_groups for p in g["params"] if p.grad is not None)

    def load_state_dict(self, state_dict):
        """Restores the state and drops the device entry table (it holds the addresses of the replaced moments)."""
        super().load_state_dict(state_dict)
        self._table = AdamTable()

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        first = next((p for g in self.param_groups for p in g["params"] if p.grad is not None), None)
        if first is None:
            return loss
        if first.is_cuda and all(g["correct_bias"] for g in self.param_groups):
            self._step_cuda(first.device)
            return loss
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                denom = st["exp_avg_sq"].sqrt().add_(group["eps"])
                step_size = group["lr"]
                if group["correct_bias"]:
                    step_size = step_size * math.sqrt(1 - b2 ** st["step"]) / (1 - b1 ** st["step"])
                p.addcdiv_(st["exp_avg"], denom, value=-step_size)
                if group["weight_decay"] > 0.0:
                    p.add_(p, alpha=-group["lr"] * group["weight_decay"])
        return loss

    def _step_cuda(self, device):
        sig = self._signature()
        t = self._table
        if t.sig != sig:
            items = []
            prior = 0
            for gi, group in enumerate(self.param_groups):
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    st = self.state[p]
                    if "exp_avg" in st:                 # moments restored by load_state_dict: keep their step count
                        prior = max(prior, int(st.get("step", 0)))
                    if "exp_avg" not in st:
                        st["step"] = 0
                        st["exp_avg"] = torch.zeros_like(p.grad)
                        st["exp_avg_sq"] = torch.zeros_like(p.grad)
                    items.append((p.data, p.grad.contiguous() if not p.grad.is_contiguous() else p.grad,
                                  st["exp_avg"], st["exp_avg_sq"], gi))
            t.build(items, len(self.param_groups), device, start_step=prior)
            t.sig = sig
        t.begin_hyper()
        for gi, group in enumerate(self.param_groups):
            t.hyper_host[gi, 0] = group["lr"]
            t.hyper_host[gi, 1] = group["weight_decay"]
            t.hyper_host[gi, 2], t.hyper_host[gi, 3] = group["betas"]
            t.hyper_host[gi, 4] = group["eps"]
        t.launch(mode=2)
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    self.state[p]["step"] += 1
