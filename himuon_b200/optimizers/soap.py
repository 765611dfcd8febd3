"""SOAP: Adam run in the eigenbasis of Shampoo's preconditioner (https://arxiv.org/abs/2409.11321).

Constructor, defaults and state keys (``step``, ``exp_avg``, ``exp_avg_sq``, ``GG``, ``Q``) follow
``src/himuon/optimizers/soap.py:14-500``: per-mode Gram statistics ``GG[k]`` kept as an EMA, an
``eigh`` initialisation of the bases, a power-iteration + QR refresh every
``precondition_frequency`` steps (with the second moment re-ordered to follow the sorted basis),
and a first step that only gathers statistics.  Single-process / DDP only, as upstream.

On a CUDA device, 2-D bf16 parameters whose sides are multiples of 8 take the kernel path
(``_step_matrix_cuda``): the six rotations of a step (``Q_L^T G Q_R`` for the gradient and for the first moment,
``Q_L R Q_R^T`` back) and the two Gram-matrix updates are tcgen05 GEMMs - the Gram EMA (``GG <- beta GG +
(1-beta) G G^T``, fp32) and the parameter update with its weight decay are fused into GEMM epilogues - and the
moment updates and the Adam ratio in the eigenbasis are the ``soap_moments`` / ``soap_ratio`` kernels.  The
eigendecompositions (``eigh`` once, power iteration + ``qr`` every ``precondition_frequency`` steps) stay on
``torch.linalg`` (cuSOLVER), as does every other parameter shape.
"""

from __future__ import annotations

from itertools import chain

import torch
from torch.optim import Optimizer


class SOAP(Optimizer):
    def __init__(
        self,
        params,
        lr: float = 3e-3,
        betas=(0.95, 0.95),
        shampoo_beta: float = -1,
        eps: float = 1e-8,
        weight_decay: float = 0.01,
        precondition_frequency: int = 10,
        max_precond_dim: int = 10000,
        merge_dims: bool = False,
        precondition_1d: bool = False,
        normalize_grads: bool = False,
        data_format: str = "channels_first",
        correct_bias: bool = True,
    ):
        defaults = dict(lr=lr, betas=betas, shampoo_beta=shampoo_beta, eps=eps, weight_decay=weight_decay,
                        precondition_frequency=precondition_frequency, max_precond_dim=max_precond_dim,
                        merge_dims=merge_dims, precondition_1d=precondition_1d, normalize_grads=normalize_grads,
                        correct_bias=correct_bias)
        super().__init__(params, defaults)
        self._data_format = data_format

    # ------------------------------------------------------------------ shape handling
    def merge_dims(self, grad, max_precond_dim):
        """Greedily fold consecutive dims while their product stays <= ``max_precond_dim``."""
        assert self._data_format in ("channels_first", "channels_last")
        if self._data_format == "channels_last" and grad.dim() == 4:
            grad = grad.permute(0, 3, 1, 2)
        merged, run = [], 1
        for size in grad.shape:
            if run * size > max_precond_dim:
                if run > 1:
                    merged.append(run)
                    run = size
                else:
                    merged.append(size)
                    run = 1
            else:
                run *= size
        if run > 1 or not merged:
            merged.append(run)
        return grad.reshape(merged)

    def _work_view(self, t, group):
        """The tensor in the shape the preconditioner acts on, plus what is needed to undo it."""
        if not group["merge_dims"]:
            return t, None
        permuted = t.dim() == 4 and self._data_format == "channels_last"
        base_shape = t.permute(0, 3, 1, 2).shape if permuted else t.shape
        return self.merge_dims(t, group["max_precond_dim"]), (base_shape, permuted)

    @staticmethod
    def _restore_view(t, undo):
        if undo is None:
            return t
        base_shape, permuted = undo
        t = t.reshape(base_shape)
        return t.permute(0, 2, 3, 1) if permuted else t

    # ------------------------------------------------------------------ preconditioner
    def init_preconditioner(self, grad, state, group):
        beta = group["shampoo_beta"] if group["shampoo_beta"] >= 0 else group["betas"][1]
        state["GG"] = []
        if grad.dim() == 1:
            if group["precondition_1d"] and grad.shape[0] <= group["max_precond_dim"]:
                state["GG"].append(torch.zeros(grad.shape[0], grad.shape[0], device=grad.device))
            else:
                state["GG"].append([])
        else:
            work, _ = self._work_view(grad, group)
            for size in work.shape:
                if size > group["max_precond_dim"]:
                    state["GG"].append([])
                else:
                    state["GG"].append(torch.zeros(size, size, device=grad.device))
        state["Q"] = None
        state["precondition_frequency"] = group["precondition_frequency"]
        state["shampoo_beta"] = beta

    @staticmethod
    def _mode_gram(work, k):
        others = list(chain(range(k), range(k + 1, work.dim())))
        return torch.tensordot(work, work, dims=[others, others])

    def update_preconditioner(self, grad, state, group):
        """EMA of the per-mode Gram matrices; (re)compute the eigenbases when due."""
        beta = state["shampoo_beta"]
        if grad.dim() == 1:
            if group["precondition_1d"] and grad.shape[0] <= group["max_precond_dim"]:
                g = grad.float()
                state["GG"][0].lerp_(torch.outer(g, g), 1 - beta)
        elif self._kernel_ok(grad, grad, state, group):
            self._gram_update_cuda(grad, state)
        else:
            work, _ = self._work_view(grad, group)
            work = work.float()
            for k, gg in enumerate(state["GG"]):
                if len(gg):
                    gg.lerp_(self._mode_gram(work, k), 1 - beta)
        if state["Q"] is None:
            state["Q"] = self._eigenbases(state["GG"])
        if state["step"] > 0 and state["step"] % state["precondition_frequency"] == 0:
            state["Q"] = self._refresh_bases(state, group)

    @staticmethod
    def _eigenbases(grams):
        """Eigenvectors (descending eigenvalue order) of each Gram matrix via ``eigh``."""
        out = []
        for gg in grams:
            if not len(gg):
                out.append([])
                continue
            m = gg.float()
            try:
                _, vecs = torch.linalg.eigh(m + 1e-30 * torch.eye(m.shape[0], device=m.device))
            except Exception:  # retry in double precision
                _, vecs = torch.linalg.eigh(m.double() + 1e-30 * torch.eye(m.shape[0], device=m.device, dtype=torch.float64))
                vecs = vecs.float()
            out.append(torch.flip(vecs, [1]))
        return out

    def _refresh_bases(self, state, group):
        """One power-iteration step followed by QR; keeps ``exp_avg_sq`` aligned with the re-sorted basis."""
        sq = state["exp_avg_sq"]
        work_sq, undo = self._work_view(sq, group)
        new_q = []
        for k, (gg, q) in enumerate(zip(state["GG"], state["Q"])):
            if not len(gg):
                new_q.append([])
                continue
            m, o = gg.float(), q.float()
            ritz = torch.diag(o.T @ m @ o)
            order = torch.argsort(ritz, descending=True)
            work_sq = work_sq.index_select(k, order)
            o = o[:, order]
            qn, _ = torch.linalg.qr(m @ o)
            new_q.append(qn)
        state["exp_avg_sq"] = self._restore_view(work_sq, undo).contiguous()
        return new_q

    def _rotate(self, t, state, group, back: bool):
        """Apply every mode's basis (``back=False``: into the eigenbasis, ``True``: out of it).

        Contracting mode 0 with ``tensordot`` moves the result to the last position, so after one pass
        over all modes the original order is restored; unpreconditioned modes are cycled the same way."""
        work, undo = self._work_view(t, group)
        for q in state["Q"]:
            if len(q):
                work = torch.tensordot(work, q.to(work.dtype), dims=[[0], [1 if back else 0]])
            else:
                work = work.permute(list(range(1, work.dim())) + [0])
        return self._restore_view(work, undo)

    def project(self, grad, state, group):
        return self._rotate(grad, state, group, back=False)

    def project_back(self, grad, state, group):
        return self._rotate(grad, state, group, back=True)

    # ------------------------------------------------------------------ kernel path (2-D bf16 matrices on CUDA)
    @staticmethod
    def _kernel_ok(p, grad, state, group) -> bool:
        if not (grad.is_cuda and grad.dtype == torch.bfloat16 and p.dtype == torch.bfloat16 and grad.dim() == 2):
            return False
        if group["merge_dims"] or group["normalize_grads"] or not grad.is_contiguous() or not p.is_contiguous():
            return False
        m, n = grad.shape
        if m % 8 or n % 8 or max(m, n) > group["max_precond_dim"]:
            return False
        gg = state.get("GG")
        return gg is None or all(len(g) for g in gg)

    @staticmethod
    def _q16(state):
        """bf16 copies of the eigenbases for the rotation GEMMs (rebuilt whenever the bases change)."""
        if state.get("_Q16_src") is not state["Q"]:
            state["_Q16"] = [q.to(torch.bfloat16).contiguous() for q in state["Q"]]
            state["_Q16_src"] = state["Q"]
        return state["_Q16"]

    def _gram_update_cuda(self, grad, state):
        from .. import ops
        beta = state["shampoo_beta"]
        ggl, ggr = state["GG"]
        ops.gemm(grad, grad, trans_b=True, alpha=1 - beta, beta=beta, aux=ggl, out=ggl)      # GG_L <- b GG_L + (1-b) G G^T
        ops.gemm(grad, grad, trans_a=True, alpha=1 - beta, beta=beta, aux=ggr, out=ggr)      # GG_R <- b GG_R + (1-b) G^T G

    def _step_matrix_cuda(self, p, grad, state, group):
        from .. import _ext, ops
        e = _ext.ext()
        b1, b2 = group["betas"]
        ql, qr = self._q16(state)
        g_rot = ops.gemm(ops.gemm(ql, grad, trans_a=True), qr)                 # Q_L^T G Q_R
        state["step"] += 1
        e.soap_moments(grad, g_rot, state["exp_avg"], state["exp_avg_sq"], b1, b2)
        m_rot = ops.gemm(ops.gemm(ql, state["exp_avg"], trans_a=True), qr)     # Q_L^T M Q_R
        e.soap_ratio(m_rot, state["exp_avg_sq"], m_rot, group["eps"])
        ops._count(2)
        step_size = group["lr"]
        if group["correct_bias"]:
            step_size = step_size * (1 - b2 ** state["step"]) ** 0.5 / (1 - b1 ** state["step"])
        keep = 1.0 - group["lr"] * group["weight_decay"] if group["weight_decay"] > 0.0 else 1.0
        # p <- (p - step * Q_L R Q_R^T) * (1 - lr*wd), the update and the decoupled decay in the last GEMM's epilogue
        ops.gemm(ops.gemm(ql, m_rot), qr, trans_b=True, alpha=-step_size * keep, beta=keep, aux=p.data, out=p.data)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                state = self.state[p]
                if "step" not in state:
                    state["step"] = 0
                if "exp_avg" not in state:
                    state["exp_avg"] = torch.zeros_like(grad)
                    state["exp_avg_sq"] = torch.zeros_like(grad)
                if "Q" not in state:
                    # first step: gather statistics only, never project with the current gradient
                    self.init_preconditioner(grad, state, group)
                    self.update_preconditioner(grad, state, group)
                    continue
                if self._kernel_ok(p, grad, state, group):
                    self._step_matrix_cuda(p, grad, state, group)
                    self.update_preconditioner(grad, state, group)
                    continue
                g_rot = self.project(grad, state, group)
                state["step"] += 1
                state["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                state["exp_avg_sq"].mul_(b2).add_(g_rot.square().to(state["exp_avg_sq"].dtype), alpha=1 - b2)
                denom = state["exp_avg_sq"].sqrt().add_(group["eps"])
                m_rot = self.project(state["exp_avg"], state, group)
                step_size = group["lr"]
                if group["correct_bias"]:
                    step_size = step_size * (1 - b2 ** state["step"]) ** 0.5 / (1 - b1 ** state["step"])
                upd = self.project_back(m_rot / denom.to(m_rot.dtype), state, group)
                if group["normalize_grads"]:
                    upd = upd / (1e-30 + upd.square().mean().sqrt())
                p.add_(upd.to(p.dtype), alpha=-step_size)
                if group["weight_decay"] > 0.0:
                    p.add_(p, alpha=-group["lr"] * group["weight_decay"])
                self.update_preconditioner(grad, state, group)
        return loss
