"""HiMuon: tile-local Newton-Schulz optimizer with cross-layer batching.

Public surface and numerics follow the reference (``src/himuon/optimizers/himuon.py:21-1109``):
same constructor, param-group keys, ``reconfigure()``, ``xlayer_plan()``, static
``newton_schulz`` / ``_tile`` / ``_untile`` helpers and introspection attributes.

The execution model is different.  On a CUDA device one optimizer step is at most

    one `momentum_tile` launch per bucket   (replica sum -> momentum -> Nesterov -> padded tile layout)
    the Newton-Schulz kernels per chunk      (tile-resident fused kernel, or 3 tcgen05 GEMMs per iteration)
    one `untile_apply` launch per bucket     (untile + crop + lr scale + weight decay + parameter update)
    one `adamw_multi` launch per dtype class (all fallback parameters)

driven by device-resident entry tables, and the whole sequence is captured into a single CUDA
graph after ``cuda_graph_warmup`` eager steps.  Learning rate and weight decay live in a small
device table refreshed from the param groups before every launch, so schedulers work without
recapture and the parameter update stays inside the graph.

Sharded parameter banks (3-D ``(N_local, H, W)`` parameters, or DTensors whose local shard is
3-D) are handled per matrix with no collective (``himuon.py:894-964``).  When a bank parameter
carries ``_hm_grad_sources`` (one gradient replica per rank, reachable through peer pointers) the
reduce-scatter is fused into the momentum kernel.
"""

from __future__ import annotations

import math
import struct
import warnings

import torch
from torch.optim import Optimizer

from ..ops import ns as ns_ops
from . import _tablecheck
from ._multi import PinnedHyper
from ..ops import reference as ref

try:  # DTensor support is optional
    from torch.distributed.tensor import DTensor as _DTensor
except Exception:  # pragma: no cover
    _DTensor = None


def _is_dtensor(t) -> bool:
    return _DTensor is not None and isinstance(t, _DTensor)


def _local(t):
    return t.to_local() if _is_dtensor(t) else t


class _Matrix:
    """One 2-D matrix the muon path updates: a whole parameter or one slot of a bank."""

    __slots__ = ("param", "slot", "group_idx", "h", "w", "block", "tile", "R", "C", "tile_base", "full")

    def __init__(self, param, slot, group_idx, h, w):
        self.param, self.slot, self.group_idx, self.h, self.w = param, slot, group_idx, h, w


class HiMuon(Optimizer):
    def __init__(
        self,
        params,
        lr=0.02,
        momentum=0.95,
        nesterov=True,
        weight_decay=0.1,
        tile_size=512,
        ns_steps=5,
        use_muon=True,
        lr_adjust="tile",
        adamw_betas=(0.95, 0.95),
        adamw_eps=1e-8,
        b_hw=None,
        cuda_graph=True,
        cuda_graph_warmup=3,
    ):
        tile_size = self._normalize_defaults(tile_size)
        defaults = dict(
            lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay, tile_size=tile_size,
            ns_steps=ns_steps, use_muon=use_muon, adamw_betas=adamw_betas, adamw_eps=adamw_eps,
        )
        super().__init__(params, defaults)
        if lr_adjust not in ("none", "tile"):
            raise ValueError(f"lr_adjust must be 'none' or 'tile', got {lr_adjust!r}")
        self.lr_adjust = lr_adjust
        self._b_hw_override = b_hw
        self._memory_budget_fraction = 0.15
        self._concat_buffers: dict[tuple, torch.Tensor] = {}
        self._cached_plan: list[dict] | None = None
        self._last_step_stats: dict = {"ns_gpu_ms": 0.0, "ns_launches": 0, "total_B": 0, "avg_batch": 0.0}
        self.profile_ns = False          # True: time the NS launches with CUDA events (one sync per eager step)
        self._cuda_graph_enabled = bool(cuda_graph)
        self._cuda_graph_warmup = int(cuda_graph_warmup)
        self._cuda_graph = None
        self._graph_step_count = 0
        self._in_graph_region = False
        self._pending_updates: list[tuple] = []
        # device-side execution state (CUDA only)
        self._exec = None                # list of per-bucket launch records
        self._adam_exec = None
        self._hyper = None               # PinnedHyper: rotating pinned rows + the device table the kernels read
        self._hyper_dev = None
        self._adam_step = None
        self._ns_workspace = ns_ops.NSWorkspace()
        self._ptr_signature = None
        self._graph_stats = dict(self._last_step_stats)
        self._graph_launches = 0
        if self._cuda_graph_enabled and any(_is_dtensor(p) for g in self.param_groups for p in g["params"]):
            warnings.warn(
                "HiMuon on DTensor parameters with cuda_graph=True: the graph's memory pool and the FSDP "
                "all-gather buffers compete for memory; pass cuda_graph=False or set "
                "PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True.", stacklevel=2)

    # ------------------------------------------------------------------ configuration
    @staticmethod
    def _normalize_defaults(tile_size):
        if isinstance(tile_size, (int, float)) and not isinstance(tile_size, bool):
            tile_size = (int(tile_size), int(tile_size))
        tile_size = tuple(int(t) for t in tile_size)
        assert len(tile_size) == 2 and all(t > 0 for t in tile_size)
        return tile_size

    def adjust_lr_for_muon(self, lr, block_shape):
        if self.lr_adjust == "none":
            return lr
        a, b = block_shape[:2]
        return lr * 0.2 * math.sqrt(max(a, b))

    def reconfigure(self, **updates):
        """Overwrite existing param-group keys in every group (e.g. ``tile_size``) and drop all cached
        plans, buffers and the captured graph (``himuon.py:188-213``).  Unknown keys are ignored."""
        for group in self.param_groups:
            for k, v in updates.items():
                if k in group:
                    group[k] = v
            if "tile_size" in updates:
                group["tile_size"] = self._normalize_defaults(updates["tile_size"])
        self._invalidate_plan_cache()

    def _invalidate_plan_cache(self):
        self._concat_buffers.clear()
        self._cached_plan = None
        self._cuda_graph = None
        self._graph_step_count = 0
        self._pending_updates.clear()
        self._exec = None
        self._adam_exec = None
        self._ptr_signature = None
        self._ns_workspace.clear()

    def load_state_dict(self, state_dict):
        """Restores the state and drops every device entry table: they hold raw addresses of the momentum and
        moment tensors that ``load_state_dict`` has just replaced."""
        super().load_state_dict(state_dict)
        self._invalidate_plan_cache()
        self._adam_step = None

    def xlayer_plan(self) -> list[dict]:
        """Snapshot of the cross-layer bucket plan (``[]`` before the first step and after
        ``reconfigure``).  Whole-matrix work of small plain parameters is scheduled the same way
        internally but, as upstream, is not part of this view."""
        if self._cached_plan is None:
            return []
        return [b for b in self._cached_plan if not b["bucket_key"][2]]

    # ------------------------------------------------------------------ static helpers (public in practice)
    @staticmethod
    def newton_schulz(G, steps=5):
        return ns_ops.newton_schulz(G, steps=steps)

    @staticmethod
    def _tile(tensor, tile_size):
        return ref.tile(tensor, tile_size)

    @staticmethod
    def _untile(tiled, info):
        return ref.untile(tiled, info)

    @staticmethod
    def _balanced_chunks(B_total: int, b_hw: int) -> list[int]:
        if B_total <= 0:
            return []
        n = math.ceil(B_total / b_hw)
        out, remaining = [], B_total
        for i in range(n):
            c = math.ceil(remaining / (n - i))
            out.append(c)
            remaining -= c
        return out

    def _auto_b_hw(self, T: int, dtype_bytes: int = 4) -> int:
        """Largest tile batch per NS call: the user cap, bounded by 15% of device memory for the four
        NS intermediates (``himuon.py:376-403``).  Without CUDA: the user cap or 1."""
        user = self._b_hw_override
        if not torch.cuda.is_available():
            return max(1, int(user)) if user is not None else 1
        total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
        mem_cap = max(1, int(self._memory_budget_fraction * total) // (4 * T * T * dtype_bytes))
        return max(1, min(int(user), mem_cap)) if user is not None else mem_cap

    def _is_dtensor(self, p) -> bool:
        return _is_dtensor(p)

    def _has_dtensor_muon(self) -> bool:
        return any(_is_dtensor(p) for g in self.param_groups if g["use_muon"] for p in g["params"])

    # ------------------------------------------------------------------ planning
    def _collect_matrices(self) -> list[_Matrix]:
        """Every matrix of the muon groups with its routing decision (``himuon.py:483-586``)."""
        mats: list[_Matrix] = []
        kinds = set()
        for gi, group in enumerate(self.param_groups):
            if not group["use_muon"]:
                continue
            th, tw = group["tile_size"]
            for p in group["params"]:
                if p.grad is None and getattr(p, "_hm_grad_sources", None) is None:
                    continue
                lp = _local(p)
                kinds.add("dtensor" if _is_dtensor(p) else "plain")
                if _is_dtensor(p) and lp.ndim != 3:
                    raise NotImplementedError(
                        f"HiMuon on sharded parameters requires bank sharding (3-D shard on the layer axis); got "
                        f"local ndim={lp.ndim}. Wrap the model with wrap_with_banks() before sharding.")
                if lp.ndim == 3:
                    N, H, W = lp.shape
                    skip = getattr(p, "_hm_skip_slots", ())
                    for n in range(N):
                        if n in skip:      # padding slot of a bank: zero forever, nothing to orthogonalise
                            continue
                        m = _Matrix(p, n, gi, H, W)
                        if th >= H and tw >= W:
                            m.full, m.tile, m.block = False, (H, W), (H, W)
                        else:
                            m.full, m.tile, m.block = False, (th, tw), (th, tw)
                        mats.append(m)
                elif lp.ndim == 2:
                    h, w = lp.shape
                    m = _Matrix(p, None, gi, h, w)
                    if h * w <= th * tw:
                        m.full, m.tile, m.block = True, (h, w), (h, w)
                    else:
                        m.full, m.tile, m.block = False, (th, tw), (th, tw)
                    mats.append(m)
                else:
                    raise ValueError(f"HiMuon muon groups take 2-D matrices or 3-D banks, got shape {tuple(lp.shape)}")
        if kinds == {"dtensor", "plain"}:
            raise RuntimeError("HiMuon: muon parameters mix DTensor banks and regular tensors; shard all or none")
        for m in mats:
            m.R = math.ceil(m.h / m.tile[0])
            m.C = math.ceil(m.w / m.tile[1])
        return mats

    def _grad_of(self, p):
        srcs = getattr(p, "_hm_grad_sources", None)
        return srcs[0] if srcs is not None else _local(p.grad)

    def _plan_buckets(self) -> list[dict]:
        """Group tiled matrices by ``(tile_h, tile_w, False, dtype)``; full-matrix NS work is grouped by
        shape the same way but kept out of the public plan, as upstream keeps it per parameter."""
        mats = self._collect_matrices()
        by_key: dict[tuple, list[_Matrix]] = {}
        for m in mats:
            key = (m.tile[0], m.tile[1], bool(m.full), self._grad_of(m.param).dtype)
            by_key.setdefault(key, []).append(m)
        plan = []
        for key, ms in by_key.items():
            th, tw, full, dtype = key
            b_hw = self._auto_b_hw(max(th, tw), dtype_bytes=torch.empty((), dtype=dtype).element_size())
            counts, params_seen = {}, []
            for m in ms:
                pid = id(m.param)
                if pid not in counts:
                    counts[pid] = 0
                    params_seen.append(pid)
                counts[pid] += m.R * m.C
            B_total = sum(counts.values())
            chunks = self._balanced_chunks(B_total, b_hw)
            plan.append({
                "bucket_key": key,
                "param_ids": params_seen,
                "tile_count_per_param": [counts[i] for i in params_seen],
                "B_total": B_total,
                "B_hw": b_hw,
                "chunk_sizes": chunks,
                "n_calls": len(chunks),
                "_entries": ms,
            })
        return plan

    def _ensure_concat_buffer(self, key, B, Th, Tw, device, dtype):
        buf = self._concat_buffers.get(key)
        if buf is None or buf.size(0) < B or buf.size(1) != Th or buf.size(2) != Tw or buf.device != device \
                or buf.dtype != dtype:
            buf = torch.empty((B, Th, Tw), device=device, dtype=dtype)
            self._concat_buffers[key] = buf
        return buf

    # ------------------------------------------------------------------ state helpers
    def _momentum_buffer(self, p):
        st = self.state[p]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros_like(self._grad_of(p))
        return st["momentum_buffer"]

    @staticmethod
    def _view2d(t, slot):
        return t if slot is None else t[slot]

    # ================================================================== torch (CPU / oracle) path
    def _step_torch(self):
        plan = self._cached_plan
        stats = {"ns_gpu_ms": 0.0, "ns_launches": 0, "total_B": 0, "avg_batch": 0.0}
        for bucket in plan:
            th, tw, full, _ = bucket["bucket_key"]
            ms: list[_Matrix] = bucket["_entries"]
            tiles, infos = [], []
            for m in ms:
                group = self.param_groups[m.group_idx]
                g = self._view2d(self._grad_of(m.param), m.slot)
                buf = self._view2d(self._momentum_buffer(m.param), m.slot)
                buf.mul_(group["momentum"]).add_(g)
                upd = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                t, info = ref.tile(upd, (th, tw))
                tiles.append(t.reshape(-1, th, tw))
                infos.append((info, t.shape, g.dtype))
            cat = torch.cat(tiles, 0)
            outs, ofs = [], 0
            steps = self.param_groups[ms[0].group_idx]["ns_steps"]
            for c in bucket["chunk_sizes"]:
                outs.append(ns_ops.newton_schulz(cat[ofs:ofs + c], steps=steps))
                ofs += c
                stats["ns_launches"] += 1
            stats["total_B"] += cat.shape[0]
            orth = torch.cat(outs, 0)
            ofs = 0
            for m, (info, shp, gdtype) in zip(ms, infos):
                group = self.param_groups[m.group_idx]
                n = shp[0] * shp[1]
                u = ref.untile(orth[ofs:ofs + n].view(shp), info).to(gdtype)
                ofs += n
                target = self._view2d(_local(m.param.data), m.slot)
                lr, wd = group["lr"], group["weight_decay"]
                if wd > 0.0:
                    target.mul_(1 - lr * wd)
                target.add_(u.to(target.dtype), alpha=-self.adjust_lr_for_muon(lr, m.block))
        if stats["ns_launches"]:
            stats["avg_batch"] = stats["total_B"] / stats["ns_launches"]
        self._last_step_stats = stats
        for group in self.param_groups:
            if group["use_muon"]:
                continue
            b1, b2 = group["adamw_betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = _local(p.grad)
                st = self.state[p]
                if "step" not in st:
                    st["step"] = torch.zeros((), device=g.device)
                    st["moment1"] = torch.zeros_like(g)
                    st["moment2"] = torch.zeros_like(g)
                st["step"].add_(1)
                st["moment1"].lerp_(g, 1 - b1)
                st["moment2"].lerp_(g.square(), 1 - b2)
                bc1 = 1 - b1 ** st["step"]
                bc2 = 1 - b2 ** st["step"]
                u = (st["moment1"] / bc1) / (st["moment2"].sqrt() / bc2 ** 0.5 + group["adamw_eps"])
                target = _local(p.data)
                if group["weight_decay"] > 0.0:
                    target.mul_(1 - group["lr"] * group["weight_decay"])
                target.add_(u.to(target.dtype), alpha=-group["lr"])

    # ================================================================== CUDA path
    def _pointer_signature(self):
        sig = []
        for group in self.param_groups:
            for p in group["params"]:
                srcs = getattr(p, "_hm_grad_sources", None)
                if srcs is not None:
                    sig.append(tuple(s.data_ptr() for s in srcs))
                elif p.grad is not None:
                    sig.append(_local(p.grad).data_ptr())
                else:
                    sig.append(0)
                sig.append(_local(p.data).data_ptr())
                st = self.state.get(p)
                if st:                                  # state tensors move when they are offloaded between steps
                    for key in ("momentum_buffer", "moment1", "moment2"):
                        v = st.get(key)
                        if torch.is_tensor(v):
                            sig.append(_local(v).data_ptr())
        return tuple(sig)

    def _build_exec(self, device):
        """Device entry tables for every bucket and for the AdamW fallback parameters."""
        from .._ext import ext
        e = ext()
        n_groups = len(self.param_groups)
        self._hyper = PinnedHyper(n_groups, device)
        self._hyper_dev = self._hyper.dev
        if self._adam_step is None:
            # resume the shared step counter from a loaded state dict when there is one
            prior = [st["step"] for st in self.state.values() if isinstance(st, dict) and "step" in st]
            self._adam_step = (prior[0].detach().to(device=device, dtype=torch.float32).clone() if prior
                               else torch.zeros((), dtype=torch.float32, device=device))
            for st in self.state.values():
                if isinstance(st, dict) and "step" in st:
                    st["step"] = self._adam_step
        records = []
        for bucket in self._cached_plan:
            th, tw, full, gdtype = bucket["bucket_key"]
            ms: list[_Matrix] = bucket["_entries"]
            B_total = bucket["B_total"]
            if th % 8 or tw % 8:
                # TMA rows are 16 bytes: a tile side that is not a multiple of 8 is padded with zeros, which
                # leaves the iteration unchanged, but only when the tile is the whole matrix.
                if any(m.R != 1 or m.C != 1 for m in ms):
                    raise ValueError(f"HiMuon on CUDA needs tile sides that are multiples of 8, got ({th}, {tw})")
                th, tw = -(-th // 8) * 8, -(-tw // 8) * 8
            buf = self._ensure_concat_buffer(bucket["bucket_key"], B_total, th, tw, device, torch.bfloat16)
            by_cfg: dict[tuple, list[_Matrix]] = {}
            tile_base = 0
            for m in ms:
                m.tile_base = tile_base
                tile_base += m.R * m.C
                group = self.param_groups[m.group_idx]
                n_src = len(getattr(m.param, "_hm_grad_sources", None) or [None])
                cfg = (float(group["momentum"]), bool(group["nesterov"]), n_src,
                       float(getattr(m.param, "_hm_grad_scale", 1.0)), _local(m.param.data).dtype)
                by_cfg.setdefault(cfg, []).append(m)
            launches = []
            for cfg, sub in by_cfg.items():
                mu, nesterov, n_src, gscale, pdtype = cfg
                mom_tab, app_tab, unit = bytearray(), bytearray(), 0
                for m in sub:
                    srcs = getattr(m.param, "_hm_grad_sources", None)
                    grads = [self._view2d(s, m.slot) for s in srcs] if srcs is not None \
                        else [self._view2d(_local(m.param.grad), m.slot)]
                    for gsrc in grads:
                        if gsrc.stride(-1) != 1:
                            raise RuntimeError("HiMuon: gradients must have unit inner stride")
                    mom = self._view2d(self._momentum_buffer(m.param), m.slot)
                    par = self._view2d(_local(m.param.data), m.slot)
                    ptrs = [g.data_ptr() for g in grads] + [0] * (8 - len(grads))
                    mom_tab += struct.pack("<8QQq6i", *ptrs, mom.data_ptr(), m.tile_base, m.h, m.w, m.R, m.C, unit,
                                           grads[0].stride(0))
                    scale = self.adjust_lr_for_muon(1.0, m.block)
                    app_tab += struct.pack("<Qq6ifi", par.data_ptr(), m.tile_base, m.h, m.w, m.R, m.C, unit,
                                           m.group_idx, scale, par.stride(0))
                    unit += e.momentum_tile_units(m.R, m.C, th)
                if _tablecheck.enabled():
                    ext_ranges = _tablecheck.Extents()
                    for m in sub:
                        for t in (getattr(m.param, "_hm_grad_sources", None) or [_local(m.param.grad)]):
                            ext_ranges.add(t)
                        ext_ranges.add(self._momentum_buffer(m.param))
                        ext_ranges.add(_local(m.param.data))
                    units_of = lambda R, C: e.momentum_tile_units(R, C, th)   # noqa: E731
                    _tablecheck.check_momentum_table(bytes(mom_tab), len(sub), th, tw, buf.shape[0], units_of, unit, n_src,
                                                     4 if gdtype == torch.float32 else 2, ext_ranges)
                    _tablecheck.check_apply_table(bytes(app_tab), len(sub), th, tw, buf.shape[0], units_of, unit, n_groups,
                                                  4 if pdtype == torch.float32 else 2, ext_ranges)
                launches.append({
                    "mom_tab": torch.frombuffer(mom_tab, dtype=torch.uint8).to(device),
                    "app_tab": torch.frombuffer(app_tab, dtype=torch.uint8).to(device),
                    "n": len(sub), "units": unit, "mu": mu, "nesterov": nesterov, "n_src": n_src, "gscale": gscale,
                    "grad_fp32": gdtype == torch.float32, "param_fp32": pdtype == torch.float32,
                })
            steps = self.param_groups[ms[0].group_idx]["ns_steps"]
            records.append({"key": bucket["bucket_key"], "buf": buf, "B": B_total, "th": th, "tw": tw,
                            "chunks": bucket["chunk_sizes"], "launches": launches, "steps": steps})
        self._exec = records
        # ---- AdamW fallback parameters, one table per (param dtype, grad dtype)
        adam: dict[tuple, dict] = {}
        for gi, group in enumerate(self.param_groups):
            if group["use_muon"]:
                continue
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = _local(p.grad)
                if not g.is_contiguous():
                    raise RuntimeError("HiMuon: AdamW-fallback gradients must be contiguous")
                st = self.state[p]
                if "moment1" not in st:
                    st["step"] = self._adam_step
                    st["moment1"] = torch.zeros_like(g)
                    st["moment2"] = torch.zeros_like(g)
                par = _local(p.data)
                rec = adam.setdefault((par.dtype, g.dtype), {"tab": bytearray(), "n": 0, "units": 0, "live": []})
                rec["tab"] += struct.pack("<4Qqq2i", par.data_ptr(), g.data_ptr(), st["moment1"].data_ptr(),
                                          st["moment2"].data_ptr(), par.numel(), rec["units"], gi, 0)
                rec["n"] += 1
                rec["units"] += (par.numel() + 4095) // 4096
                rec["live"] += [par, g, st["moment1"], st["moment2"]]
        if _tablecheck.enabled():
            for (pdt, gdt), r in adam.items():
                _tablecheck.check_adam_table(bytes(r["tab"]), r["n"], r["units"], n_groups, pdt.itemsize, gdt.itemsize,
                                             _tablecheck.Extents(r["live"]))
        self._adam_exec = [
            {"tab": torch.frombuffer(r["tab"], dtype=torch.uint8).to(device), "n": r["n"], "units": r["units"],
             "param_fp32": k[0] == torch.float32, "state_fp32": k[1] == torch.float32}
            for k, r in adam.items()
        ]
        self._pending_updates = [(m.param, None, m.group_idx) for b in self._cached_plan for m in b["_entries"]]

    def _refresh_hyper(self):
        h = self._hyper.begin()
        for gi, group in enumerate(self.param_groups):
            h[gi, 0] = group["lr"]
            h[gi, 1] = group["weight_decay"]
            h[gi, 2], h[gi, 3] = group["adamw_betas"]
            h[gi, 4] = group["adamw_eps"]
        self._hyper.commit()

    def _launch_all(self, timing: list | None = None):
        from .._ext import ext
        from ..ops import _count
        e = ext()
        stats = {"ns_gpu_ms": 0.0, "ns_launches": 0, "total_B": 0, "avg_batch": 0.0}
        for rec in self._exec:
            buf, th, tw = rec["buf"], rec["th"], rec["tw"]
            for L in rec["launches"]:
                e.momentum_tile(L["mom_tab"], L["n"], L["units"], th, tw, buf, L["mu"], L["nesterov"], L["gscale"],
                                L["n_src"], L["grad_fp32"])
                _count()
            ofs = 0
            for c in rec["chunks"]:
                if timing is not None:
                    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    ev0.record()
                ns_ops.ns_inplace_cuda(buf[ofs:ofs + c], rec["steps"], workspace=self._ns_workspace)
                if timing is not None:
                    ev1.record()
                    timing.append((ev0, ev1))
                ofs += c
                stats["ns_launches"] += 1
            stats["total_B"] += rec["B"]
            for L in rec["launches"]:
                e.untile_apply(L["app_tab"], L["n"], L["units"], th, tw, buf, self._hyper_dev, L["param_fp32"])
                _count()
        for A in self._adam_exec:
            e.adamw_multi(A["tab"], A["n"], A["units"], self._hyper_dev, self._adam_step, 0, A["param_fp32"],
                          A["state_fp32"])
            _count()
        if self._adam_exec:
            e.adamw_step_advance(self._adam_step)
            _count()
        if stats["ns_launches"]:
            stats["avg_batch"] = stats["total_B"] / stats["ns_launches"]
        return stats

    def _step_cuda(self, device):
        sig = self._pointer_signature()
        if self._exec is None or sig != self._ptr_signature:
            if self._cuda_graph is not None:
                warnings.warn("HiMuon: gradient or parameter addresses changed after graph capture; recapturing "
                              "(call zero_grad(set_to_none=False) to keep them stable)")
                self._cuda_graph = None
                self._graph_step_count = 0
            self._build_exec(device)
            self._ptr_signature = sig
        self._refresh_hyper()
        if self._cuda_graph is not None:
            from ..ops import _count
            self._cuda_graph.replay()
            _count(self._graph_launches)      # the kernels recorded in the graph run again on every replay
            self._graph_step_count += 1
            self._last_step_stats = dict(self._graph_stats, ns_gpu_ms=0.0)
            return
        use_graph = self._cuda_graph_enabled
        if use_graph and self._graph_step_count >= self._cuda_graph_warmup:
            from ..ops import _count, launch_count
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            self._in_graph_region = True
            before = launch_count()
            try:
                with torch.cuda.graph(graph):
                    stats = self._launch_all()
            finally:
                self._in_graph_region = False
            self._graph_launches = launch_count() - before
            _count(-self._graph_launches)     # capture records the kernels without running them
            _count(self._graph_launches)      # ... and the replay below runs them once
            self._cuda_graph = graph
            self._graph_stats = stats
            graph.replay()
            self._graph_step_count += 1
            self._last_step_stats = dict(stats, ns_gpu_ms=0.0)
            return
        timing = [] if self.profile_ns else None
        stats = self._launch_all(timing)
        if timing:
            torch.cuda.synchronize()
            stats["ns_gpu_ms"] = sum(a.elapsed_time(b) for a, b in timing)
        self._last_step_stats = stats
        self._graph_step_count += 1

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._cached_plan is None:
            self._cached_plan = self._plan_buckets()
        device = None
        for group in self.param_groups:
            for p in group["params"]:
                device = _local(p.data).device
                break
            if device is not None:
                break
        if device is not None and device.type == "cuda":
            self._step_cuda(device)
        else:
            self._step_torch()
        return loss
