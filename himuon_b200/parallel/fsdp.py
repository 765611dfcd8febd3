"""Bank-sharded engine (the FSDP path).

Same-shape per-layer projections are stacked into ``(n, H, W)`` banks (:mod:`himuon_b200.fsdp_bank`) and sharded on
the layer axis in whole matrices, so the optimizer needs no collective (the reference's layout,
``src/himuon/fsdp_bank`` + ``train_fsdp.py:108-133``).  What this engine decides itself:

* **Placement is round-robin.**  Layer ``l`` of every bank lives on rank ``l % world`` (k|v and gate|up keep their two
  slots together), at local position ``l // world``.  Consecutive layers therefore have different owners - a
  per-layer fetch spreads over all NVLink ports instead of draining one GPU - and the zero pad slots that make the
  layer count a multiple of the world size spread over the ranks too (36 layers on 8 ranks: four ranks own 5 real
  matrices per bank and four own 4, instead of seven owning 5 and one owning 1).
* **Weights: gathered copy or staging ring** (``weights=``).

  - ``"gathered"``: every rank keeps a full bf16 working copy of the peers' layers (its own layers are read from the
    shard itself), refreshed once per optimizer step by copy-engine pulls over NVLink.  The refresh is deferred to the
    start of the next forward pass and issued layer group by layer group on a side stream, and the forward pass waits
    group by group, so all but the first group's copies run beside the first micro-batch (``gather_blocks > 0``
    selects one ``multi_copy`` kernel launch right after the optimizer step instead).  Accumulation micro-steps do no
    parameter communication (180 GB of HBM hold the copy).
  - ``"ring"``: no full copy.  Layers are taken in groups of ``world`` consecutive layers (one per owner); two
    group-sized staging slots rotate.  While group ``g`` computes, a side stream copies group ``g+1`` (``g-1`` in
    backward) from the owners' shards with the copy engines - no SM is taken from the GEMMs, and rank ``r`` visits
    the owners in the order ``r+1, r+2, ...`` so that at any moment every owner serves exactly one reader.  Each
    remote matrix crosses NVLink once per pass and is read by the GEMMs from local memory.  Per-rank weight memory is
    ``1/world`` of the banks plus the two slots.
  - ``"peer"``: no copy at all; the GEMMs' own TMA loads read the owner's shard through its peer mapping.

* **Gradients: replicated or sharded accumulation** (``grads=``).

  - ``"replicated"``: every rank accumulates its micro-batches in a full-bank buffer written by the weight-gradient
    GEMMs' epilogues; the owner sums the ``world`` replicas once per step, inside HiMuon's ``momentum_tile`` kernel
    through peer pointers (other optimizers: one ``reduce_replicas`` launch per bank).  This is what FSDP2 does under
    gradient accumulation too (unsharded gradients accumulate locally, one reduce-scatter per optimizer step).
    With HiMuon on CUDA the peers' replicas of a rank's layers need not wait for the optimizer step (``grad_prefetch``,
    opt-in): in the last micro-batch of a step, whenever the backward pass leaves a layer group, a side stream meets the
    other ranks at a barrier of its own and lets the copy engines pull the peers' finished gradients of this rank's
    layer of the group into local staging buffers, beside the backward GEMMs of the earlier layers;
    ``momentum_tile`` then sums local buffers only and the optimizer step moves nothing over NVLink.
  - ``"sharded"``: no full-bank buffer.  The weight gradients of one layer group land in a group-sized staging
    buffer; when the backward pass leaves the group, every owner sums its layer over the ranks (peer loads) straight
    into its own ``(n_local, H, W)`` accumulator.  Per-rank gradient memory is ``1/world`` of the banks plus one
    group; the price is one reduce-scatter per group per micro-batch on the critical path.

* Embeddings, lm_head and norms stay replicated; their gradients share one fused all-reduce per step.

On CPU (gloo) the same bookkeeping runs over ``torch.distributed`` collectives, which keeps placement, ring rotation
and the fences testable without a GPU.
"""

from __future__ import annotations

import struct
import warnings
from contextlib import contextmanager

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..fsdp_bank import Llama3BankScheme, Qwen3BankScheme, unbank_state_dict, wrap_with_banks
from .fence import LayerFence as _GroupFence
from .symm import SymmetricHeap, _world


class _BankState:
    __slots__ = ("spec", "unit", "n_units", "n_local", "shard", "shard_off", "grad_full", "grad_off", "gathered",
                 "param", "sinks", "pair_sinks", "peer_shards", "ring", "gring", "gring_off", "grad_shard", "grad_peer", "grad_stage")


class ShardedEngine:
    def __init__(self, model: nn.Module, use_banks: bool = True, cpu_offload: bool = False, timeout_s: float = 120.0,
                 gather_blocks: int = 0, peer_weights: bool = False, weights: str | None = None,
                 grads: str = "replicated", nvls: bool = False, debug: bool = False, grad_prefetch: bool = False):
        """``weights``: ``"gathered"`` (default), ``"ring"`` or ``"peer"`` (``peer_weights=True`` is the older spelling
        of the last); ``grads``: ``"replicated"`` (default) or ``"sharded"``; see the module docstring.
        ``nvls``: bind the symmetric heap to an NVLink multicast object; the gradient reductions onto the owners then
        read through it (``multimem.ld_reduce``: the switch sums the ranks' copies, the owner receives one copy's worth
        of bytes instead of ``world - 1``) and the replicated parameters' all-reduce goes through the switch too.
        ``debug``: race / overrun checks for development - guard zones after every heap region (``heap.check_canaries()``,
        verified in ``zero_grad``), host-side bounds checks of the optimizers' device tables, and staging slots and group gradient buffers are filled with NaN whenever their
        contents become stale, so a kernel that reads a slot before its copy has landed poisons the loss visibly.
        ``grad_prefetch``: pull the peers' gradient replicas of this rank's layers group by group during the last
        micro-batch's backward pass (replicated gradients with HiMuon on CUDA; off by default, which leaves the peer
        reads inside ``momentum_tile``: measured on 2 and 4 GPUs the optimizer step gets 5 ms shorter and the last
        backward pass as much longer).
        ``cpu_offload``: keep the optimizer's state tensors in pinned host memory between steps (see
        :class:`OptimizerStateOffload`; the reference's ``--cpu-offload``, ``train_fsdp.py:58,120``)."""
        self.model = model
        self.rank, self.world = _world()
        self.cpu_offload = bool(cpu_offload)
        # gradient pre-fetch (decided in attach_optimizer): a stream of its own, so that weight copies never queue
        # behind a barrier that waits for the slowest rank
        self._grad_prefetch_wanted = grad_prefetch
        self.grad_prefetch = False
        self._grad_stream = None
        self._sync_pass = True
        self.graph_key_sync = False       # True: the synchronising micro-batch gets a CUDA graph of its own
        self.grad_pulls = 0               # layer groups pulled so far (tests, diagnostics)
        self.gather_blocks = gather_blocks
        first = next(model.parameters())
        self.device, self.dtype = first.device, first.dtype
        self.cuda = self.device.type == "cuda"
        weights = weights or ("peer" if peer_weights else "gathered")
        if weights not in ("gathered", "ring", "peer") or grads not in ("replicated", "sharded"):
            raise ValueError(f"ShardedEngine: unknown mode weights={weights!r} grads={grads!r}")
        if weights == "peer" and not (self.cuda and self.dtype == torch.bfloat16):
            weights = "gathered"                      # peer reads exist only in the TMA GEMMs
        if self.world == 1:
            weights, grads = "gathered", "replicated"   # one rank owns everything: the shard is the working copy
        self.weights_mode, self.grads_mode = weights, grads
        self.peer_weights = weights == "peer"
        esz = torch.empty((), dtype=self.dtype).element_size()
        self.banks = None
        bank_full = []
        if use_banks:
            scheme = Llama3BankScheme() if getattr(model.config, "model_type", "qwen3") == "llama" else Qwen3BankScheme()
            model, self.banks = wrap_with_banks(model, scheme, self.world)
            bank_full = [(b, getattr(model, b.spec.name)) for b in self.banks]
        self.n_layers = max((b.spec.n_logical // self._unit_of(b.spec) for b, _ in bank_full), default=0)
        self.n_groups = -(-self.n_layers // self.world) if self.n_layers else 0
        self._pad = 16 * max(1, self.world)
        replicated = [p for n, p in model.named_parameters() if p.requires_grad
                      and (self.banks is None or n not in {b.spec.name for b in self.banks})]
        rep_by_dtype: dict[torch.dtype, list] = {}
        for p in replicated:
            rep_by_dtype.setdefault(p.dtype, []).append(p)
        need = sum(self._padded(sum(p.numel() for p in ps)) * torch.empty((), dtype=dt).element_size() + 4096
                   for dt, ps in rep_by_dtype.items())
        for b, full in bank_full:
            H, W = b.spec.matrix_shape
            unit = self._unit_of(b.spec)
            n_local = unit * self.n_groups
            slots = n_local                                            # the owned shard
            slots += n_local * self.world if grads == "replicated" else unit * self.world   # gradient buffer
            need += slots * H * W * esz + 16384
        self.debug = bool(debug)
        if self.debug:
            need += 64 * SymmetricHeap.CANARY_BYTES + 64 * 1024
            from ..optimizers import _tablecheck
            _tablecheck.enable(True)              # the optimizers validate their device tables against the live tensors
        self.heap = SymmetricHeap(need, self.device, timeout_s, multicast=nvls, canaries=self.debug)
        self.nvls = self.heap.has_multicast

        # ---- replicated parameters: gradients in one flat symmetric region per dtype
        self.regions = []
        for dt, ps in rep_by_dtype.items():
            n = self._padded(sum(p.numel() for p in ps))
            flat, offset = self.heap.alloc((n,), dt)
            flat.zero_()
            cursor = 0
            for p in ps:
                if self.world > 1:
                    dist.broadcast(p.data, src=0)
                p.grad = flat[cursor:cursor + p.numel()].view(p.shape)
                cursor += p.numel()
            self.regions.append((flat, offset))

        # ---- banks
        self.state: dict[str, _BankState] = {}
        for b, full in bank_full:
            st = _BankState()
            st.spec = b.spec
            H, W = b.spec.matrix_shape
            st.unit = self._unit_of(b.spec)
            st.n_units = b.spec.n_logical // st.unit
            st.n_local = st.unit * self.n_groups
            n_phys = st.n_local * self.world
            if self.world > 1:
                dist.broadcast(full.data, src=0)
            st.shard, st.shard_off = self.heap.alloc((st.n_local, H, W), self.dtype)
            st.shard.zero_()
            for s in range(b.spec.n_logical):
                owner, loc = self._place(st, s)
                if owner == self.rank:
                    st.shard[loc].copy_(full.data[s])
            st.grad_full = st.gring = st.grad_shard = st.grad_peer = st.grad_stage = None
            st.grad_off = st.gring_off = 0
            if grads == "replicated":
                st.grad_full, st.grad_off = self.heap.alloc((n_phys, H, W), self.dtype)
                st.grad_full.zero_()
            else:
                st.gring, st.gring_off = self.heap.alloc((st.unit * self.world, H, W), self.dtype)
                st.gring.zero_()
                st.grad_shard = torch.zeros(st.n_local, H, W, device=self.device, dtype=self.dtype)
            st.peer_shards = st.gathered = st.ring = None
            if self.world == 1:
                st.gathered = st.shard
            elif weights == "peer":
                st.peer_shards = [st.shard if r == self.rank else
                                  self.heap.view(r, st.shard_off, (st.n_local, H, W), self.dtype)
                                  for r in range(self.world)]
            elif weights == "ring":
                st.ring = [torch.empty(st.unit * self.world, H, W, device=self.device, dtype=self.dtype) for _ in range(2)]
                if self.cuda:
                    st.peer_shards = [st.shard if r == self.rank else
                                      self.heap.view(r, st.shard_off, (st.n_local, H, W), self.dtype)
                                      for r in range(self.world)]
            else:
                st.gathered = torch.zeros(n_phys, H, W, device=self.device, dtype=self.dtype)
                for s in range(b.spec.n_logical):
                    st.gathered[self._phys(st, s)].copy_(full.data[s])
                if self.cuda:
                    st.peer_shards = [st.shard if r == self.rank else
                                      self.heap.view(r, st.shard_off, (st.n_local, H, W), self.dtype)
                                      for r in range(self.world)]
            param = nn.Parameter(st.shard, requires_grad=True)
            param._bank_spec = b.spec
            # pad slots (layers past the model's depth) hold zeros and need no optimizer work
            param._hm_skip_slots = {lu * st.unit + k for lu in range(self.n_groups) for k in range(st.unit)
                                    if lu * self.world + self.rank >= st.n_units}
            if self.cuda and grads == "replicated":
                slice_off = st.grad_off + self.rank * st.n_local * H * W * esz
                param._hm_grad_sources = [self.heap.view(r, slice_off, (st.n_local, H, W), self.dtype)
                                          for r in range(self.world)]
                param._hm_grad_scale = 1.0 / self.world
            if grads == "sharded":
                param.grad = st.grad_shard
            setattr(model, b.spec.name, param)
            st.param = param
            self._make_sinks(st)
            self.state[b.spec.name] = st
            b.parameter = None            # the un-sharded original is released
        del bank_full
        if self.cuda:
            torch.cuda.empty_cache()
        object.__setattr__(model, "_bank_engine", self if self.banks is not None else None)
        # Gathered copy on CUDA: the once-per-step re-gather is deferred to the next forward pass and issued group by
        # group on the copy stream, so that all but the first group's copies run beside the first micro-batch.
        self._overlap_regather = self.cuda and self.world > 1 and self.banks is not None and weights == "gathered" \
            and gather_blocks <= 0
        self._regather_pending = False
        self._group_ready: dict[int, object] = {}
        object.__setattr__(model, "_layer_hooks", self if (self.uses_fences or self._overlap_regather) else None)
        self.materialize_grads = False    # True: produce .grad for bank shards (optimizers without the fused path)
        self._copy_table = None
        self._offload = None
        # staging-ring bookkeeping (host side; it describes the work enqueued so far, in program order)
        self._slot_group = [None, None]
        self._slot_ready = [None, None]
        self._copy_stream = torch.cuda.Stream(self.device) if (self.cuda and self.world > 1 and weights in ("ring", "gathered")) else None
        self.ring_fetches = 0             # groups copied so far (tests, diagnostics)
        self.group_reductions = 0
        if self.world > 1:
            self.heap.barrier()

    # ------------------------------------------------------------------ placement
    @staticmethod
    def _unit_of(spec) -> int:
        """Slots per layer: 2 for the interleaved k|v and gate|up banks, 1 otherwise."""
        return 2 if spec.name in ("kv_bank", "gate_up_bank") else 1

    def _place(self, st: _BankState, slot: int) -> tuple[int, int]:
        """Bank slot (the index ``rewire_linear`` recorded) -> (owner rank, index in the owner's shard)."""
        u, k = divmod(slot, st.unit)
        return u % self.world, (u // self.world) * st.unit + k

    def _phys(self, st: _BankState, slot: int) -> int:
        """Position of a bank slot in the owner-major full-size buffers (gathered copy, replicated gradients)."""
        owner, loc = self._place(st, slot)
        return owner * st.n_local + loc

    def _ring_pos(self, st: _BankState, slot: int) -> tuple[int, int]:
        """Bank slot -> (layer group, index in a group-sized staging buffer)."""
        u, k = divmod(slot, st.unit)
        return u // self.world, (u % self.world) * st.unit + k

    def _make_sinks(self, st: _BankState):
        H, W = st.spec.matrix_shape
        n = st.spec.n_logical
        if st.grad_full is not None:
            st.sinks = [ops.GradSink(st.grad_full[self._phys(st, s)]) for s in range(n)]
            st.pair_sinks = {s: ops.GradSink(st.grad_full[self._phys(st, s):self._phys(st, s) + 2].view(2 * H, W))
                             for s in range(0, n - 1, 2)} if st.unit == 2 else {}
        else:
            st.sinks = [ops.GradSink(st.gring[self._ring_pos(st, s)[1]]) for s in range(n)]
            st.pair_sinks = {s: ops.GradSink(st.gring[self._ring_pos(st, s)[1]:self._ring_pos(st, s)[1] + 2].view(2 * H, W))
                             for s in range(0, n - 1, 2)} if st.unit == 2 else {}

    def _padded(self, n: int) -> int:
        return -(-n // self._pad) * self._pad

    def bank_bytes(self) -> dict:
        """Bytes this rank holds for bank weights and bank gradients, and the size of the whole (unsharded) banks
        without and with the pad layers that make the layer count a multiple of the world size."""
        esz = torch.empty((), dtype=self.dtype).element_size()
        w = g = total = padded = 0
        for st in self.state.values():
            H, W = st.spec.matrix_shape
            m = H * W * esz
            total += st.spec.n_logical * m
            padded += st.n_local * self.world * m
            w += st.n_local * m
            if st.gathered is not None and st.gathered is not st.shard:
                w += st.gathered.shape[0] * m
            if st.ring is not None:
                w += sum(r.shape[0] for r in st.ring) * m
            if st.grad_full is not None:
                g += st.grad_full.shape[0] * m
            if st.gring is not None:
                g += (st.gring.shape[0] + st.grad_shard.shape[0]) * m
            g += sum(t.shape[0] for t in (st.grad_stage or []) if t is not None) * m
        return {"weights": w, "grads": g, "banks_total": total, "banks_padded": padded}

    # ------------------------------------------------------------------ optimizer hookup
    def attach_optimizer(self, optimizer):
        """HiMuon reads the gradient replicas itself (fused reduce-scatter); any other optimizer gets a reduced
        ``.grad`` on the bank shards.  With ``cpu_offload`` the optimizer's ``step`` is wrapped so that its state
        lives in pinned host memory between steps."""
        from ..optimizers import HiMuon
        # with a multicast heap the replicas are summed by the switch in one reduce launch per bank instead of by peer
        # loads inside momentum_tile
        fused = isinstance(optimizer, HiMuon) and self.cuda and self.grads_mode == "replicated" and not self.nvls
        self.materialize_grads = not fused and self.grads_mode == "replicated"
        if not fused:
            for st in self.state.values():
                if hasattr(st.param, "_hm_grad_sources"):
                    del st.param._hm_grad_sources
        if fused and self.world > 1 and self.weights_mode != "peer" and self._grad_prefetch_wanted and not self.grad_prefetch:
            self.grad_prefetch = True
            self.graph_key_sync = True
            self._grad_stream = torch.cuda.Stream(self.device)
            for st in self.state.values():
                st.grad_peer = list(st.param._hm_grad_sources)       # peer r's replica of this rank's layers
                st.grad_stage = [None if r == self.rank else torch.zeros_like(st.shard) for r in range(self.world)]
                st.param._hm_grad_sources = [st.grad_peer[r] if r == self.rank else st.grad_stage[r]
                                             for r in range(self.world)]
            object.__setattr__(self.model, "_layer_hooks", self)
        if self.cpu_offload and self.cuda:
            self._offload = OptimizerStateOffload(optimizer)
        return optimizer

    # ------------------------------------------------------------------ forward / backward plumbing
    def _weights(self, st: _BankState, idx: int, n: int) -> torch.Tensor:
        """Bank slots ``idx .. idx+n`` as an ``(n, H, W)`` tensor from wherever this mode keeps them: the gathered
        copy, the owner's shard (own layers; or, in peer mode, seen through the peer mapping, which only this
        package's own TMA GEMMs ever read) or the staging slot of the layer's group."""
        owner, loc = self._place(st, idx)
        if st.gathered is not None:
            if self._regather_pending:               # a caller outside the decoder's layer loop: gather everything now
                self._start_regather()
                self._wait_all_groups()
            if owner == self.rank and st.gathered is not st.shard:
                return st.shard[loc:loc + n]          # own layers are read in place; the re-gather skips them
            p = self._phys(st, idx)
            return st.gathered[p:p + n]
        if st.ring is None:
            return st.peer_shards[owner][loc:loc + n]
        if owner == self.rank:
            return st.shard[loc:loc + n]
        g, pos = self._ring_pos(st, idx)
        if self._slot_group[g % 2] != g:
            self._acquire(g)                         # a caller outside the layer loop (or the fences are not in use)
        return st.ring[g % 2][pos:pos + n]

    def linear(self, x, bank_name: str, idx: int, bias=None):
        st = self.state[bank_name]
        if self.world > 1:
            # Looked up again in backward, not saved by autograd: staged weights come and go between the two passes,
            # and own layers are views of the heap-resident shard, whose version counter other heap writes may share.
            y = ops.linear(x, None, sink=st.sinks[idx], w_getter=lambda: self._weights(st, idx, 1)[0])
        else:
            y = ops.linear(x, self._weights(st, idx, 1)[0], sink=st.sinks[idx])
        return y if bias is None else y + bias

    def linear_pair(self, x, bank_name: str, idx: int):
        """Slots ``idx`` and ``idx+1`` applied as one ``(2H, W)`` projection (one GEMM in each direction)."""
        st = self.state[bank_name]
        H, W = st.spec.matrix_shape
        if self.world > 1:
            return ops.linear(x, None, sink=st.pair_sinks[idx],
                              w_getter=lambda: self._weights(st, idx, 2).view(2 * H, W))
        return ops.linear(x, self._weights(st, idx, 2).view(2 * H, W), sink=st.pair_sinks[idx])

    # ---- layer-group fences (called by the decoder's layer loop)
    @property
    def uses_fences(self) -> bool:
        return self.banks is not None and self.world > 1 and (self.weights_mode == "ring" or self.grads_mode == "sharded"
                                                              or self.grad_prefetch)

    def pre_layer(self, i: int, h, delta):
        """Before decoder layer ``i``: at the first layer of a group make the group's weights available and start
        fetching the next group."""
        if i % self.world:
            return h, delta
        g = i // self.world
        if self._overlap_regather:
            if i == 0 and self._regather_pending:
                self._start_regather()
            ready = self._group_ready.pop(g, None)
            if ready is not None:
                torch.cuda.current_stream(self.device).wait_event(ready)
        if not self.uses_fences:
            return h, delta
        if i == 0:
            self._begin_pass()
        if self.weights_mode == "ring":
            self._acquire(g)
            if g + 1 < self.n_groups:
                self._prefetch(g + 1)
        if torch.is_grad_enabled() and h.requires_grad:
            h, delta = _GroupFence.apply(self, "start", g, h, delta)
        return h, delta

    def post_layer(self, i: int, h, delta):
        """After decoder layer ``i``: the last layer of a group closes it (the backward pass enters the group here)."""
        if not self.uses_fences or ((i + 1) % self.world and i + 1 != self.n_layers):
            return h, delta
        if torch.is_grad_enabled() and h.requires_grad:
            h, delta = _GroupFence.apply(self, "end", i // self.world, h, delta)
        return h, delta

    def _start_regather(self):
        """Gathered mode, after an optimizer step: all owners have updated their shards (barrier), then the copy engines
        pull the peers' layers group by group on the copy stream; the forward pass waits group by group, so only the
        first group's copies are exposed.  Runs eagerly or as part of the captured first micro-batch of a step."""
        self._regather_pending = False
        self.heap.barrier()
        ops._count()
        main = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(main)
        self._group_ready = {}
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(start)
            for g in range(self.n_groups):
                for j in range(1, self.world):
                    owner = (self.rank + j) % self.world
                    for st in self.state.values():
                        lo = owner * st.n_local + g * st.unit
                        st.gathered[lo:lo + st.unit].copy_(st.peer_shards[owner][g * st.unit:(g + 1) * st.unit], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._copy_stream)
                self._group_ready[g] = ev

    def _wait_all_groups(self):
        main = torch.cuda.current_stream(self.device)
        for ev in self._group_ready.values():
            main.wait_event(ev)
        self._group_ready = {}

    def _begin_pass(self):
        """A new forward pass.  Group-staged gradient sinks start by overwriting.  The weight staging slots keep what
        they hold: the weights only change in the optimizer step (``zero_grad`` invalidates the slots), and a backward
        pass ends with groups 0 and 1 staged, which is exactly what the next micro-batch's forward pass needs first."""
        if self.grads_mode == "sharded":
            if self.debug:
                for st in self.state.values():
                    st.gring.fill_(float("nan"))
            for st in self.state.values():
                for s in st.sinks:
                    s.reset()
                for s in st.pair_sinks.values():
                    s.reset()

    def _on_backward_boundary(self, kind: str, g: int):
        if kind == "end":                              # the backward pass is about to run group g's layers
            if self.weights_mode == "ring":
                self._acquire(g)
                if g > 0:
                    self._prefetch(g - 1)
        else:                                          # group g's layers are done
            if self.grads_mode == "sharded":
                self._reduce_group(g)
            elif self.grad_prefetch and self._sync_pass:
                self._pull_group_grads(g)

    def _pull_group_grads(self, g: int):
        """Last micro-batch of a step, layer group ``g`` differentiated: once every rank is past the group (a barrier
        on the gradient stream's own channel), copy the peers' accumulated gradients of this rank's layer of the
        group into the local staging buffers the optimizer reads.  Group 0 is the last one of a backward pass; the
        compute stream joins the gradient stream there (inside the micro-batch's CUDA graph when one is captured)."""
        self.grad_pulls += 1
        main = torch.cuda.current_stream(self.device)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(self._grad_stream):
            self._grad_stream.wait_event(done)
            self.heap.barrier(channel=1)
            ops._count()
            for j in range(1, self.world):
                src = (self.rank + j) % self.world     # every rank's memory is read by one puller at a time
                for st in self.state.values():
                    if g * self.world + self.rank >= st.n_units:
                        continue                       # this rank's slot of the group is a pad layer
                    lo, hi = g * st.unit, (g + 1) * st.unit
                    st.grad_stage[src][lo:hi].copy_(st.grad_peer[src][lo:hi], non_blocking=True)
            if g == 0:
                landed = torch.cuda.Event()
                landed.record(self._grad_stream)
        if g == 0:
            main.wait_event(landed)

    def _prefetch(self, g: int):
        """Start copying layer group ``g`` into its staging slot.  The copies are ordered after everything enqueued on
        the compute stream so far (the slot's previous group is no longer needed at this point of the layer loop)."""
        slot = g % 2
        if self._slot_group[slot] == g:
            return
        self._slot_group[slot] = g
        self.ring_fetches += 1
        if not self.cuda:
            for st in self.state.values():
                dist.all_gather_into_tensor(st.ring[slot], st.shard[g * st.unit:(g + 1) * st.unit].contiguous())
            self._slot_ready[slot] = None
            return
        main = torch.cuda.current_stream(self.device)
        free = torch.cuda.Event()
        free.record(main)
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(free)
            # owners in the order rank+1, rank+2, ...: at any moment every owner is read by exactly one rank
            for j in range(1, self.world):
                owner = (self.rank + j) % self.world
                for st in self.state.values():
                    dst = st.ring[slot][owner * st.unit:(owner + 1) * st.unit]
                    dst.copy_(st.peer_shards[owner][g * st.unit:(g + 1) * st.unit], non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(self._copy_stream)
        self._slot_ready[slot] = ready

    def _acquire(self, g: int):
        """Make the compute stream wait until layer group ``g`` sits in its staging slot (fetching it now if no
        prefetch is under way)."""
        slot = g % 2
        if self._slot_group[slot] != g:
            self._prefetch(g)
        ready = self._slot_ready[slot]
        if ready is not None:
            torch.cuda.current_stream(self.device).wait_event(ready)
            self._slot_ready[slot] = None

    def _reduce_group(self, g: int):
        """Sharded gradients: add this micro-batch's gradients of layer group ``g``, summed over the ranks, to the
        owners' accumulators.  Every rank owns one layer of the group, so this is a reduce-scatter; the barriers
        before and after make the peers' staging buffers complete before they are read and free before the next
        group overwrites them."""
        self.group_reductions += 1
        scale = 1.0 / self.world
        if not self.cuda:
            for st in self.state.values():
                work = st.gring.float()
                dist.all_reduce(work)
                if g * self.world + self.rank < st.n_units:
                    mine = work[self.rank * st.unit:(self.rank + 1) * st.unit] * scale
                    st.grad_shard[g * st.unit:(g + 1) * st.unit].add_(mine.to(self.dtype))
            return
        self.heap.barrier()
        ops._count()
        for st in self.state.values():
            if g * self.world + self.rank >= st.n_units:
                continue                               # this rank's slot of the group is a pad layer
            H, W = st.spec.matrix_shape
            esz = st.shard.element_size()
            off = st.gring_off + self.rank * st.unit * H * W * esz
            self.heap.comm.reduce_to(off, st.grad_shard[g * st.unit:(g + 1) * st.unit], scale, 1.0, self.nvls)
            ops._count()
        self.heap.barrier()
        ops._count()

    @contextmanager
    def no_sync(self):
        """Accumulation micro-steps: nothing is exchanged (the gradient pre-fetch belongs to the last micro-batch)."""
        prev, self._sync_pass = self._sync_pass, False
        try:
            yield
        finally:
            self._sync_pass = prev

    def finish_backward(self):
        """Make every rank's accumulated gradients visible and reduce what the optimizer cannot reduce itself."""
        if self.world == 1:
            if self.materialize_grads:
                for st in self.state.values():
                    st.param.grad = st.grad_full
            return
        for flat, offset in self.regions:          # also orders this rank after every peer's backward
            big = flat.numel() * flat.element_size() > (256 << 10)
            self.heap.allreduce_(flat, offset, 1.0 / self.world, algo=3 if (self.nvls and big) else 0)
        if not self.regions:
            self.heap.barrier()
        if not self.materialize_grads:
            return
        for st in self.state.values():
            H, W = st.spec.matrix_shape
            lo = self.rank * st.n_local
            if st.param.grad is None:
                st.param.grad = torch.empty_like(st.shard)
            if self.cuda:
                esz = st.shard.element_size()
                self.heap.comm.reduce_to(st.grad_off + lo * H * W * esz, st.param.grad, 1.0 / self.world, 0.0, self.nvls)
                ops._count()
            else:
                work = st.grad_full.float()
                dist.all_reduce(work)
                st.param.grad.copy_(work[lo:lo + st.n_local] / self.world)

    def zero_grad(self, set_to_none: bool = False):
        """Runs after ``optimizer.step()``: refresh the gathered working copy and reset the accumulators."""
        if self.world > 1:
            if self._overlap_regather:
                self._wait_all_groups()            # leftovers of a forward pass that stopped early
                self._regather_pending = True      # barrier + copies happen at the start of the next forward pass
            else:
                self.heap.barrier()                # every owner has finished updating its shards
                self._regather()
        for flat, _ in self.regions:
            flat.zero_()
        for st in self.state.values():
            for s in st.sinks:
                s.reset()
            for s in st.pair_sinks.values():
                s.reset()
            if st.grad_shard is not None:
                st.grad_shard.zero_()
            if self.materialize_grads and set_to_none and self.world > 1:
                st.param.grad = None
        self._slot_group = [None, None]            # the shards changed: staged copies are stale
        self._slot_ready = [None, None]
        if self.debug:
            for st in self.state.values():
                for slot in (st.ring or []):
                    slot.fill_(float("nan"))
                for stage in (st.grad_stage or []):
                    if stage is not None:              # pad slots keep zeros (momentum_tile skips them)
                        for lu in range(self.n_groups):
                            if lu * self.world + self.rank < st.n_units:
                                stage[lu * st.unit:(lu + 1) * st.unit].fill_(float("nan"))
            bad = self.heap.check_canaries()
            if bad:
                raise RuntimeError(f"ShardedEngine(debug): heap guard zones overwritten at offsets {bad}")

    def _regather(self):
        if all(st.gathered is None for st in self.state.values()):
            return                                   # ring / peer modes keep no gathered copy
        if not self.cuda:
            for st in self.state.values():
                dist.all_gather_into_tensor(st.gathered, st.shard.contiguous())
            return
        if self.gather_blocks <= 0:
            # Copy engines (measured 0.94 of the peer-copy rate against 0.55 for the SM copy kernel at two ranks):
            # one copy per (owner, bank), owners in the order rank+1, rank+2, ... so that every owner serves one
            # reader at a time.  Own layers are read from the shard itself (see _weights), so nothing is copied for them.
            for j in range(1, self.world):
                r = (self.rank + j) % self.world
                for st in self.state.values():
                    if st.gathered is None:
                        continue
                    H, W = st.spec.matrix_shape
                    src = self.heap.view(r, st.shard_off, (st.n_local, H, W), self.dtype)
                    st.gathered[r * st.n_local:(r + 1) * st.n_local].copy_(src, non_blocking=True)
            return
        if self._copy_table is None:                 # gather_blocks > 0: the multi_copy kernel on that many blocks
            ext = self.heap._ext
            tab, units, n = bytearray(), 0, 0
            for st in self.state.values():
                if st.gathered is None:
                    continue
                H, W = st.spec.matrix_shape
                nbytes = st.n_local * H * W * st.shard.element_size()
                for r in range(self.world):
                    src = self.heap.view(r, st.shard_off, (st.n_local, H, W), self.dtype)
                    dst = st.gathered[r * st.n_local:(r + 1) * st.n_local]
                    tab += struct.pack("<QQqq", src.data_ptr(), dst.data_ptr(), nbytes, units)
                    units += int(ext.multi_copy_units(nbytes))
                    n += 1
            self._copy_table = (torch.frombuffer(tab, dtype=torch.uint8).to(self.device), n, units)
        tab, n, units = self._copy_table
        self.heap.comm.copy_segments(tab, n, units, self.gather_blocks)
        ops._count()

    # ------------------------------------------------------------------ checkpoints
    def full_state_dict(self) -> dict:
        """Full, un-banked state dict with the Hugging Face ``model.layers.{i}.*`` keys on rank 0 (``{}`` on the other
        ranks, which do not write; the reference gathers to rank 0 the same way, ``train_fsdp.py:285-297``).  The
        banks are gathered one at a time from the owners' shards."""
        sd = {}
        bank_names = set(self.state)
        if self.rank == 0:
            for k, v in self.model.state_dict().items():
                if k not in bank_names:
                    sd[k] = v.detach().cpu()
        if self.banks is None:
            return sd
        for name, st in self.state.items():
            if self.world > 1:
                full = torch.empty(st.n_local * self.world, *st.spec.matrix_shape, device=self.device, dtype=self.dtype)
                dist.all_gather_into_tensor(full, st.shard.detach().contiguous())
            else:
                full = st.shard.detach()
            if self.rank == 0:
                order = torch.tensor([self._phys(st, s) for s in range(st.spec.n_logical)], device=full.device)
                canon = full.index_select(0, order).cpu()
                pad = st.spec.n_padded - canon.shape[0]
                if pad > 0:
                    canon = torch.cat([canon, canon.new_zeros(pad, *canon.shape[1:])], 0)
                sd[name] = canon
            del full
        return unbank_state_dict(sd, self.banks) if self.rank == 0 else {}

    def close(self):
        if self._offload is not None:
            self._offload.restore()
            self._offload = None
        for p in self.model.parameters():
            p.grad = None
            if hasattr(p, "_hm_grad_sources"):
                del p._hm_grad_sources
        self.state = {}
        self.regions = []
        self._copy_table = None
        self.heap.close()


class OptimizerStateOffload:
    """Keeps an optimizer's state tensors (momentum, Adam moments) in pinned host memory between steps.

    ``step()`` is wrapped: the state is copied to the device right before it and back to the host right after, both
    asynchronously on the compute stream, and the device copies are released in between, so the forward and backward
    passes have that memory for activations.  This is the part of FSDP2's ``CPUOffloadPolicy``
    (``train_fsdp.py:58,120``) that matters on a 180 GB device; parameters and gradients stay in HBM because every
    GEMM needs them.  Device addresses of the state change from step to step, so CUDA-graph capture of the optimizer
    is switched off and the optimizers' device tables are rebuilt when they notice the change.
    """

    def __init__(self, optimizer):
        self.optimizer = optimizer
        self._host: dict[tuple, torch.Tensor] = {}
        if getattr(optimizer, "_cuda_graph_enabled", False):
            warnings.warn("cpu_offload: CUDA-graph capture of the optimizer step is disabled (state addresses change)")
            optimizer._cuda_graph_enabled = False
            if hasattr(optimizer, "_invalidate_plan_cache"):
                optimizer._invalidate_plan_cache()
        self._inner_step = optimizer.step
        optimizer.step = self._step
        self.bytes_offloaded = 0

    def _step(self, *a, **k):
        self._load()
        out = self._inner_step(*a, **k)
        self._store()
        return out

    def _load(self):
        for p, st in self.optimizer.state.items():
            for key, v in list(st.items()):
                if torch.is_tensor(v) and v.device.type == "cpu" and (id(p), key) in self._host:
                    st[key] = v.to(p.device, non_blocking=True)

    def _store(self):
        total = 0
        for p, st in self.optimizer.state.items():
            for key, v in list(st.items()):
                if torch.is_tensor(v) and v.is_cuda and v.numel() > 1:
                    host = self._host.get((id(p), key))
                    if host is None or host.shape != v.shape or host.dtype != v.dtype:
                        host = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                        self._host[(id(p), key)] = host
                    host.copy_(v, non_blocking=True)
                    st[key] = host
                    total += v.numel() * v.element_size()
        self.bytes_offloaded = total

    def restore(self):
        """Bring the state back to the device and unwrap ``step`` (before a state-dict save, or at shutdown)."""
        self._load()
        self.optimizer.step = self._inner_step
