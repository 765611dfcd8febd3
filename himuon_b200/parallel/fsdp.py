"""Bank-sharded engine (the FSDP path).

Same-shape per-layer projections are stacked into ``(n_padded, H, W)`` banks
(:mod:`himuon_b200.fsdp_bank`) and sharded on the layer axis: rank ``r`` owns the contiguous slots
``[r*N_local, (r+1)*N_local)`` of every bank, i.e. whole matrices, so the optimizer needs no
collective (the reference's layout, ``src/himuon/fsdp_bank`` + ``train_fsdp.py:108-133``).

What differs from the reference's FSDP2 execution:

* **All-gather once per optimizer step, not per micro-step.**  180 GB of HBM hold a full bf16
  working copy of every bank, refreshed after each optimizer step by one ``multi_copy`` launch that
  pulls the peers' shards over NVLink; all accumulation micro-steps reuse it.
* **Weight gradients go straight into a symmetric full-bank buffer** (the wgrad GEMM accumulates in
  its epilogue), never through autograd's index-select backward.
* **Reduce-scatter fused into the optimizer.**  The owner reads the ``world`` replicas of its slots
  through peer pointers inside HiMuon's ``momentum_tile`` kernel (sum -> 1/world -> momentum -> tile
  layout); other optimizers get a plain ``.grad`` from one ``reduce_replicas`` launch.
* Embeddings, lm_head and norms stay replicated; their gradients share the fused all-reduce.

On CPU (gloo) the same bookkeeping runs over ``torch.distributed`` collectives.
"""

from __future__ import annotations

import struct
from contextlib import contextmanager

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..fsdp_bank import Llama3BankScheme, Qwen3BankScheme, unbank_state_dict, wrap_with_banks
from .symm import SymmetricHeap, _world


class _BankState:
    __slots__ = ("spec", "n_local", "shard", "shard_off", "grad_full", "grad_off", "gathered", "param", "sinks",
                 "pair_sinks", "peer_shards")


class ShardedEngine:
    def __init__(self, model: nn.Module, use_banks: bool = True, cpu_offload: bool = False, timeout_s: float = 120.0,
                 gather_blocks: int = 0, peer_weights: bool = False):
        """``peer_weights``: keep no gathered copy of the banks; every projection's GEMM (forward and dgrad) reads
        the weight tiles by TMA straight from the owner rank's shard over NVLink, so the all-gather is fused into the
        GEMMs' operand loads.  Saves one full copy of the banks and the per-step re-gather at the price of fetching
        the weights over NVLink in every micro-step; off by default (180 GB of HBM hold the copy)."""
        self.model = model
        self.rank, self.world = _world()
        self.cpu_offload = cpu_offload
        self.gather_blocks = gather_blocks
        first = next(model.parameters())
        self.device, self.dtype = first.device, first.dtype
        self.cuda = self.device.type == "cuda"
        self.peer_weights = bool(peer_weights) and self.cuda and self.dtype == torch.bfloat16
        esz = torch.empty((), dtype=self.dtype).element_size()
        self.banks = None
        bank_full = []
        if use_banks:
            scheme = Llama3BankScheme() if getattr(model.config, "model_type", "qwen3") == "llama" else Qwen3BankScheme()
            model, self.banks = wrap_with_banks(model, scheme, self.world)
            bank_full = [(b, getattr(model, b.spec.name)) for b in self.banks]
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
            need += (b.spec.n_padded // self.world + b.spec.n_padded) * H * W * esz + 8192
        self.heap = SymmetricHeap(need, self.device, timeout_s)

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

        # ---- banks: owned shard + full-bank gradient buffer in the heap, gathered working copy outside it
        self.state: dict[str, _BankState] = {}
        for b, full in bank_full:
            st = _BankState()
            st.spec = b.spec
            H, W = b.spec.matrix_shape
            n_pad = b.spec.n_padded
            st.n_local = n_pad // self.world
            if self.world > 1:
                dist.broadcast(full.data, src=0)
            st.shard, st.shard_off = self.heap.alloc((st.n_local, H, W), self.dtype)
            st.shard.copy_(full.data[self.rank * st.n_local:(self.rank + 1) * st.n_local])
            st.grad_full, st.grad_off = self.heap.alloc((n_pad, H, W), self.dtype)
            st.grad_full.zero_()
            st.peer_shards = None
            if self.world == 1:
                st.gathered = st.shard
            elif self.peer_weights and st.n_local % 2 == 0:       # an even shard: no k|v or gate|up pair straddles ranks
                st.gathered = None
                st.peer_shards = [st.shard if r == self.rank else
                                  self.heap.view(r, st.shard_off, (st.n_local, H, W), self.dtype)
                                  for r in range(self.world)]
            else:
                st.gathered = torch.empty(n_pad, H, W, device=self.device, dtype=self.dtype)
                st.gathered.copy_(full.data)
            param = nn.Parameter(st.shard, requires_grad=True)
            param._bank_spec = b.spec
            lo = self.rank * st.n_local
            param._hm_skip_slots = {i for i in range(st.n_local) if lo + i >= b.spec.n_logical}
            if self.cuda:
                slice_off = st.grad_off + lo * H * W * esz
                param._hm_grad_sources = [self.heap.view(r, slice_off, (st.n_local, H, W), self.dtype)
                                          for r in range(self.world)]
                param._hm_grad_scale = 1.0 / self.world
            setattr(model, b.spec.name, param)
            st.param = param
            st.sinks = [ops.GradSink(st.grad_full[i]) for i in range(n_pad)]
            # neighbouring slots (k|v, gate|up) viewed as one (2H, W) matrix for the fused pair GEMMs
            st.pair_sinks = {i: ops.GradSink(st.grad_full[i:i + 2].view(2 * H, W)) for i in range(0, n_pad - 1, 2)}
            self.state[b.spec.name] = st
            b.parameter = None            # the un-sharded original is released
        del bank_full
        if self.cuda:
            torch.cuda.empty_cache()
        object.__setattr__(model, "_bank_engine", self if self.banks is not None else None)
        self.materialize_grads = False    # True: produce .grad for bank shards (optimizers without the fused path)
        self._copy_table = None
        if self.world > 1:
            self.heap.barrier()

    def _padded(self, n: int) -> int:
        return -(-n // self._pad) * self._pad

    # ------------------------------------------------------------------ optimizer hookup
    def attach_optimizer(self, optimizer):
        """HiMuon reads the gradient replicas itself (fused reduce-scatter); any other optimizer gets a
        reduced ``.grad`` on the bank shards."""
        from ..optimizers import HiMuon
        self.materialize_grads = not (isinstance(optimizer, HiMuon) and self.cuda)
        if self.materialize_grads:
            for st in self.state.values():
                if hasattr(st.param, "_hm_grad_sources"):
                    del st.param._hm_grad_sources

    # ------------------------------------------------------------------ forward / backward plumbing
    def _weights(self, st: _BankState, idx: int, n: int) -> torch.Tensor:
        """Slots ``idx .. idx+n`` as an ``(n, H, W)`` tensor: the gathered copy, or the owner's shard seen through
        its peer mapping (only this package's own TMA GEMMs ever read that memory)."""
        if st.gathered is not None:
            return st.gathered[idx:idx + n]
        r, j = divmod(idx, st.n_local)
        return st.peer_shards[r][j:j + n]

    def linear(self, x, bank_name: str, idx: int, bias=None):
        st = self.state[bank_name]
        y = ops.linear(x, self._weights(st, idx, 1)[0], sink=st.sinks[idx])
        return y if bias is None else y + bias

    def linear_pair(self, x, bank_name: str, idx: int):
        """Slots ``idx`` and ``idx+1`` applied as one ``(2H, W)`` projection (one GEMM in each direction)."""
        st = self.state[bank_name]
        H, W = st.spec.matrix_shape
        return ops.linear(x, self._weights(st, idx, 2).view(2 * H, W), sink=st.pair_sinks[idx])

    @contextmanager
    def no_sync(self):
        yield

    def finish_backward(self):
        """Make every rank's accumulated gradients visible and reduce what the optimizer cannot reduce itself."""
        if self.world == 1:
            if self.materialize_grads:
                for st in self.state.values():
                    st.param.grad = st.grad_full
            return
        for flat, offset in self.regions:          # also orders this rank after every peer's backward
            self.heap.allreduce_(flat, offset, 1.0 / self.world)
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
                self.heap.comm.reduce_to(st.grad_off + lo * H * W * esz, st.param.grad, 1.0 / self.world)
                ops._count()
            else:
                work = st.grad_full.float()
                dist.all_reduce(work)
                st.param.grad.copy_(work[lo:lo + st.n_local] / self.world)

    def zero_grad(self, set_to_none: bool = False):
        """Runs after ``optimizer.step()``: refresh the gathered working copy and reset the accumulators."""
        if self.world > 1:
            self.heap.barrier()                    # every owner has finished updating its shards
            self._regather()
        for flat, _ in self.regions:
            flat.zero_()
        for st in self.state.values():
            for s in st.sinks:
                s.reset()
            for s in st.pair_sinks.values():
                s.reset()
            if self.materialize_grads and set_to_none and self.world > 1:
                st.param.grad = None

    def _regather(self):
        if not self.cuda:
            for st in self.state.values():
                dist.all_gather_into_tensor(st.gathered, st.shard.contiguous())
            return
        if all(st.gathered is None for st in self.state.values()):
            return                                   # every bank is read in place through the peer mappings
        if self._copy_table is None:
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
        """Full, un-banked state dict with the Hugging Face ``model.layers.{i}.*`` keys (every rank holds the
        gathered banks, so no communication is needed; the reference gathers to rank 0, ``train_fsdp.py:285-297``)."""
        sd = {}
        bank_names = set(self.state)
        for k, v in self.model.state_dict().items():
            if k not in bank_names:
                sd[k] = v.detach().cpu()
        if self.banks is None:
            return sd
        for name, st in self.state.items():
            if st.gathered is not None:
                sd[name] = st.gathered.detach().cpu()
            else:
                full = torch.empty(st.spec.n_padded, *st.spec.matrix_shape, device=self.device, dtype=self.dtype)
                dist.all_gather_into_tensor(full, st.shard.detach().contiguous())   # every rank sends its own shard
                sd[name] = full.cpu()
        return unbank_state_dict(sd, self.banks)

    def close(self):
        for p in self.model.parameters():
            p.grad = None
            if hasattr(p, "_hm_grad_sources"):
                del p._hm_grad_sources
        self.state = {}
        self.regions = []
        self._copy_table = None
        self.heap.close()
