"""Symmetric memory: one device heap per rank, mapped into every rank of the node.

Each rank ``cudaMalloc``s a heap, publishes its CUDA IPC handle through ``torch.distributed`` and
opens the peers' handles, after which any rank can address any other rank's heap with ordinary
loads and stores over NVLink.  Every rank allocates the same sequence of regions, so a region is
identified by its byte offset and ``peer_view(r, ...)`` returns rank ``r``'s copy of it.

With ``multicast=True`` the heap is created with the CUDA virtual-memory API instead (``csrc/vmm.cpp``) and every
rank's memory is also bound to one NVLink multicast object: ``multimem`` loads through the multicast address are
reduced inside the NVLink switch and ``multimem`` stores are replicated by it (NVLS), which the all-reduce
(``algo=3``) and ``reduce_to(multicast=True)`` kernels use.  Where the device or the setup does not support it the
heap falls back to the IPC kind on every rank together.  A rank must not exit while its memory is bound to the
multicast object and peers may still touch it: ``close()`` synchronises, meets the other ranks at a barrier and only
then unbinds and unmaps.

The first bytes of the heap hold the flag area used by the kernels' bounded-wait handshakes.
On CPU (gloo) runs the heap is ordinary host memory and the collectives fall back to
``torch.distributed`` calls, which keeps the engines' host-side logic testable without a GPU.
The reference has no counterpart: it delegates all communication to NCCL through DDP / FSDP2.
"""

from __future__ import annotations

import os
import warnings

import torch
import torch.distributed as dist

_DT = {torch.bfloat16: "bf16", torch.float32: "f32", torch.int32: "i32", torch.uint8: "u8", torch.int64: "i64"}
_ALIGN = 1024


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class SymmetricHeap:
    CANARY_BYTES = 1024
    CANARY_VALUE = 0xA5

    def __init__(self, nbytes: int, device: torch.device, timeout_s: float = 120.0, multicast: bool = False,
                 canaries: bool = False):
        """``canaries``: debugging aid against out-of-bounds writes by the kernels that address the heap through raw
        pointers (there is no memory checker to lean on): every region gets a guard zone filled with a byte pattern
        after it, and ``check_canaries()`` reports any zone that no longer holds the pattern.  Every rank must pass
        the same value (the regions' offsets have to agree)."""
        self.rank, self.world = _world()
        self.canaries = bool(canaries)
        self._guards: list[int] = []
        self.has_multicast = False
        self._vmm = False
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.cursor = 0
        self.comm = None
        self._ext = None
        self._opened: list[int] = []
        self._own_ptr = 0
        if self.cuda:
            from .._ext import ext
            self._ext = ext()
            flag_bytes = int(self._ext.Comm.flag_bytes())
            self.flag_bytes = -(-flag_bytes // _ALIGN) * _ALIGN
            self.nbytes = self.flag_bytes + -(-int(nbytes) // _ALIGN) * _ALIGN + _ALIGN
            torch.cuda.set_device(self.device)
            mc_ptr = 0
            if multicast and self.world > 1:
                mc_ptr = self._setup_multicast()
            if not self._vmm:
                ptr, handle = self._ext.symm_alloc(self.nbytes)
                self._own_ptr = ptr
                self.ptrs = [ptr]
                if self.world > 1:
                    handles = [None] * self.world
                    dist.all_gather_object(handles, handle)
                    self.ptrs = []
                    for r, h in enumerate(handles):
                        if r == self.rank:
                            self.ptrs.append(ptr)
                        else:
                            p = self._ext.symm_open(h)
                            self._opened.append(p)
                            self.ptrs.append(p)
            self.comm = self._ext.Comm(self.rank, self.world, self.ptrs, float(timeout_s), int(mc_ptr))
            self.cursor = self.flag_bytes
            if self.world > 1:
                dist.barrier()
        else:
            self.flag_bytes = 0
            self.nbytes = -(-int(nbytes) // _ALIGN) * _ALIGN + _ALIGN
            self._host = torch.zeros(self.nbytes, dtype=torch.uint8)

    # ------------------------------------------------------------------ NVLS setup
    def _setup_multicast(self) -> int:
        """cuMemCreate'd heap, peers mapped through exchanged descriptors, everything bound to one multicast object.
        Returns the multicast address, or 0 after falling back (all ranks take the same decision)."""
        e, dev = self._ext, self.device.index or 0
        ok = bool(e.vmm_multicast_supported(dev))
        votes = [None] * self.world
        dist.all_gather_object(votes, ok)
        if not all(votes):
            if self.rank == 0:
                warnings.warn("SymmetricHeap: NVLink multicast is not supported here; using the IPC heap")
            return 0
        # Stages end with a vote so that a failure on one rank makes every rank fall back at the same point instead of
        # leaving the others waiting in a collective.
        st: dict = {}

        def vote(stage_fn) -> bool:
            err = None
            try:
                stage_fn()
            except Exception as ex:              # noqa: BLE001 - any failure means: fall back, on every rank
                err = f"{type(ex).__name__}: {ex}"
            errs = [None] * self.world
            dist.all_gather_object(errs, err)
            bad = [x for x in errs if x is not None]
            if bad:
                st["error"] = bad[0]
            return not bad

        def stage_alloc():
            st["size"] = int(e.vmm_round_size(self.nbytes, dev, self.world))
            st["idx"], st["ptr"], st["fd"] = e.vmm_alloc(st["size"], dev)

        def stage_import():
            infos = [None] * self.world
            dist.all_gather_object(infos, (os.getpid(), int(st["fd"])))
            st["ptrs"] = [st["ptr"] if r == self.rank else int(e.vmm_import(pid, rfd, st["size"], dev))
                          for r, (pid, rfd) in enumerate(infos)]

        def stage_mc_create():
            if self.rank == 0:
                st["mc"], st["mc_fd"] = e.mc_create(self.world, st["size"], dev)

        def stage_mc_import():
            box = [(os.getpid(), int(st["mc_fd"]))] if self.rank == 0 else [None]
            dist.broadcast_object_list(box, src=0)
            if self.rank != 0:
                st["mc"] = e.mc_import(box[0][0], box[0][1], st["size"], dev)
            e.mc_add_device(st["mc"], dev)

        def stage_bind():                        # runs after every device has been added (the vote is the barrier)
            e.mc_bind(st["mc"], st["idx"])

        def stage_map():                         # runs after every rank's memory has been bound
            st["mc_ptr"] = int(e.mc_map(st["mc"]))

        ok = all(vote(f) for f in (stage_alloc, stage_import, stage_mc_create, stage_mc_import, stage_bind, stage_map))
        if not ok:
            torch.cuda.synchronize(self.device)
            dist.barrier()
            e.vmm_release_all()
            if self.rank == 0:
                warnings.warn(f"SymmetricHeap: multicast setup failed ({st.get('error')}); using the IPC heap")
            return 0
        size, ptrs, mc_ptr = st["size"], st["ptrs"], st["mc_ptr"]
        self.nbytes = size
        self.ptrs = ptrs
        self._own_ptr = 0
        self._vmm = True
        self.has_multicast = True
        return mc_ptr

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape, dtype) -> tuple[torch.Tensor, int]:
        """Reserve a region (same call sequence on every rank); returns the local tensor and its offset."""
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        offset = -(-self.cursor // _ALIGN) * _ALIGN
        guard = self.CANARY_BYTES if self.canaries else 0
        if offset + nbytes + guard > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {offset + nbytes + guard} bytes, have {self.nbytes}")
        self.cursor = offset + nbytes + guard
        if guard:
            self.view(self.rank, offset + nbytes, (guard,), torch.uint8).fill_(self.CANARY_VALUE)
            self._guards.append(offset + nbytes)
        return self.view(self.rank, offset, shape, dtype), offset

    def check_canaries(self) -> list[int]:
        """Offsets of the guard zones on this rank that were overwritten (empty when all are intact or canaries are
        off).  Synchronises with the device."""
        bad = []
        for off in self._guards:
            zone = self.view(self.rank, off, (self.CANARY_BYTES,), torch.uint8)
            if not bool((zone == self.CANARY_VALUE).all()):
                bad.append(off)
        return bad

    def view(self, rank: int, offset: int, shape, dtype) -> torch.Tensor:
        """Rank ``rank``'s copy of the region at ``offset`` as a tensor on this device."""
        shape = [int(s) for s in shape]
        if self.cuda:
            return self._ext.tensor_view(self.ptrs[rank] + offset, shape, _DT[dtype], self.device.index or 0)
        if rank != self.rank:
            raise RuntimeError("peer views need CUDA peer mappings; CPU runs use the torch.distributed fallbacks")
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self._host[offset:offset + nbytes].view(dtype).view(shape)

    # ------------------------------------------------------------------ collectives
    def barrier(self, channel: int = 0):
        """Stream-ordered barrier between the ranks' GPUs on the current stream.  ``channel=1`` is a second, independent
        barrier (own flags and counters) for a side stream: calls on one channel must come in the same order on every
        rank, calls on different channels may interleave differently from rank to rank."""
        if self.world == 1:
            return
        if self.cuda:
            self.comm.barrier(channel)
        else:
            dist.barrier()

    def allreduce_(self, tensor: torch.Tensor, offset: int, scale: float, max_blocks: int = 0, algo: int = 0):
        """In-place sum over ranks of the region ``tensor`` (at ``offset``) times ``scale``.  ``algo``: 0 and 2 run the
        two-shot kernel, 1 the one-shot kernel (regions up to 2 MiB; measured no faster than two-shot at any size, so
        never chosen automatically), 3 reduces and broadcasts through the NVLink switch (needs a multicast heap); ``max_blocks`` caps the two-shot grid (a small grid
        leaves the SMs to a compute stream that runs beside it)."""
        if self.world == 1:
            if scale != 1.0:
                tensor.mul_(scale)
            return
        if self.cuda:
            from ..ops import _count
            self.comm.allreduce(offset, tensor.numel(), tensor.dtype == torch.float32, float(scale), int(max_blocks),
                                int(algo))
            _count()
        else:
            work = tensor.float() if tensor.dtype == torch.bfloat16 else tensor
            dist.all_reduce(work)
            tensor.copy_(work * scale)

    def set_timeout(self, seconds: float):
        if self.comm is not None:
            self.comm.set_timeout(float(seconds))

    def close(self):
        if self.cuda and self._ext is not None:
            torch.cuda.synchronize(self.device)
            if self.world > 1 and dist.is_initialized():
                dist.barrier()
            self.comm = None
            if self._vmm:
                # all ranks are idle and past the barrier: nobody touches the multicast object any more
                self._ext.vmm_release_all()
                self._vmm = self.has_multicast = False
                if self.world > 1 and dist.is_initialized():
                    dist.barrier()
            for p in self._opened:
                self._ext.symm_close(p)
            self._opened = []
            if self._own_ptr:
                self._ext.symm_free(self._own_ptr)
                self._own_ptr = 0
