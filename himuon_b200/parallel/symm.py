"""Symmetric memory: one device heap per rank, mapped into every rank of the node.

Each rank ``cudaMalloc``s a heap, publishes its CUDA IPC handle through ``torch.distributed`` and
opens the peers' handles, after which any rank can address any other rank's heap with ordinary
loads and stores over NVLink.  Every rank allocates the same sequence of regions, so a region is
identified by its byte offset and ``peer_view(r, ...)`` returns rank ``r``'s copy of it.

The first bytes of the heap hold the flag area used by the kernels' bounded-wait handshakes.
On CPU (gloo) runs the heap is ordinary host memory and the collectives fall back to
``torch.distributed`` calls, which keeps the engines' host-side logic testable without a GPU.
The reference has no counterpart: it delegates all communication to NCCL through DDP / FSDP2.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_DT = {torch.bfloat16: "bf16", torch.float32: "f32", torch.int32: "i32", torch.uint8: "u8", torch.int64: "i64"}
_ALIGN = 1024


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class SymmetricHeap:
    def __init__(self, nbytes: int, device: torch.device, timeout_s: float = 120.0):
        self.rank, self.world = _world()
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
            self.comm = self._ext.Comm(self.rank, self.world, self.ptrs, float(timeout_s))
            self.cursor = self.flag_bytes
            if self.world > 1:
                dist.barrier()
        else:
            self.flag_bytes = 0
            self.nbytes = -(-int(nbytes) // _ALIGN) * _ALIGN + _ALIGN
            self._host = torch.zeros(self.nbytes, dtype=torch.uint8)

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape, dtype) -> tuple[torch.Tensor, int]:
        """Reserve a region (same call sequence on every rank); returns the local tensor and its offset."""
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        offset = -(-self.cursor // _ALIGN) * _ALIGN
        if offset + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {offset + nbytes} bytes, have {self.nbytes}")
        self.cursor = offset + nbytes
        return self.view(self.rank, offset, shape, dtype), offset

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
    def barrier(self):
        if self.world == 1:
            return
        if self.cuda:
            self.comm.barrier()
        else:
            dist.barrier()

    def allreduce_(self, tensor: torch.Tensor, offset: int, scale: float, max_blocks: int = 0, algo: int = 0):
        """In-place sum over ranks of the region ``tensor`` (at ``offset``) times ``scale``.  ``algo``: 0 picks the
        one-shot kernel up to 256 KiB and the two-shot kernel above, 1 / 2 force one of them; ``max_blocks`` caps the
        two-shot grid (a small grid leaves the SMs to a compute stream that runs beside it)."""
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
            for p in self._opened:
                self._ext.symm_close(p)
            self._opened = []
            if self._own_ptr:
                self._ext.symm_free(self._own_ptr)
                self._own_ptr = 0
