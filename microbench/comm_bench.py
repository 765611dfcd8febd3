"""Collective microbenchmark over the symmetric heap (run under torchrun, one rank per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29555 \
        -m microbench.comm_bench [--max-mb 1024] [--nccl] [--json out.json]

Times, with CUDA events on the launching stream after a barrier (maximum over ranks, median of ``--iters`` launches
after ``--warmup``), the kernels the engines use for their bulk traffic:

* ``allreduce`` - the fused two-shot all-reduce on region sizes from 64 KiB to
  ``--max-mb`` and on the gradient sizes of Qwen3-0.6B (data-parallel configuration);
* ``allreduce_16blk`` - the same with the 16-block grid the data-parallel engine uses beside the backward GEMMs;
* ``bank_gather`` - ``multi_copy`` pulling every peer's bank shard (the once-per-step re-gather of the gathered mode);
* ``ring_fetch`` - the copy-engine fetch of one layer group into a staging slot (owners visited in rotated order);
* ``reduce_scatter`` - ``reduce_replicas`` summing the ranks' copies of this rank's slice (the owner-side half of a
  reduce-scatter; the same loads happen inside ``momentum_tile`` for HiMuon);
* with ``--nccl`` the NCCL calls a stock PyTorch stack would issue for the same job (``all_reduce``,
  ``all_gather_into_tensor``, ``reduce_scatter_tensor``) for comparison.

Reported per line: milliseconds, algorithm bandwidth (payload / time), bus bandwidth (bytes each GPU must move over its
NVLink ports / time) and that as a fraction of the measured 770 GB/s per direction peer-copy rate of this pool.
Between timed launches of the small sizes a buffer larger than the L2 is rewritten so that no launch finds its data cached.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

LINK_GBS = 770.0      # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1.0)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
    return statistics.median(times)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--nvls", action="store_true", help="bind the heap to an NVLink multicast object and also time the "
                    "multimem variants (all-reduce through the switch, switch-side reduce)")
    ap.add_argument("--json", type=str, default=None)
    args = ap.parse_args()

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=device)
    rank, world = dist.get_rank(), dist.get_world_size()

    from himuon_b200 import ops
    from himuon_b200.parallel.symm import SymmetricHeap

    max_bytes = args.max_mb << 20
    heap = SymmetricHeap(2 * max_bytes + (64 << 20), device, timeout_s=30.0, multicast=args.nvls)
    if args.nvls and rank == 0:
        print(f"# multicast heap: {heap.has_multicast}", flush=True)
    flush = torch.zeros(160 << 20, device=device, dtype=torch.float32)      # 640 MB > 126 MB L2
    rows = []

    def report(name, nbytes, ms, bus_bytes):
        alg = nbytes / ms / 1e6
        bus = bus_bytes / ms / 1e6
        rows.append({"op": name, "bytes": nbytes, "ms": ms, "alg_GBs": alg, "bus_GBs": bus, "frac_of_link": bus / LINK_GBS,
                     "n_gpus": world})
        if rank == 0:
            print(f"{name:28s} {nbytes / 2**20:10.2f} MiB  {ms:9.4f} ms  alg {alg:8.1f} GB/s  bus {bus:8.1f} GB/s "
                  f"({bus / LINK_GBS:5.2f} of {LINK_GBS:.0f})", flush=True)

    unit = 16 * world
    buf, off = heap.alloc((max_bytes // 2,), torch.bfloat16)
    buf.normal_()
    sizes = [64 << 10, 256 << 10, 1 << 20, 16 << 20, 64 << 20, 256 << 20, 1 << 30]
    sizes = [s for s in sizes if s <= max_bytes]
    qwen06 = 596_049_920 * 2            # Qwen3-0.6B trainable parameters (tied embeddings) in bf16
    if qwen06 <= max_bytes:
        sizes.append(qwen06)
    ar_factor = 2.0 * (world - 1) / world
    for nbytes in sizes:
        n = (nbytes // 2) // unit * unit
        fl = flush if nbytes <= (256 << 20) else None
        ms = _time(lambda: heap.allreduce_(buf[:n], off, 1.0 / world), args.iters, args.warmup, fl)
        report("allreduce", n * 2, ms, ar_factor * n * 2)
        if nbytes >= (16 << 20):
            ms = _time(lambda: heap.allreduce_(buf[:n], off, 1.0 / world, max_blocks=16), args.iters, args.warmup, fl)
            report("allreduce_16blk", n * 2, ms, ar_factor * n * 2)
        if nbytes <= (1 << 20):
            ms = _time(lambda: heap.allreduce_(buf[:n], off, 1.0 / world, algo=1), args.iters, args.warmup, fl)
            report("allreduce_oneshot", n * 2, ms, ar_factor * n * 2)
        if heap.has_multicast and nbytes >= (1 << 20):
            ms = _time(lambda: heap.allreduce_(buf[:n], off, 1.0 / world, algo=3), args.iters, args.warmup, fl)
            report("allreduce_nvls", n * 2, ms, ar_factor * n * 2)
        if args.nccl:
            t = buf[:n]
            ms = _time(lambda: dist.all_reduce(t), args.iters, args.warmup, fl)
            report("nccl_all_reduce", n * 2, ms, ar_factor * n * 2)

    # ---- all-gather of bank shards (multi_copy) and the copy-engine ring fetch
    import struct
    ext = heap._ext
    shard_bytes = min(max_bytes // world, 512 << 20) // 4096 * 4096
    shard, soff = heap.alloc((shard_bytes // 2,), torch.bfloat16)
    shard.normal_()
    gathered = torch.empty(world, shard_bytes // 2, device=device, dtype=torch.bfloat16)
    tab, units = bytearray(), 0
    for r in range(world):
        src = heap.view(r, soff, (shard_bytes // 2,), torch.bfloat16)
        tab += struct.pack("<QQqq", src.data_ptr(), gathered[r].data_ptr(), shard_bytes, units)
        units += int(ext.multi_copy_units(shard_bytes))
    tab_dev = torch.frombuffer(tab, dtype=torch.uint8).to(device)
    heap.barrier()
    ms = _time(lambda: heap.comm.copy_segments(tab_dev, world, units, 0), args.iters, args.warmup, None)
    report("bank_gather(multi_copy)", shard_bytes * world, ms, shard_bytes * (world - 1))
    if args.nccl:
        flat = gathered.view(-1)
        ms = _time(lambda: dist.all_gather_into_tensor(flat, shard), args.iters, args.warmup, None)
        report("nccl_all_gather", shard_bytes * world, ms, shard_bytes * (world - 1))
    peers = [heap.view(r, soff, (shard_bytes // 2,), torch.bfloat16) for r in range(world)]

    def ring_fetch():
        for j in range(1, world):
            o = (rank + j) % world
            gathered[o].copy_(peers[o], non_blocking=True)

    ms = _time(ring_fetch, args.iters, args.warmup, None)
    report("ring_fetch(copy engines)", shard_bytes * (world - 1), ms, shard_bytes * (world - 1))

    # ---- owner-side reduce (reduce-scatter half)
    out = torch.empty(shard_bytes // 2, device=device, dtype=torch.bfloat16)
    ms = _time(lambda: heap.comm.reduce_to(soff, out, 1.0 / world, 0.0), args.iters, args.warmup, None)
    report("reduce_scatter(reduce_to)", shard_bytes * world, ms, shard_bytes * (world - 1))
    if heap.has_multicast:
        # the switch sums the copies: this rank receives one copy's worth of bytes, but every GPU still sends its
        # copy of the other ranks' slices, so the outgoing direction carries what the plain reduce-scatter carries
        ms = _time(lambda: heap.comm.reduce_to(soff, out, 1.0 / world, 0.0, True), args.iters, args.warmup, None)
        report("reduce_scatter_nvls", shard_bytes * world, ms, shard_bytes * (world - 1))
    if args.nccl:
        full = gathered.view(-1)
        ms = _time(lambda: dist.reduce_scatter_tensor(out, full), args.iters, args.warmup, None)
        report("nccl_reduce_scatter", shard_bytes * world, ms, shard_bytes * (world - 1))

    torch.cuda.synchronize()
    ops.check_status()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
