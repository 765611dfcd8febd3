// Collectives over peer-mapped (symmetric) memory on NVLink 5 / NVSwitch: plain peer loads and
// stores, per-block flag handshakes with bounded waits, no NCCL and no multicast loads.
//
//   peer_barrier     : stream-ordered barrier between the ranks' GPUs (one tiny launch)
//   allreduce_symm   : one-launch all-reduce with the average / cast fused: two-shot (reduce-scatter by
//                      peer loads, all-gather by peer stores); a one-shot variant (every rank reads
//                      everything, no peer stores) exists for regions up to 2 MiB and is selected by hand;
//                      replaces the DDP reducer's bucketed NCCL all-reduce (reference:
//                      train_ddp.py:90, implicit)
//   reduce_replicas  : out = beta * out + scale * sum_r replica_r, the owner-side half of a
//                      reduce-scatter: for optimizers that need a plain `.grad` (HiMuon fuses this
//                      step into momentum_tile instead), and for the per-layer-group gradient
//                      reduce-scatter of the sharded-gradient mode (beta = 1 accumulates micro-batches)
//   multi_copy       : one launch that pulls many (peer -> local) segments; the bank all-gather
//
// Every wait on a peer flag is bounded: on expiry the kernel records status 6 and returns, so a
// missing rank surfaces as an error on the host instead of a hung GPU.
#include "himuon.h"
#include "sm100_common.cuh"

namespace himuon {

__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until *flag >= target.  Returns false after `limit_ns` (status code 6 recorded).
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int target, unsigned long long limit_ns, int* status) {
  if (ld_acquire_sys(flag) >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys(flag) < target) {
    if ((++spins & 0x3F) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, 0, 6);
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}

// Handshake of block `slot` with the same block index on every peer.
//   flags[r]  : rank r's flag array (peer-mapped); entry [slot*8 + src] is written by rank `src`
//   epoch     : this rank's private counter for `slot`, advanced here (graph-replay safe)
__device__ __forceinline__ bool block_handshake(CommPeers peers, int slot, int* epoch_local, int which, bool* ok_shared) {
  __syncthreads();
  if (threadIdx.x == 0) {
    // One system-scope fence publishes everything this block (and, through the barrier above, its threads) wrote;
    // the flag stores that follow it can then be relaxed - a release per peer would repeat the fence world times.
    __threadfence_system();
    const int e = ++epoch_local[slot * 2 + which];
    bool ok = true;
    for (int r = 0; r < peers.world; ++r)
      st_relaxed_sys(peers.flags[r] + (which * kCommMaxBlocks + slot) * 8 + peers.rank, e);
    for (int r = 0; r < peers.world && ok; ++r)
      ok = wait_flag_ge(peers.flags[peers.rank] + (which * kCommMaxBlocks + slot) * 8 + r, e, peers.limit_ns, peers.status);
    *ok_shared = ok;
  }
  __syncthreads();
  return *ok_shared;
}

// The barrier owns the last block slot (no collective's grid reaches it).  Its two phases are two independent
// channels with their own flags and epoch counters: channel 0 for barriers on the stream that also runs the other
// collectives, channel 1 for barriers on a side stream whose order against channel 0 differs from rank to rank.
__global__ void peer_barrier_kernel(CommPeers peers, int* epoch_local, int channel) {
  __shared__ bool ok;
  block_handshake(peers, kCommMaxBlocks - 1, epoch_local, channel, &ok);
}

void peer_barrier(const CommPeers& peers, int* epoch_local, cudaStream_t s, int channel) {
  if (peers.world <= 1) return;
  peer_barrier_kernel<<<1, 32, 0, s>>>(peers, epoch_local, channel & 1);
}

// ------------------------------------------------------------------------------------------------ all-reduce
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_symm_kernel(CommPeers peers, CommBufs bufs, long long n_elems, float scale, int* epoch_local) {
  __shared__ bool ok;
  constexpr int VEC = 16 / sizeof(T);
  const int world = peers.world, rank = peers.rank;
  if (!block_handshake(peers, blockIdx.x, epoch_local, 0, &ok)) return;
  const long long n_vec = n_elems / VEC;                       // n_elems is padded to VEC * world by the caller
  const long long per_rank = n_vec / world;
  const long long v0 = per_rank * rank;
  for (long long v = v0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < v0 + per_rank;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int r = 0; r < world; ++r) {
      const uint4 x = reinterpret_cast<const uint4*>(bufs.ptr[r])[v];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      if (sizeof(T) == 2) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { acc[2 * q] += bf16_lo(w[q]); acc[2 * q + 1] += bf16_hi(w[q]); }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += __uint_as_float(w[q]);
      }
    }
    uint4 o;
    if (sizeof(T) == 2) {
      o.x = pack_bf16x2(acc[0] * scale, acc[1] * scale); o.y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
      o.z = pack_bf16x2(acc[4] * scale, acc[5] * scale); o.w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
    } else {
      o.x = __float_as_uint(acc[0] * scale); o.y = __float_as_uint(acc[1] * scale);
      o.z = __float_as_uint(acc[2] * scale); o.w = __float_as_uint(acc[3] * scale);
    }
    for (int r = 0; r < world; ++r) reinterpret_cast<uint4*>(bufs.ptr[(rank + r) % world])[v] = o;
  }
  block_handshake(peers, blockIdx.x, epoch_local, 1, &ok);
}

// One-shot variant for small, latency-bound regions: every rank reads the whole region from all ranks and keeps the
// sums in registers, a second handshake tells it that the peers have finished reading its copy, then it writes its
// own copy.  No peer stores, and no rank waits for data to arrive from another one.
constexpr int kOneShotVecPerThread = 4;
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(CommPeers peers, CommBufs bufs, long long n_elems, float scale, int* epoch_local) {
  __shared__ bool ok;
  constexpr int VEC = 16 / sizeof(T);
  const int world = peers.world, rank = peers.rank;
  if (!block_handshake(peers, blockIdx.x, epoch_local, 0, &ok)) return;
  const long long n_vec = n_elems / VEC;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long v0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  uint4 res[kOneShotVecPerThread];
#pragma unroll
  for (int k = 0; k < kOneShotVecPerThread; ++k) {
    const long long v = v0 + k * stride;
    if (v >= n_vec) break;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int r = 0; r < world; ++r) {
      const uint4 x = reinterpret_cast<const uint4*>(bufs.ptr[(rank + r) % world])[v];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      if (sizeof(T) == 2) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { acc[2 * q] += bf16_lo(w[q]); acc[2 * q + 1] += bf16_hi(w[q]); }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += __uint_as_float(w[q]);
      }
    }
    if (sizeof(T) == 2) {
      res[k].x = pack_bf16x2(acc[0] * scale, acc[1] * scale); res[k].y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
      res[k].z = pack_bf16x2(acc[4] * scale, acc[5] * scale); res[k].w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
    } else {
      res[k].x = __float_as_uint(acc[0] * scale); res[k].y = __float_as_uint(acc[1] * scale);
      res[k].z = __float_as_uint(acc[2] * scale); res[k].w = __float_as_uint(acc[3] * scale);
    }
  }
  if (!block_handshake(peers, blockIdx.x, epoch_local, 1, &ok)) return;   // every rank has read this block's vectors
#pragma unroll
  for (int k = 0; k < kOneShotVecPerThread; ++k) {
    const long long v = v0 + k * stride;
    if (v >= n_vec) break;
    reinterpret_cast<uint4*>(bufs.ptr[rank])[v] = res[k];
  }
}

// Largest region (bytes) the one-shot kernel takes: 64 blocks x 512 threads x 4 vectors of 16 bytes.
constexpr long long kOneShotMaxBytes = 64LL * 512 * kOneShotVecPerThread * 16;

void allreduce_symm(const CommPeers& peers, const CommBufs& bufs, long long n_elems, int is_fp32, float scale,
                    int* epoch_local, int max_blocks, cudaStream_t s, int algo) {
  if (n_elems <= 0) return;
  const int vec = is_fp32 ? 4 : 8;
  if (n_elems % (static_cast<long long>(vec) * peers.world))
    throw std::runtime_error("himuon allreduce: element count must be a multiple of (16 bytes * world size)");
  // algo 0 and 2: two-shot, 1: one-shot.  The one-shot kernel is never picked automatically: with its two handshakes
  // it measured no faster than the two-shot kernel even at 64 KiB (0.035 vs 0.032 ms on 2 ranks, 0.053 vs 0.039 ms
  // on 4), because every rank then reads `world` copies where the two-shot kernel reads and writes one.
  const long long bytes = n_elems * (is_fp32 ? 4 : 2);
  if (algo == 1 && bytes > kOneShotMaxBytes)
    throw std::runtime_error("himuon allreduce: region too large for the one-shot kernel");
  if (algo == 1) {
    const long long n_vec = n_elems / vec;
    long long blocks = (n_vec + 512LL * kOneShotVecPerThread - 1) / (512LL * kOneShotVecPerThread);
    if (blocks < 1) blocks = 1;                       // by the size limit above, blocks <= 64 < kCommMaxBlocks
    if (is_fp32)
      allreduce_oneshot_kernel<float><<<static_cast<int>(blocks), 512, 0, s>>>(peers, bufs, n_elems, scale, epoch_local);
    else
      allreduce_oneshot_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 512, 0, s>>>(peers, bufs, n_elems, scale, epoch_local);
    return;
  }
  const long long per_rank_vec = n_elems / vec / peers.world;
  long long blocks = (per_rank_vec + 511) / 512;
  const int cap = max_blocks > 0 ? max_blocks : num_sms();
  if (blocks > cap) blocks = cap;
  if (blocks > kCommMaxBlocks - 1) blocks = kCommMaxBlocks - 1;
  if (blocks < 1) blocks = 1;
  if (is_fp32)
    allreduce_symm_kernel<float><<<static_cast<int>(blocks), 512, 0, s>>>(peers, bufs, n_elems, scale, epoch_local);
  else
    allreduce_symm_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 512, 0, s>>>(peers, bufs, n_elems, scale, epoch_local);
}

// ------------------------------------------------------------------------------------------------ NVLS (multimem)
// `mc` is the multicast address of the same region on every rank (memory created by cuMemCreate and bound to one
// multicast object, see vmm.cpp).  A multimem.ld_reduce through it makes the NVLink switch read every rank's copy and
// return the sum, so the reducing rank receives one copy's worth of bytes instead of world-1; a multimem.st makes the
// switch write every rank's copy, so the broadcasting rank sends each byte once.
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce_add(const void* mc_addr) {
  uint4 r;
  if (sizeof(T) == 2)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               :: "l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
template <typename T>
__device__ __forceinline__ uint4 scale_vec(const uint4& x, float scale) {
  uint4 o;
  if (sizeof(T) == 2) {
    o.x = pack_bf16x2(bf16_lo(x.x) * scale, bf16_hi(x.x) * scale); o.y = pack_bf16x2(bf16_lo(x.y) * scale, bf16_hi(x.y) * scale);
    o.z = pack_bf16x2(bf16_lo(x.z) * scale, bf16_hi(x.z) * scale); o.w = pack_bf16x2(bf16_lo(x.w) * scale, bf16_hi(x.w) * scale);
  } else {
    o.x = __float_as_uint(__uint_as_float(x.x) * scale); o.y = __float_as_uint(__uint_as_float(x.y) * scale);
    o.z = __float_as_uint(__uint_as_float(x.z) * scale); o.w = __float_as_uint(__uint_as_float(x.w) * scale);
  }
  return o;
}

// Two-shot all-reduce through the switch: each rank reduces its 1/world slice with multimem.ld_reduce and writes the
// result to every rank with multimem.st.  Same handshakes as the peer-pointer kernel.
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_nvls_kernel(CommPeers peers, char* mc, long long n_elems, float scale, int* epoch_local) {
  __shared__ bool ok;
  constexpr int VEC = 16 / sizeof(T);
  if (!block_handshake(peers, blockIdx.x, epoch_local, 0, &ok)) return;
  const long long n_vec = n_elems / VEC;
  const long long per_rank = n_vec / peers.world;
  const long long v0 = per_rank * peers.rank;
  for (long long v = v0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < v0 + per_rank;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 sum = multimem_ld_reduce_add<T>(mc + v * 16);
    multimem_st_v4(mc + v * 16, scale_vec<T>(sum, scale));
  }
  block_handshake(peers, blockIdx.x, epoch_local, 1, &ok);
}

void allreduce_nvls(const CommPeers& peers, void* mc_region, long long n_elems, int is_fp32, float scale, int* epoch_local,
                    int max_blocks, cudaStream_t s) {
  if (n_elems <= 0) return;
  const int vec = is_fp32 ? 4 : 8;
  if (n_elems % (static_cast<long long>(vec) * peers.world))
    throw std::runtime_error("himuon allreduce: element count must be a multiple of (16 bytes * world size)");
  const long long per_rank_vec = n_elems / vec / peers.world;
  long long blocks = (per_rank_vec + 511) / 512;
  const int cap = max_blocks > 0 ? max_blocks : num_sms();
  if (blocks > cap) blocks = cap;
  if (blocks > kCommMaxBlocks - 1) blocks = kCommMaxBlocks - 1;
  if (blocks < 1) blocks = 1;
  if (is_fp32)
    allreduce_nvls_kernel<float><<<static_cast<int>(blocks), 512, 0, s>>>(peers, static_cast<char*>(mc_region), n_elems, scale, epoch_local);
  else
    allreduce_nvls_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 512, 0, s>>>(peers, static_cast<char*>(mc_region), n_elems, scale, epoch_local);
}

// out = beta * out + scale * (sum over ranks of the region behind `mc`), the sum taken by the switch.  The caller
// orders this after the ranks' writes (a barrier) exactly as for reduce_replicas.
template <typename T>
__global__ void __launch_bounds__(512)
reduce_nvls_kernel(const char* mc, T* __restrict__ out, long long n_elems, float scale, float beta) {
  constexpr int VEC = 16 / sizeof(T);
  const long long n_vec = n_elems / VEC;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < n_vec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 o = scale_vec<T>(multimem_ld_reduce_add<T>(mc + v * 16), scale);
    if (beta != 0.f) {
      const uint4 x = scale_vec<T>(reinterpret_cast<const uint4*>(out)[v], beta);
      if (sizeof(T) == 2) {
        o.x = pack_bf16x2(bf16_lo(o.x) + bf16_lo(x.x), bf16_hi(o.x) + bf16_hi(x.x)); o.y = pack_bf16x2(bf16_lo(o.y) + bf16_lo(x.y), bf16_hi(o.y) + bf16_hi(x.y));
        o.z = pack_bf16x2(bf16_lo(o.z) + bf16_lo(x.z), bf16_hi(o.z) + bf16_hi(x.z)); o.w = pack_bf16x2(bf16_lo(o.w) + bf16_lo(x.w), bf16_hi(o.w) + bf16_hi(x.w));
      } else {
        o.x = __float_as_uint(__uint_as_float(o.x) + __uint_as_float(x.x)); o.y = __float_as_uint(__uint_as_float(o.y) + __uint_as_float(x.y));
        o.z = __float_as_uint(__uint_as_float(o.z) + __uint_as_float(x.z)); o.w = __float_as_uint(__uint_as_float(o.w) + __uint_as_float(x.w));
      }
    }
    reinterpret_cast<uint4*>(out)[v] = o;
  }
}

void reduce_nvls(const void* mc_region, void* out, long long n_elems, int is_fp32, float scale, float beta, cudaStream_t s) {
  if (n_elems <= 0) return;
  const int vec = is_fp32 ? 4 : 8;
  if (n_elems % vec) throw std::runtime_error("himuon reduce_nvls: element count must be a multiple of 16 bytes");
  long long blocks = (n_elems / vec + 511) / 512;
  const long long cap = static_cast<long long>(num_sms()) * 2;
  if (blocks > cap) blocks = cap;
  if (is_fp32)
    reduce_nvls_kernel<float><<<static_cast<int>(blocks), 512, 0, s>>>(static_cast<const char*>(mc_region), static_cast<float*>(out), n_elems, scale, beta);
  else
    reduce_nvls_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 512, 0, s>>>(static_cast<const char*>(mc_region), static_cast<__nv_bfloat16*>(out), n_elems, scale, beta);
}

// ------------------------------------------------------------------------------------------------ reduce replicas
template <typename T>
__global__ void __launch_bounds__(512)
reduce_replicas_kernel(CommBufs srcs, int n_src, T* __restrict__ out, long long n_elems, float scale, float beta) {
  constexpr int VEC = 16 / sizeof(T);
  const long long n_vec = n_elems / VEC;
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < n_vec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int r = 0; r < n_src; ++r) {
      const uint4 x = reinterpret_cast<const uint4*>(srcs.ptr[r])[v];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      if (sizeof(T) == 2) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { acc[2 * q] += bf16_lo(w[q]); acc[2 * q + 1] += bf16_hi(w[q]); }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += __uint_as_float(w[q]);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= scale;
    if (beta != 0.f) {                                   // accumulate onto what `out` already holds
      const uint4 x = reinterpret_cast<const uint4*>(out)[v];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
      if (sizeof(T) == 2) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { acc[2 * q] += beta * bf16_lo(w[q]); acc[2 * q + 1] += beta * bf16_hi(w[q]); }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += beta * __uint_as_float(w[q]);
      }
    }
    uint4 o;
    if (sizeof(T) == 2) {
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    } else {
      o.x = __float_as_uint(acc[0]); o.y = __float_as_uint(acc[1]);
      o.z = __float_as_uint(acc[2]); o.w = __float_as_uint(acc[3]);
    }
    reinterpret_cast<uint4*>(out)[v] = o;
  }
}

void reduce_replicas(const CommBufs& srcs, int n_src, void* out, long long n_elems, int is_fp32, float scale,
                     cudaStream_t s, float beta) {
  if (n_elems <= 0) return;
  const int vec = is_fp32 ? 4 : 8;
  if (n_elems % vec) throw std::runtime_error("himuon reduce_replicas: element count must be a multiple of 16 bytes");
  long long blocks = (n_elems / vec + 511) / 512;
  const long long cap = static_cast<long long>(num_sms()) * 2;
  if (blocks > cap) blocks = cap;
  if (is_fp32)
    reduce_replicas_kernel<float><<<static_cast<int>(blocks), 512, 0, s>>>(srcs, n_src, reinterpret_cast<float*>(out), n_elems, scale, beta);
  else
    reduce_replicas_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 512, 0, s>>>(srcs, n_src, reinterpret_cast<__nv_bfloat16*>(out), n_elems, scale, beta);
}

// ------------------------------------------------------------------------------------------------ multi copy
constexpr long long kCopyUnit = 1 << 16;   // bytes per work unit

__global__ void __launch_bounds__(512)
multi_copy_kernel(const CopySeg* __restrict__ segs, int n_segs, long long total_units) {
  for (long long unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
    int lo = 0, hi = n_segs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (segs[mid].unit_begin <= unit) lo = mid; else hi = mid - 1;
    }
    const CopySeg sg = segs[lo];
    const long long off = (unit - sg.unit_begin) * kCopyUnit;
    const long long len = min(kCopyUnit, sg.bytes - off);
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(sg.src) + off);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(sg.dst) + off);
    const int nv = static_cast<int>(len >> 4);
#pragma unroll 4
    for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = src[i];
  }
}

long long multi_copy_units(long long bytes) { return (bytes + kCopyUnit - 1) / kCopyUnit; }

void multi_copy(const CopySeg* segs_dev, int n_segs, long long total_units, int max_blocks, cudaStream_t s) {
  if (total_units <= 0) return;
  long long blocks = total_units;
  const long long cap = max_blocks > 0 ? max_blocks : num_sms();
  if (blocks > cap) blocks = cap;
  multi_copy_kernel<<<static_cast<int>(blocks), 512, 0, s>>>(segs_dev, n_segs, total_units);
}

}  // namespace himuon
