// Definitions shared by the attention kernels (128-wide and 64-wide KV-block variants).
#pragma once

#include "himuon.h"
#include "sm100_common.cuh"
#include "tma_host.h"

namespace himuon {

constexpr int AT = 128;                 // tile rows (queries) and tile columns (keys)
constexpr int HD = 128;                 // head dim
constexpr uint32_t TILE_BYTES = AT * HD * 2;   // 32 KB: two 64-column halves of 16 KB
constexpr uint32_t HALF_BYTES = 16384;
constexpr float kLog2e = 1.4426950408889634f;

// Byte offset of the 16-byte chunk `c16` (0..15) of row `r` in a [128 rows][128 cols] bf16 tile
// stored as two K-major SWIZZLE_128B halves.
__device__ __forceinline__ uint32_t sw128_off(int r, int c16) {
  return static_cast<uint32_t>((c16 >> 3) * HALF_BYTES + r * 128 + (((c16 & 7) ^ (r & 7)) << 4));
}
// K-major operand descriptor for k-step ks (16 columns each) of such a tile.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int ks) {
  return umma_smem_desc(base + (ks >> 2) * HALF_BYTES + (ks & 3) * 32, 16, 1024);
}
// MN-major operand descriptor for k-step ks (16 rows each) of the same bytes viewed as [K rows][M/N cols].
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int ks) {
  return umma_smem_desc(base + ks * 2048, HALF_BYTES, 1024);
}

struct AttnDev {
  void* o; float* lse; float* delta;
  const void* o_in; const void* d_o;
  void* dq; void* dk; void* dv;
  int B, S, Hq, Hkv, nblk;
  int split_heads;      // dkv kernel: 1 = one CTA per (KV block, query head) writing per-head partials
  long long ld_o, ld_do, ld_dq, ld_dk, ld_dv;
  float scale_log2, scale;
  int* status;
};

struct AttnBars {
  uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_empty[2], p_ready, o_done;
  uint32_t tmem_slot;
  int abort_flag;
};

struct BwdBars {
  uint64_t a_full, a_empty, b_full, b_empty, sp_full, ds_ready, acc_done;
  uint32_t tmem_slot;
  int abort_flag;
};

// 4-D tensor map over a (B, S, H, 128) view: box = 64 head-dim columns x `rows` sequence positions of one head.
inline CUtensorMap head_tmap(const void* ptr, int B, int S, int H, long long ld, int rows = AT) {
  // dims (innermost first): head_dim, heads, sequence, batch
  const uint64_t dims[4] = {HD, static_cast<uint64_t>(H), static_cast<uint64_t>(S), static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {HD * 2, static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(ld) * 2 * static_cast<uint64_t>(S)};
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(rows), 1};
  return make_tmap(ptr, 4, dims, strides, box, 2, true);
}


// CTAs start in linear block order (x fastest).  The causal work of a CTA depends only on its position along the
// sequence, so that position is decoded as the slowest coordinate: all the heaviest blocks start first and the
// light ones fill the tail of the launch (longest-processing-time order).  `sblk` counts from 0 = first started.
__device__ __forceinline__ void attn_block_coords(int& sblk, int& head, int& batch) {
  const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const int per = gridDim.y * gridDim.z;
  sblk = lin / per;
  const int r = lin - sblk * per;
  batch = r / gridDim.y;
  head = r - batch * gridDim.y;
}

// 64-wide KV-block kernels (two CTAs per SM): forward and dQ.
void flash_fwd_kv64(const AttnArgs& a, cudaStream_t s);
void flash_bwd_dq_kv64(const AttnArgs& a, cudaStream_t s);

// dK/dV pass in the transposed formulation (P^T and dS^T stay in tensor memory); S must be a multiple of 128.
bool flash_bwd_dkv_t_supported(const AttnArgs& a);
void flash_bwd_dkv_t(const AttnArgs& a, const AttnDev& p, int heads_y, cudaStream_t s);
bool flash_bwd_dq_t_supported(const AttnArgs& a);
void flash_bwd_dq_t(const AttnArgs& a, const AttnDev& p, cudaStream_t s);

}  // namespace himuon
