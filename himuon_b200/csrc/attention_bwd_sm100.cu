// Flash attention backward, dK/dV pass, in the transposed formulation.
//
// CTA = (KV block of 128 positions, head, batch).  K_j and V_j stay in shared memory; Q and dO stream through in
// sub-blocks of 64 query positions.  The score tile is computed transposed,
//     S^T = K Q^T  and  dP^T = V dO^T        (128 key rows on the TMEM lanes, 64 query columns),
// so that after the softmax threads turn it into P^T and dS^T (bf16, written back over the same TMEM columns) those
// tiles are already in the layout of a tensor-memory A operand:
//     dV += P^T dO   and   dK += dS^T Q      (A from TMEM, B = the streamed tile read along the head dimension).
// Nothing but Q/dO/K/V touches shared memory, which leaves room for four streamed stages, and the two S^T/dP^T
// buffers let the tensor core work on sub-block i+1 while the softmax threads work on sub-block i.
//
// TMEM (512 columns): S^T buffers at 0 and 64 (P^T over the first 32 columns of each), dP^T buffers at 128 and 192
// (dS^T likewise), dV at 256, dK at 384.
// Requires S to be a multiple of 128; the per-row statistics (log-sum-exp, delta) arrive by bulk copies.
#include "attention_common.cuh"

#include <string>

namespace himuon {

namespace {

constexpr int BQ = 64;                               // query positions per streamed sub-block
constexpr uint32_t Q_HALF = BQ * 128;                // one 64-column half of a sub-block: 8 KB
constexpr uint32_t Q_TILE = 2 * Q_HALF;              // 16 KB
constexpr int NST = 4;                               // streamed stages of (Q, dO, lse, delta)
constexpr uint32_t STAT_BYTES = 2 * BQ * 4;          // lse[64] then delta[64]
constexpr uint32_t STAGE_BYTES = 2 * Q_TILE + STAT_BYTES;
// warp 0: TMA producer, warp 1: MMA issue, warps 2-5 and 6-9: two softmax groups of 128 threads (one per TMEM
// lane) that take alternate sub-blocks, so two warps per scheduler hide each other's MUFU and TMEM latencies
constexpr int BWD_THREADS = 320;

struct DkvBars {
  uint64_t kv_full, qd_full[NST], qd_empty[NST], s_full[2], p_ready[2], acc_done;
  uint32_t tmem_slot;
  int abort_flag;
};

__device__ __forceinline__ uint64_t sub_desc_kmajor(uint32_t base, int ks) {   // [64 q][128 hd] as the K-major B operand
  return umma_smem_desc(base + (ks >> 2) * Q_HALF + (ks & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t sub_desc_mnmajor(uint32_t base, int ks) {  // the same bytes read along the head dim
  return umma_smem_desc(base + ks * 2048, Q_HALF, 1024);
}
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

}  // namespace

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkv_t_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, AttnDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;                 // NST x 16 KB
  uint8_t* sDO = sQ + NST * Q_TILE;                    // NST x 16 KB
  float* sStat = reinterpret_cast<float*>(sDO + NST * Q_TILE);   // NST x (lse[64], delta[64])
  DkvBars* bars = reinterpret_cast<DkvBars*>(reinterpret_cast<uint8_t*>(sStat) + NST * STAT_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int kb, hy, b;
  attn_block_coords(kb, hy, b);        // early KV blocks (attended by the most query blocks) start first
  const int Gall = p.Hq / p.Hkv;
  const int G = p.split_heads ? 1 : Gall;
  const int hk = p.split_heads ? hy / Gall : hy;
  const int h_first = p.split_heads ? hy : hk * Gall;
  const int out_head = p.split_heads ? hy : hk;
  const int nsub = (p.S - kb * AT) / BQ;               // query sub-blocks from the diagonal to the end
  const int iters = G * nsub;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int i = 0; i < NST; ++i) { mbar_init(&bars->qd_full[i], 1); mbar_init(&bars->qd_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_ready[i], 128); }
    mbar_init(&bars->acc_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 384;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      mbar_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
      tma_load_4d(sK, &tmK, &bars->kv_full, 0, hk, kb * AT, b);
      tma_load_4d(sK + HALF_BYTES, &tmK, &bars->kv_full, 64, hk, kb * AT, b);
      tma_load_4d(sV, &tmV, &bars->kv_full, 0, hk, kb * AT, b);
      tma_load_4d(sV + HALF_BYTES, &tmV, &bars->kv_full, 64, hk, kb * AT, b);
      for (int it = 0; it < iters; ++it) {
        const int g = it / nsub;
        const int h = h_first + g;
        const int q0 = kb * AT + (it - g * nsub) * BQ;
        const int st = it % NST;
        if (!mbar_wait(&bars->qd_empty[st], ((it / NST) & 1) ^ 1, abort_flag, p.status, 4)) break;
        mbar_expect_tx(&bars->qd_full[st], STAGE_BYTES);
        uint8_t* q_dst = sQ + st * Q_TILE;
        uint8_t* do_dst = sDO + st * Q_TILE;
        tma_load_4d(q_dst, &tmQ, &bars->qd_full[st], 0, h, q0, b);
        tma_load_4d(q_dst + Q_HALF, &tmQ, &bars->qd_full[st], 64, h, q0, b);
        tma_load_4d(do_dst, &tmDO, &bars->qd_full[st], 0, h, q0, b);
        tma_load_4d(do_dst + Q_HALF, &tmDO, &bars->qd_full[st], 64, h, q0, b);
        const long long stat_idx = (static_cast<long long>(b) * p.Hq + h) * p.S + q0;
        bulk_load_1d(sStat + st * 2 * BQ, p.lse + stat_idx, BQ * 4, &bars->qd_full[st]);
        bulk_load_1d(sStat + st * 2 * BQ + BQ, p.delta + stat_idx, BQ * 4, &bars->qd_full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BQ, false, false);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, false, true);
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), q_base = smem_u32(sQ), do_base = smem_u32(sDO);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, p.status, 4);
      auto issue_sp = [&](int it) -> bool {
        const int st = it % NST, buf = it & 1;
        if (!mbar_wait(&bars->qd_full[st], (it / NST) & 1, abort_flag, p.status, 4)) return false;
        tc_fence_after();
        // The buffer's previous contents (P^T, dS^T of sub-block it-2) were consumed by MMAs issued earlier, which
        // the tensor core executes in order before these.
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tS + buf * BQ, desc_kmajor(k_base, ks), sub_desc_kmajor(q_base + st * Q_TILE, ks), idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tDP + buf * BQ, desc_kmajor(v_base, ks), sub_desc_kmajor(do_base + st * Q_TILE, ks), idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(&bars->s_full[buf]);
        return true;
      };
      if (ok) ok = issue_sp(0);
      for (int it = 0; ok && it < iters; ++it) {
        if (it + 1 < iters) { ok = issue_sp(it + 1); if (!ok) break; }
        const int st = it % NST, buf = it & 1;
        if (!mbar_wait(&bars->p_ready[buf], (it >> 1) & 1, abort_flag, p.status, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks)
          umma_ts(tDV, tS + buf * BQ + ks * 8, sub_desc_mnmajor(do_base + st * Q_TILE, ks), idesc_acc, (it > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks)
          umma_ts(tDK, tDP + buf * BQ + ks * 8, sub_desc_mnmajor(q_base + st * Q_TILE, ks), idesc_acc, (it > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&bars->qd_empty[st]);
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue: one thread per key row
    const int wg = (warp - 2) >> 2;                       // 0: even sub-blocks (buffer 0), 1: odd sub-blocks (buffer 1)
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int kv_idx = kb * AT + row;
    const int buf = wg;
    bool ok = true;
    for (int it = wg; it < iters; it += 2) {
      const int g = it / nsub;
      const int q0 = kb * AT + (it - g * nsub) * BQ;
      const int st = it % NST;
      if (!mbar_wait(&bars->qd_full[st], (it / NST) & 1, abort_flag, p.status, 4)) { ok = false; break; }
      if (!mbar_wait(&bars->s_full[buf], (it >> 1) & 1, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      const float* lse_s = sStat + st * 2 * BQ;
      const float* delta_s = lse_s + BQ;
      const bool diag = q0 < kb * AT + AT;               // some keys of this block lie after some of these queries
#pragma unroll
      for (int c = 0; c < BQ / 32; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld32(tS + buf * BQ + lane_off + c * 32, sv);
        tmem_ld32(tDP + buf * BQ + lane_off + c * 32, dv);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse_s + c * 32 + t);
          const float4 d4 = *reinterpret_cast<const float4*>(delta_s + c * 32 + t);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
          float pr[4], ds[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float pv = exp2f(fmaf(__uint_as_float(sv[t + u]), p.scale_log2, -lv[u]));
            if (diag && (q0 + c * 32 + t + u < kv_idx)) pv = 0.f;
            pr[u] = pv;
            ds[u] = pv * (__uint_as_float(dv[t + u]) - dl[u]);      // the softmax scale is applied to dK once, at the end
          }
          pk[t >> 1] = pack_bf16x2(pr[0], pr[1]);
          pk[(t >> 1) + 1] = pack_bf16x2(pr[2], pr[3]);
          dk[t >> 1] = pack_bf16x2(ds[0], ds[1]);
          dk[(t >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
        }
        // The bf16 tiles occupy the first 32 columns of their buffers, i.e. only columns of the first fp32 chunk,
        // which this thread has already read: 16 packed columns per chunk.
        tmem_st16(tS + buf * BQ + lane_off + c * 16, pk);
        tmem_st16(tDP + buf * BQ + lane_off + c * 16, dk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[buf]);
    }
    if (ok && mbar_wait(&bars->acc_done, 0, abort_flag, p.status, 4)) {
      tc_fence_after();
      // group 0 stores dV, group 1 stores dK
      __nv_bfloat16* dst0 = reinterpret_cast<__nv_bfloat16*>(wg == 0 ? p.dv : p.dk) +
                            (static_cast<long long>(b) * p.S + kv_idx) * (wg == 0 ? p.ld_dv : p.ld_dk) + out_head * HD;
      const uint32_t t_src = (wg == 0 ? tDV : tDK) + lane_off;
      const float out_scale = wg == 0 ? 1.f : p.scale;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(t_src + c * 32, v);
        tmem_ld_wait();
        __nv_bfloat16* dst = dst0 + c * 32;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o4;
          o4.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]) * out_scale, __uint_as_float(v[8 * q + 1]) * out_scale);
          o4.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]) * out_scale, __uint_as_float(v[8 * q + 3]) * out_scale);
          o4.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]) * out_scale, __uint_as_float(v[8 * q + 5]) * out_scale);
          o4.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]) * out_scale, __uint_as_float(v[8 * q + 7]) * out_scale);
          *reinterpret_cast<uint4*>(dst + q * 8) = o4;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ================================================================================================ backward: dQ
// CTA = (query block of 128 positions, head, batch).  Q_i and dO_i stay in shared memory; K and V stream through in
// sub-blocks of 64 positions.  S = Q K^T and dP = dO V^T land in one of two TMEM buffer pairs; the softmax threads
// (one per query row) write dS as bf16 over the first 32 columns of the dP buffer, which is then the tensor-memory
// A operand of dQ += dS K.  Also produces delta = rowsum(O * dO) for the dK/dV pass.
// TMEM: S buffers at 0 and 64, dP buffers at 128 and 192, dQ at 256.
struct DqBars {
  uint64_t qd_full, kv_full[NST], kv_empty[NST], s_full[2], p_ready[2], acc_done;
  uint32_t tmem_slot;
  int abort_flag;
  float delta[AT];
};

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dq_t_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, AttnDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;                 // NST x 16 KB
  uint8_t* sV = sK + NST * Q_TILE;                     // NST x 16 KB
  DqBars* bars = reinterpret_cast<DqBars*>(sV + NST * Q_TILE);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int sblk, h, b;
  attn_block_coords(sblk, h, b);
  const int qb = gridDim.x - 1 - sblk;                 // heavy (late) query blocks first
  const int hk = h / (p.Hq / p.Hkv);
  const int nkv = (qb + 1) * (AT / BQ);                // KV sub-blocks up to and including the diagonal

  if (threadIdx.x == 0) {
    mbar_init(&bars->qd_full, 1);
    for (int i = 0; i < NST; ++i) { mbar_init(&bars->kv_full[i], 1); mbar_init(&bars->kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_ready[i], 128); }
    mbar_init(&bars->acc_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDQ = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->qd_full, 2 * TILE_BYTES);
      tma_load_4d(sQ, &tmQ, &bars->qd_full, 0, h, qb * AT, b);
      tma_load_4d(sQ + HALF_BYTES, &tmQ, &bars->qd_full, 64, h, qb * AT, b);
      tma_load_4d(sDO, &tmDO, &bars->qd_full, 0, h, qb * AT, b);
      tma_load_4d(sDO + HALF_BYTES, &tmDO, &bars->qd_full, 64, h, qb * AT, b);
      for (int j = 0; j < nkv; ++j) {
        const int st = j % NST;
        if (!mbar_wait(&bars->kv_empty[st], ((j / NST) & 1) ^ 1, abort_flag, p.status, 4)) break;
        mbar_expect_tx(&bars->kv_full[st], 2 * Q_TILE);
        uint8_t* k_dst = sK + st * Q_TILE;
        uint8_t* v_dst = sV + st * Q_TILE;
        tma_load_4d(k_dst, &tmK, &bars->kv_full[st], 0, hk, j * BQ, b);
        tma_load_4d(k_dst + Q_HALF, &tmK, &bars->kv_full[st], 64, hk, j * BQ, b);
        tma_load_4d(v_dst, &tmV, &bars->kv_full[st], 0, hk, j * BQ, b);
        tma_load_4d(v_dst + Q_HALF, &tmV, &bars->kv_full[st], 64, hk, j * BQ, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BQ, false, false);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, false, true);
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), k_base = smem_u32(sK), v_base = smem_u32(sV);
      bool ok = mbar_wait(&bars->qd_full, 0, abort_flag, p.status, 4);
      auto issue_sp = [&](int j) -> bool {
        const int st = j % NST, buf = j & 1;
        if (!mbar_wait(&bars->kv_full[st], (j / NST) & 1, abort_flag, p.status, 4)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tS + buf * BQ, desc_kmajor(q_base, ks), sub_desc_kmajor(k_base + st * Q_TILE, ks), idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tDP + buf * BQ, desc_kmajor(do_base, ks), sub_desc_kmajor(v_base + st * Q_TILE, ks), idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(&bars->s_full[buf]);
        return true;
      };
      if (ok) ok = issue_sp(0);
      for (int j = 0; ok && j < nkv; ++j) {
        if (j + 1 < nkv) { ok = issue_sp(j + 1); if (!ok) break; }
        const int st = j % NST, buf = j & 1;
        if (!mbar_wait(&bars->p_ready[buf], (j >> 1) & 1, abort_flag, p.status, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks)
          umma_ts(tDQ, tDP + buf * BQ + ks * 8, sub_desc_mnmajor(k_base + st * Q_TILE, ks), idesc_acc, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&bars->kv_empty[st]);
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    const int wg = (warp - 2) >> 2;                       // 0: even KV sub-blocks (buffer 0), 1: odd (buffer 1)
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int q_idx = qb * AT + row;
    const long long stat_idx = (static_cast<long long>(b) * p.Hq + h) * p.S + q_idx;
    const float lse2 = p.lse[stat_idx];
    if (wg == 0) {
      float d = 0.f;
      const __nv_bfloat16* op = reinterpret_cast<const __nv_bfloat16*>(p.o_in) + (static_cast<long long>(b) * p.S + q_idx) * p.ld_o + h * HD;
      const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(p.d_o) + (static_cast<long long>(b) * p.S + q_idx) * p.ld_do + h * HD;
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        const uint4 a = reinterpret_cast<const uint4*>(op)[c], g = reinterpret_cast<const uint4*>(gp)[c];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) d += bf16_lo(aw[q]) * bf16_lo(gw[q]) + bf16_hi(aw[q]) * bf16_hi(gw[q]);
      }
      p.delta[stat_idx] = d;
      bars->delta[row] = d;
    }
    named_barrier(1, 256);                                // both groups: the block's delta values are in shared memory
    const float delta = bars->delta[row];
    const int buf = wg;
    bool ok = true;
    for (int j = wg; j < nkv; j += 2) {
      if (!mbar_wait(&bars->s_full[buf], (j >> 1) & 1, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BQ;
      const bool diag = (kv0 + BQ - 1 > qb * AT);
#pragma unroll
      for (int c = 0; c < BQ / 32; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld32(tS + buf * BQ + lane_off + c * 32, sv);
        tmem_ld32(tDP + buf * BQ + lane_off + c * 32, dv);
        tmem_ld_wait();
        uint32_t dk[16];
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          float p0 = exp2f(fmaf(__uint_as_float(sv[t]), p.scale_log2, -lse2));
          float p1 = exp2f(fmaf(__uint_as_float(sv[t + 1]), p.scale_log2, -lse2));
          if (diag && (kv0 + c * 32 + t > q_idx)) p0 = 0.f;
          if (diag && (kv0 + c * 32 + t + 1 > q_idx)) p1 = 0.f;
          dk[t >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv[t]) - delta), p1 * (__uint_as_float(dv[t + 1]) - delta));
        }
        tmem_st16(tDP + buf * BQ + lane_off + c * 16, dk);  // dS over columns of the first dP chunk (already read)
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[buf]);
    }
    if (ok && mbar_wait(&bars->acc_done, 0, abort_flag, p.status, 4)) {
      tc_fence_after();
      // each group stores one 64-column half of the dQ rows
      __nv_bfloat16* dqp = reinterpret_cast<__nv_bfloat16*>(p.dq) + (static_cast<long long>(b) * p.S + q_idx) * p.ld_dq + h * HD + wg * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(tDQ + lane_off + wg * 64 + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o4;                                      // dS was left unscaled: the softmax scale lands here
          o4.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]) * p.scale, __uint_as_float(v[8 * q + 1]) * p.scale);
          o4.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]) * p.scale, __uint_as_float(v[8 * q + 3]) * p.scale);
          o4.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]) * p.scale, __uint_as_float(v[8 * q + 5]) * p.scale);
          o4.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]) * p.scale, __uint_as_float(v[8 * q + 7]) * p.scale);
          *reinterpret_cast<uint4*>(dqp + c * 32 + q * 8) = o4;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// The pipelined kernels take sequence lengths that are multiples of 128 with 16-byte aligned row statistics; other
// shapes run the kernels of attention_sm100.cu / attention_kv64_sm100.cu.
bool flash_bwd_dkv_t_supported(const AttnArgs& a) {
  return a.S % AT == 0 && (reinterpret_cast<uintptr_t>(a.lse) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.delta) & 15) == 0;
}

bool flash_bwd_dq_t_supported(const AttnArgs& a) { return flash_bwd_dkv_t_supported(a); }

// `p` carries the output pointers and the split_heads flag chosen by the caller; the grid's y extent is the number of
// query heads (split_heads) or KV heads.
void flash_bwd_dkv_t(const AttnArgs& a, const AttnDev& p, int heads_y, cudaStream_t s) {
  constexpr size_t SMEM = 1024 + 2 * TILE_BYTES + 2 * NST * Q_TILE + NST * STAT_BYTES + sizeof(DkvBars) + 64;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(flash_bwd_dkv_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM); attr = true; }
  const CUtensorMap tq = head_tmap(a.q, a.B, a.S, a.Hq, a.ld_q, BQ), tk = head_tmap(a.k, a.B, a.S, a.Hkv, a.ld_k),
                    tv = head_tmap(a.v, a.B, a.S, a.Hkv, a.ld_v), tdo = head_tmap(a.d_o, a.B, a.S, a.Hq, a.ld_do, BQ);
  flash_bwd_dkv_t_kernel<<<dim3(p.nblk, heads_y, a.B), BWD_THREADS, SMEM, s>>>(tq, tk, tv, tdo, p);
}

void flash_bwd_dq_t(const AttnArgs& a, const AttnDev& p, cudaStream_t s) {
  constexpr size_t SMEM = 1024 + 2 * TILE_BYTES + 2 * NST * Q_TILE + sizeof(DqBars) + 64;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(flash_bwd_dq_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM); attr = true; }
  const CUtensorMap tq = head_tmap(a.q, a.B, a.S, a.Hq, a.ld_q), tk = head_tmap(a.k, a.B, a.S, a.Hkv, a.ld_k, BQ),
                    tv = head_tmap(a.v, a.B, a.S, a.Hkv, a.ld_v, BQ), tdo = head_tmap(a.d_o, a.B, a.S, a.Hq, a.ld_do);
  flash_bwd_dq_t_kernel<<<dim3(p.nblk, a.Hq, a.B), BWD_THREADS, SMEM, s>>>(tq, tk, tv, tdo, p);
}

}  // namespace himuon
