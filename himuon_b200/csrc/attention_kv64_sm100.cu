// Flash attention forward and dQ kernels with 64-wide KV blocks.
//
// K/V arrive in blocks of 64 positions: shared memory stays at 96 KB and the TMEM footprint at 256 columns, so two
// CTAs run on every SM and one CTA's tensor-core work overlaps the other's softmax.  The dQ kernel here serves
// sequence lengths that are not a multiple of 128; the others take the pipelined kernel of attention_bwd_sm100.cu.
#include "attention_common.cuh"

#include <string>

namespace himuon {

constexpr int BKV = 64;                              // KV positions per block
constexpr uint32_t KV_HALF = BKV * 128;              // one 64-column half of a K or V block: 8 KB
constexpr uint32_t KV_TILE = 2 * KV_HALF;            // 16 KB
constexpr uint32_t P_BYTES = AT * BKV * 2;           // probabilities / dS of one block: 128 x 64 bf16 = 16 KB

__device__ __forceinline__ uint64_t kv_desc_kmajor(uint32_t base, int ks) {   // K block as the K-major B operand of Q K^T
  return umma_smem_desc(base + (ks >> 2) * KV_HALF + (ks & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t kv_desc_mnmajor(uint32_t base, int ks) {  // K or V block read along the head dim
  return umma_smem_desc(base + ks * 2048, KV_HALF, 1024);
}
__device__ __forceinline__ uint64_t p_desc_kmajor(uint32_t base, int ks) {    // 128 x 64 block, one 128-byte line per row
  return umma_smem_desc(base + ks * 32, 16, 1024);
}
__device__ __forceinline__ uint32_t p_off(int r, int c16) {                  // 16-byte chunk c16 (0..7) of row r
  return static_cast<uint32_t>(r * 128 + ((c16 ^ (r & 7)) << 4));
}

// ================================================================================================ forward, P in TMEM
// CTA = (128 query rows, head, batch); loops over 64-wide KV blocks up to the diagonal; S(j+1) = Q K^T is issued
// before P(j) V so the tensor core overlaps the softmax; O stays in TMEM and is rescaled lazily (only when a row max
// grows by > 2^8).  The probabilities never touch shared memory: the softmax threads write P (bf16) over the first 32
// columns of the S buffer they just read and P·V runs with the A operand in tensor memory.  The two S buffers
// therefore double-buffer P as well, the wait for the previous P·V is only needed on the rare O rescale, S is read
// from TMEM once, and K and V each have two 16 KB stages.
struct Fwd64TBars {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], o_done;
  uint32_t tmem_slot;
  int abort_flag;
};

__global__ void __launch_bounds__(192, 2)
flash_fwd64_t_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, AttnDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sQ = smem;                          // 32 KB
  uint8_t* sK = smem + TILE_BYTES;             // 2 stages x 16 KB
  uint8_t* sV = sK + 2 * KV_TILE;              // 2 stages x 16 KB
  Fwd64TBars* bars = reinterpret_cast<Fwd64TBars*>(sV + 2 * KV_TILE);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int sblk, h, b;
  attn_block_coords(sblk, h, b);
  const int qb = gridDim.x - 1 - sblk;         // heavy (late) query blocks first
  const int hk = h / (p.Hq / p.Hkv);
  int nkv = (qb + 1) * (AT / BKV);             // KV blocks up to and including the diagonal
  const int nkv_all = (p.S + BKV - 1) / BKV;
  if (nkv > nkv_all) nkv = nkv_all;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1); mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1); mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_ready[i], 128);
    }
    mbar_init(&bars->o_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t tS0 = tmem, tO = tmem + 128;   // S / P buffers at columns 0 and 64, O at 128

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, TILE_BYTES);
      tma_load_4d(sQ, &tmQ, &bars->q_full, 0, h, qb * AT, b);
      tma_load_4d(sQ + HALF_BYTES, &tmQ, &bars->q_full, 64, h, qb * AT, b);
      for (int j = 0; j < nkv; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&bars->k_empty[st], par, abort_flag, p.status, 4)) break;
        mbar_expect_tx(&bars->k_full[st], KV_TILE);
        tma_load_4d(sK + st * KV_TILE, &tmK, &bars->k_full[st], 0, hk, j * BKV, b);
        tma_load_4d(sK + st * KV_TILE + KV_HALF, &tmK, &bars->k_full[st], 64, hk, j * BKV, b);
        if (!mbar_wait(&bars->v_empty[st], par, abort_flag, p.status, 4)) break;
        mbar_expect_tx(&bars->v_full[st], KV_TILE);
        tma_load_4d(sV + st * KV_TILE, &tmV, &bars->v_full[st], 0, hk, j * BKV, b);
        tma_load_4d(sV + st * KV_TILE + KV_HALF, &tmV, &bars->v_full[st], 64, hk, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BKV, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, false, true);
      const uint32_t q_base = smem_u32(sQ), v_base = smem_u32(sV);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, p.status, 4);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&bars->k_full[st], (j >> 1) & 1, abort_flag, p.status, 4)) return false;
        tc_fence_after();
        // buffer st held S(j-2) / P(j-2): the softmax threads are done with it (p_ready(j-2) was waited for) and the
        // P(j-2)·V MMAs were issued earlier, which the tensor core executes in order before these
        const uint32_t k_base = smem_u32(sK + st * KV_TILE);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tS0 + st * BKV, desc_kmajor(q_base, ks), kv_desc_kmajor(k_base, ks), idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(&bars->k_empty[st]);
        umma_commit(&bars->s_full[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < nkv; ++j) {
        if (j + 1 < nkv) { ok = issue_s(j + 1); if (!ok) break; }
        const int st = j & 1;
        if (!mbar_wait(&bars->p_ready[st], (j >> 1) & 1, abort_flag, p.status, 4)) break;
        if (!mbar_wait(&bars->v_full[st], (j >> 1) & 1, abort_flag, p.status, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks)
          umma_ts(tO, tS0 + st * BKV + ks * 8, kv_desc_mnmajor(v_base + st * KV_TILE, ks), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&bars->v_empty[st]);
        umma_commit(&bars->o_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue: one thread per query row
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int q_idx = qb * AT + row;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      const int st = j & 1;
      if (!mbar_wait(&bars->s_full[st], (j >> 1) & 1, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tS = tS0 + st * BKV + lane_off;
      const int kv0 = j * BKV;
      const bool diag = (kv0 + BKV - 1 > qb * AT);       // the block reaches past the first row of this query tile
      uint32_t v0[32], v1[32];
      tmem_ld32(tS, v0);
      tmem_ld32(tS + 32, v1);
      tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int t = 0; t < 32; ++t) {
        float s0 = __uint_as_float(v0[t]) * p.scale_log2, s1 = __uint_as_float(v1[t]) * p.scale_log2;
        if (diag && (kv0 + t > q_idx)) s0 = -INFINITY;
        if (diag && (kv0 + 32 + t > q_idx)) s1 = -INFINITY;
        v0[t] = __float_as_uint(s0);
        v1[t] = __float_as_uint(s1);
        mx = fmaxf(mx, fmaxf(s0, s1));
      }
      const float m_new = fmaxf(m_used, mx);
      const bool need = (j > 0) && (m_new - m_used > 8.f);
      const bool warp_need = __any_sync(0xffffffffu, need);
      if (j == 0) {
        m_used = m_new;
      } else if (warp_need) {
        // O (and l) move to the new maximum: the previous P·V must have landed in O first
        const float alpha = exp2f(m_used - m_new);
        m_used = m_new;
        if (!mbar_wait(&bars->o_done, (j - 1) & 1, abort_flag, p.status, 4)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(tO + lane_off + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
          tmem_st32(tO + lane_off + c * 32, v);
        }
        l *= alpha;
      }
      uint32_t pk[32];
      float rs = 0.f;
#pragma unroll
      for (int t = 0; t < 32; t += 2) {
        // masked entries are -inf: exp2 gives exactly 0
        pk[t >> 1] = pack_bf16x2(exp2f(__uint_as_float(v0[t]) - m_used), exp2f(__uint_as_float(v0[t + 1]) - m_used));
        pk[16 + (t >> 1)] = pack_bf16x2(exp2f(__uint_as_float(v1[t]) - m_used), exp2f(__uint_as_float(v1[t + 1]) - m_used));
        rs += bf16_lo(pk[t >> 1]) + bf16_hi(pk[t >> 1]) + bf16_lo(pk[16 + (t >> 1)]) + bf16_hi(pk[16 + (t >> 1)]);
      }
      l += rs;
      tmem_st32(tS, pk);                     // P over the first 32 columns of the S buffer just read
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[st]);
    }
    if (ok && mbar_wait(&bars->o_done, (nkv - 1) & 1, abort_flag, p.status, 4)) {
      tc_fence_after();
      const float inv = 1.f / l;
      const bool row_ok = q_idx < p.S;
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.o) + (static_cast<long long>(b) * p.S + q_idx) * p.ld_o + h * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tO + lane_off + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]) * inv, __uint_as_float(v[8 * q + 1]) * inv);
            o4.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]) * inv, __uint_as_float(v[8 * q + 3]) * inv);
            o4.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]) * inv, __uint_as_float(v[8 * q + 5]) * inv);
            o4.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]) * inv, __uint_as_float(v[8 * q + 7]) * inv);
            *reinterpret_cast<uint4*>(op + c * 32 + q * 8) = o4;
          }
        }
      }
      if (row_ok) p.lse[(static_cast<long long>(b) * p.Hq + h) * p.S + q_idx] = m_used + log2f(l);   // base-2 log-sum-exp of the scaled scores
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ================================================================================================ backward: dQ
// CTA = (query block, head, batch).  Resident: Q, dO.  Streamed: K_j, V_j (64 positions).  dS reuses V's shared
// memory once dP = dO V^T has consumed V.  TMEM: S (64) | dP (64) | dQ (128).
__global__ void __launch_bounds__(192, 2)
flash_bwd_dq64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, AttnDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;
  uint8_t* sV = sK + KV_TILE;
  uint8_t* sDS = sV;                                    // alias (see above)
  BwdBars* bars = reinterpret_cast<BwdBars*>(sV + KV_TILE);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int sblk, h, b;
  attn_block_coords(sblk, h, b);
  const int qb = gridDim.x - 1 - sblk;         // heavy (late) query blocks first
  const int hk = h / (p.Hq / p.Hkv);
  int nkv = (qb + 1) * (AT / BKV);
  const int nkv_all = (p.S + BKV - 1) / BKV;
  if (nkv > nkv_all) nkv = nkv_all;

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1); mbar_init(&bars->a_empty, 1);
    mbar_init(&bars->b_full, 1); mbar_init(&bars->b_empty, 1);
    mbar_init(&bars->sp_full, 1); mbar_init(&bars->ds_ready, 128); mbar_init(&bars->acc_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 64, tDQ = tmem + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->a_full, 2 * TILE_BYTES);
      tma_load_4d(sQ, &tmQ, &bars->a_full, 0, h, qb * AT, b);
      tma_load_4d(sQ + HALF_BYTES, &tmQ, &bars->a_full, 64, h, qb * AT, b);
      tma_load_4d(sDO, &tmDO, &bars->a_full, 0, h, qb * AT, b);
      tma_load_4d(sDO + HALF_BYTES, &tmDO, &bars->a_full, 64, h, qb * AT, b);
      for (int j = 0; j < nkv; ++j) {
        if (!mbar_wait(&bars->b_empty, (j & 1) ^ 1, abort_flag, p.status, 4)) break;
        mbar_expect_tx(&bars->b_full, 2 * KV_TILE);
        tma_load_4d(sK, &tmK, &bars->b_full, 0, hk, j * BKV, b);
        tma_load_4d(sK + KV_HALF, &tmK, &bars->b_full, 64, hk, j * BKV, b);
        tma_load_4d(sV, &tmV, &bars->b_full, 0, hk, j * BKV, b);
        tma_load_4d(sV + KV_HALF, &tmV, &bars->b_full, 64, hk, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, BKV, false, false);
      constexpr uint32_t idesc_kmn = umma_idesc_bf16(128, 128, false, true);
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), k_base = smem_u32(sK), v_base = smem_u32(sV),
                     ds_base = smem_u32(sDS);
      bool ok = mbar_wait(&bars->a_full, 0, abort_flag, p.status, 4);
      for (int j = 0; ok && j < nkv; ++j) {
        if (!mbar_wait(&bars->b_full, j & 1, abort_flag, p.status, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ss(tS, desc_kmajor(q_base, ks), kv_desc_kmajor(k_base, ks), idesc_kk, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ss(tDP, desc_kmajor(do_base, ks), kv_desc_kmajor(v_base, ks), idesc_kk, ks > 0 ? 1u : 0u);
        umma_commit(&bars->sp_full);
        if (!mbar_wait(&bars->ds_ready, j & 1, abort_flag, p.status, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks)
          umma_ss(tDQ, p_desc_kmajor(ds_base, ks), kv_desc_mnmajor(k_base, ks), idesc_kmn, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&bars->b_empty);
        umma_commit(&bars->acc_done);
      }
    }
  } else {
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int q_idx = qb * AT + row;
    const bool row_ok = q_idx < p.S;
    const long long stat_idx = (static_cast<long long>(b) * p.Hq + h) * p.S + q_idx;
    float lse2 = 0.f, delta = 0.f;
    if (row_ok) {
      lse2 = p.lse[stat_idx];
      const __nv_bfloat16* op = reinterpret_cast<const __nv_bfloat16*>(p.o_in) + (static_cast<long long>(b) * p.S + q_idx) * p.ld_o + h * HD;
      const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(p.d_o) + (static_cast<long long>(b) * p.S + q_idx) * p.ld_do + h * HD;
#pragma unroll 4
      for (int c = 0; c < 16; ++c) {
        const uint4 a = reinterpret_cast<const uint4*>(op)[c], g = reinterpret_cast<const uint4*>(gp)[c];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) delta += bf16_lo(aw[q]) * bf16_lo(gw[q]) + bf16_hi(aw[q]) * bf16_hi(gw[q]);
      }
      p.delta[stat_idx] = delta;
    }
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      if (!mbar_wait(&bars->sp_full, j & 1, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BKV;
      const bool diag = (kv0 + BKV - 1 > qb * AT);
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld32(tS + lane_off + c * 32, sv);
        tmem_ld32(tDP + lane_off + c * 32, dv);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          float p0 = exp2f(__uint_as_float(sv[t]) * p.scale_log2 - lse2);
          float p1 = exp2f(__uint_as_float(sv[t + 1]) * p.scale_log2 - lse2);
          if (!row_ok || (diag && (kv0 + c * 32 + t > q_idx))) p0 = 0.f;
          if (!row_ok || (diag && (kv0 + c * 32 + t + 1 > q_idx))) p1 = 0.f;
          pk[t >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv[t]) - delta) * p.scale,
                                   p1 * (__uint_as_float(dv[t + 1]) - delta) * p.scale);
        }
        // sp_full means both S and dP (which read V) are complete, so V's buffer may now hold dS
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(sDS + p_off(row, c * 4 + q)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&bars->ds_ready);
    }
    if (ok && mbar_wait(&bars->acc_done, (nkv - 1) & 1, abort_flag, p.status, 4)) {
      tc_fence_after();
      __nv_bfloat16* dqp = reinterpret_cast<__nv_bfloat16*>(p.dq) + (static_cast<long long>(b) * p.S + q_idx) * p.ld_dq + h * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tDQ + lane_off + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
            o4.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
            o4.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
            o4.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
            *reinterpret_cast<uint4*>(dqp + c * 32 + q * 8) = o4;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// ================================================================================================ host
static AttnDev make_dev(const AttnArgs& a) {
  AttnDev p{};
  p.o = a.o; p.lse = a.lse; p.delta = a.delta; p.o_in = a.o; p.d_o = a.d_o; p.dq = a.dq; p.dk = a.dk; p.dv = a.dv;
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv;
  p.ld_o = a.ld_o; p.ld_do = a.ld_do; p.ld_dq = a.ld_dq; p.ld_dk = a.ld_dk; p.ld_dv = a.ld_dv;
  p.nblk = (a.S + AT - 1) / AT;
  p.scale = a.scale; p.scale_log2 = a.scale * kLog2e;
  p.status = status_word_ptr();
  return p;
}

void flash_fwd_kv64(const AttnArgs& a, cudaStream_t s) {
  constexpr size_t SMEM = 1024 + TILE_BYTES + 3 * KV_TILE + P_BYTES + 256;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(flash_fwd64_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    attr = true;
  }
  const AttnDev p = make_dev(a);
  const CUtensorMap tq = head_tmap(a.q, a.B, a.S, a.Hq, a.ld_q), tk = head_tmap(a.k, a.B, a.S, a.Hkv, a.ld_k, BKV),
                    tv = head_tmap(a.v, a.B, a.S, a.Hkv, a.ld_v, BKV);
  flash_fwd64_t_kernel<<<dim3(p.nblk, a.Hq, a.B), 192, SMEM, s>>>(tq, tk, tv, p);
}

void flash_bwd_dq_kv64(const AttnArgs& a, cudaStream_t s) {
  constexpr size_t SMEM = 1024 + 2 * TILE_BYTES + 2 * KV_TILE + 256;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(flash_bwd_dq64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM); attr = true; }
  const AttnDev p = make_dev(a);
  const CUtensorMap tq = head_tmap(a.q, a.B, a.S, a.Hq, a.ld_q), tk = head_tmap(a.k, a.B, a.S, a.Hkv, a.ld_k, BKV),
                    tv = head_tmap(a.v, a.B, a.S, a.Hkv, a.ld_v, BKV), tdo = head_tmap(a.d_o, a.B, a.S, a.Hq, a.ld_do);
  flash_bwd_dq64_kernel<<<dim3(p.nblk, a.Hq, a.B), 192, SMEM, s>>>(tq, tk, tv, tdo, p);
}

}  // namespace himuon
