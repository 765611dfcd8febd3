// Causal grouped-query flash attention for head_dim 128 on sm_100a: the host entry points (flash_attn_fwd,
// flash_attn_bwd) and the dK/dV kernel for sequence lengths that are not a multiple of 128.
//
// Every score / value product runs on tcgen05 tensor cores with TMEM accumulators; Q, K, V and dO tiles arrive by
// TMA (128-byte swizzle, no multicast).  One thread owns one row of a 128-row tile, so row max / row sum need no
// shuffles.  Forward and the ragged-length dQ pass live in attention_kv64_sm100.cu, the pipelined backward kernels
// (sequence lengths that are multiples of 128) in attention_bwd_sm100.cu.  The dK/dV kernel here: CTA = (KV block,
// KV head or query head), loops over the query blocks at or below the diagonal, keeps dK and dV in TMEM, P and dS go
// through swizzled shared memory; grouped heads need no atomics.
//
// The reference reaches attention through HF `sdpa` (PyTorch library kernels); it ships no attention code of its own.
#include "attention_common.cuh"


namespace himuon {

// ================================================================================================ backward: dK, dV
// CTA = (KV block, KV head, batch).  Resident: K_j, V_j.  Streamed: Q_i, dO_i over (group head, query block).
// TMEM: S | dP | dV | dK (128 columns each).
__global__ void __launch_bounds__(192, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, AttnDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;
  uint8_t* sDO = smem + 3 * TILE_BYTES;
  uint8_t* sP = smem + 4 * TILE_BYTES;
  uint8_t* sDS = smem + 5 * TILE_BYTES;
  BwdBars* bars = reinterpret_cast<BwdBars*>(smem + 6 * TILE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int kb, hy, b;
  attn_block_coords(kb, hy, b);        // early KV blocks (attended by the most query blocks) start first
  // Grouped heads: either this CTA walks all G query heads of KV head hy, or (split_heads) it handles the
  // single query head hy and its output is a per-head partial that a later pass sums over the group.
  const int Gall = p.Hq / p.Hkv;
  const int G = p.split_heads ? 1 : Gall;
  const int hk = p.split_heads ? hy / Gall : hy;
  const int h_first = p.split_heads ? hy : hk * Gall;
  const int out_head = p.split_heads ? hy : hk;
  const int nq = p.nblk - kb;          // query blocks kb .. nblk-1
  const int iters = G * nq;

  if (threadIdx.x == 0) {
    mbar_init(&bars->a_full, 1); mbar_init(&bars->a_empty, 1);
    mbar_init(&bars->b_full, 1); mbar_init(&bars->b_empty, 1);
    mbar_init(&bars->sp_full, 1); mbar_init(&bars->ds_ready, 128); mbar_init(&bars->acc_done, 1);
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
    if (lane == 0) {
      mbar_expect_tx(&bars->a_full, 2 * TILE_BYTES);
      tma_load_4d(sK, &tmK, &bars->a_full, 0, hk, kb * AT, b);
      tma_load_4d(sK + HALF_BYTES, &tmK, &bars->a_full, 64, hk, kb * AT, b);
      tma_load_4d(sV, &tmV, &bars->a_full, 0, hk, kb * AT, b);
      tma_load_4d(sV + HALF_BYTES, &tmV, &bars->a_full, 64, hk, kb * AT, b);
      for (int it = 0; it < iters; ++it) {
        const int g = it / nq, qi = kb + (it - g * nq);
        const int h = h_first + g;
        if (!mbar_wait(&bars->b_empty, (it & 1) ^ 1, abort_flag, p.status, 4)) break;
        mbar_expect_tx(&bars->b_full, 2 * TILE_BYTES);
        tma_load_4d(sQ, &tmQ, &bars->b_full, 0, h, qi * AT, b);
        tma_load_4d(sQ + HALF_BYTES, &tmQ, &bars->b_full, 64, h, qi * AT, b);
        tma_load_4d(sDO, &tmDO, &bars->b_full, 0, h, qi * AT, b);
        tma_load_4d(sDO + HALF_BYTES, &tmDO, &bars->b_full, 64, h, qi * AT, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_mm = umma_idesc_bf16(128, 128, true, true);
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), k_base = smem_u32(sK), v_base = smem_u32(sV),
                     p_base = smem_u32(sP), ds_base = smem_u32(sDS);
      bool ok = mbar_wait(&bars->a_full, 0, abort_flag, p.status, 4);
      for (int it = 0; ok && it < iters; ++it) {
        if (!mbar_wait(&bars->b_full, it & 1, abort_flag, p.status, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ss(tS, desc_kmajor(q_base, ks), desc_kmajor(k_base, ks), idesc_kk, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ss(tDP, desc_kmajor(do_base, ks), desc_kmajor(v_base, ks), idesc_kk, ks > 0 ? 1u : 0u);
        umma_commit(&bars->sp_full);
        if (!mbar_wait(&bars->ds_ready, it & 1, abort_flag, p.status, 4)) break;
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q : both operands MN-major views of [query rows][cols] tiles
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tDV, desc_mnmajor(p_base, ks), desc_mnmajor(do_base, ks), idesc_mm, (it > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tDK, desc_mnmajor(ds_base, ks), desc_mnmajor(q_base, ks), idesc_mm, (it > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&bars->b_empty);
        umma_commit(&bars->acc_done);
      }
    }
  } else {
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      const int g = it / nq, qi = kb + (it - g * nq);
      const int h = h_first + g;
      const int q_idx = qi * AT + row;
      const bool row_ok = q_idx < p.S;
      float lse2 = 0.f, delta = 0.f;
      if (row_ok) {
        const long long stat_idx = (static_cast<long long>(b) * p.Hq + h) * p.S + q_idx;
        lse2 = p.lse[stat_idx];
        delta = p.delta[stat_idx];
      }
      if (!mbar_wait(&bars->sp_full, it & 1, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      if (it > 0 && !mbar_wait(&bars->acc_done, (it - 1) & 1, abort_flag, p.status, 4)) { ok = false; break; }
      const bool diag = (qi == kb);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld32(tS + lane_off + c * 32, sv);
        tmem_ld32(tDP + lane_off + c * 32, dv);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          float p0 = exp2f(__uint_as_float(sv[t]) * p.scale_log2 - lse2);
          float p1 = exp2f(__uint_as_float(sv[t + 1]) * p.scale_log2 - lse2);
          if (!row_ok || (diag && (c * 32 + t > row))) p0 = 0.f;
          if (!row_ok || (diag && (c * 32 + t + 1 > row))) p1 = 0.f;
          pk[t >> 1] = pack_bf16x2(p0, p1);
          dk[t >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv[t]) - delta) * p.scale,
                                   p1 * (__uint_as_float(dv[t + 1]) - delta) * p.scale);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          *reinterpret_cast<uint4*>(sP + sw128_off(row, c * 4 + q)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
          *reinterpret_cast<uint4*>(sDS + sw128_off(row, c * 4 + q)) = make_uint4(dk[4 * q], dk[4 * q + 1], dk[4 * q + 2], dk[4 * q + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&bars->ds_ready);
    }
    if (ok && mbar_wait(&bars->acc_done, (iters - 1) & 1, abort_flag, p.status, 4)) {
      tc_fence_after();
      const int k_idx = kb * AT + row;   // accumulator rows are key positions
      const bool row_ok = k_idx < p.S;
      __nv_bfloat16* dkp = reinterpret_cast<__nv_bfloat16*>(p.dk) + (static_cast<long long>(b) * p.S + k_idx) * p.ld_dk + out_head * HD;
      __nv_bfloat16* dvp = reinterpret_cast<__nv_bfloat16*>(p.dv) + (static_cast<long long>(b) * p.S + k_idx) * p.ld_dv + out_head * HD;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t v[32];
        tmem_ld32((c < 4 ? tDV : tDK) + lane_off + (c & 3) * 32, v);
        tmem_ld_wait();
        __nv_bfloat16* dst = (c < 4 ? dvp : dkp) + (c & 3) * 32;
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
            o4.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
            o4.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
            o4.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
            *reinterpret_cast<uint4*>(dst + q * 8) = o4;
          }
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

// ================================================================================================ host
static void check_attn(const AttnArgs& a) {
  if (a.S <= 0 || a.B <= 0 || a.Hq <= 0 || a.Hkv <= 0 || a.Hq % a.Hkv) throw std::runtime_error("himuon attention: bad sizes");
  if (a.ld_q % 8 || a.ld_k % 8 || a.ld_v % 8 || a.ld_o % 8) throw std::runtime_error("himuon attention: token strides must be multiples of 8");
}

void flash_attn_fwd(const AttnArgs& a, cudaStream_t s) {
  check_attn(a);
  flash_fwd_kv64(a, s);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("himuon flash_attn_fwd launch failed: ") + cudaGetErrorString(e));
}

void flash_attn_bwd(const AttnArgs& a, cudaStream_t s) {
  check_attn(a);
  if (a.ld_do % 8 || a.ld_dq % 8 || a.ld_dk % 8 || a.ld_dv % 8) throw std::runtime_error("himuon attention: gradient strides must be multiples of 8");
  constexpr size_t SMEM_DKV = 1024 + 6 * TILE_BYTES + 512;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_DKV);
    attr = true;
  }
  AttnDev p{};
  p.lse = a.lse; p.delta = a.delta; p.o_in = a.o; p.d_o = a.d_o; p.dq = a.dq; p.dk = a.dk; p.dv = a.dv;
  p.B = a.B; p.S = a.S; p.Hq = a.Hq; p.Hkv = a.Hkv;
  p.ld_o = a.ld_o; p.ld_do = a.ld_do; p.ld_dq = a.ld_dq; p.ld_dk = a.ld_dk; p.ld_dv = a.ld_dv;
  p.nblk = (a.S + AT - 1) / AT;
  p.scale = a.scale; p.scale_log2 = a.scale * kLog2e;
  p.status = status_word_ptr();
  const CUtensorMap tq = head_tmap(a.q, a.B, a.S, a.Hq, a.ld_q), tk = head_tmap(a.k, a.B, a.S, a.Hkv, a.ld_k),
                    tv = head_tmap(a.v, a.B, a.S, a.Hkv, a.ld_v), tdo = head_tmap(a.d_o, a.B, a.S, a.Hq, a.ld_do);
  if (flash_bwd_dq_t_supported(a)) flash_bwd_dq_t(a, p, s);
  else flash_bwd_dq_kv64(a, s);                       // sequence lengths that are not a multiple of 128
  const int G = a.Hq / a.Hkv;
  if (G > 1 && a.dk_part != nullptr && a.dv_part != nullptr) {
    // one CTA per (KV block, query head): G times more CTAs, balanced across the SMs; the per-head partial
    // gradients are then summed over each group
    AttnDev ps = p;
    ps.split_heads = 1;
    ps.dk = a.dk_part; ps.dv = a.dv_part; ps.ld_dk = a.ld_part; ps.ld_dv = a.ld_part;
    if (flash_bwd_dkv_t_supported(a)) flash_bwd_dkv_t(a, ps, a.Hq, s);
    else flash_bwd_dkv_kernel<<<dim3(p.nblk, a.Hq, a.B), 192, SMEM_DKV, s>>>(tq, tk, tv, tdo, ps);
    const long long tokens = static_cast<long long>(a.B) * a.S;
    group_sum_heads(a.dk_part, a.dk, tokens, a.Hkv, G, a.ld_part, a.ld_dk, s);
    group_sum_heads(a.dv_part, a.dv, tokens, a.Hkv, G, a.ld_part, a.ld_dv, s);
  } else if (flash_bwd_dkv_t_supported(a)) {
    flash_bwd_dkv_t(a, p, a.Hkv, s);
  } else {
    flash_bwd_dkv_kernel<<<dim3(p.nblk, a.Hkv, a.B), 192, SMEM_DKV, s>>>(tq, tk, tv, tdo, p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("himuon flash_attn_bwd launch failed: ") + cudaGetErrorString(e));
}

}  // namespace himuon
