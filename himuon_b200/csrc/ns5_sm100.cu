// Tile-resident quintic Newton-Schulz for small tiles (rows <= 128, cols in {64,128,192,256}).
//
// One CTA owns one tile for the whole computation: X, A = X X^T and B = c*A*A + b*A live in
// swizzled shared memory as bf16 UMMA operands, every product runs on tcgen05 with fp32
// accumulators in TMEM, and nothing but the input and the result touches HBM.  The three products
// of an iteration form a chain (each is drained to shared memory before the next is issued), so
// the chain's latency is hidden by co-resident CTAs, and the kernel keeps its footprint small to
// fit as many as possible: B overwrites A in place (every thread rewrites the row chunks it has
// just read), and tiles up to 128 columns wide use a single 128-column accumulator for all three
// products - 64 KB of shared memory and 128 TMEM columns per CTA, three CTAs per SM.  Wider tiles
// need 256 columns for B*X and run two CTAs per SM.  Rounding points follow the reference's
// fused Triton kernel (src/himuon/triton_kernels/ns5_smem.py:46-104): normalise in fp32 then
// round; A, B and B*X are rounded to bf16; X <- bf16(bf16(B X) + a*X).
//
// Rows are padded to the 128-row UMMA shape by TMA zero fill, so short tiles cost a full
// 128-row MMA but need no separate code path.
#include "himuon.h"
#include "sm100_common.cuh"
#include "tma_host.h"

namespace himuon {

constexpr uint32_t NS_HALF = 16384;   // one [128 rows][64 cols] bf16 swizzled block

__device__ __forceinline__ uint32_t ns_sw_off(int r, int c16) {   // 16-byte chunk c16 of row r
  return static_cast<uint32_t>((c16 >> 3) * NS_HALF + r * 128 + (((c16 & 7) ^ (r & 7)) << 4));
}
__device__ __forceinline__ uint64_t ns_desc_k(uint32_t base, int ks) {
  return umma_smem_desc(base + (ks >> 2) * NS_HALF + (ks & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t ns_desc_mn(uint32_t base, int ks) {
  return umma_smem_desc(base + ks * 2048, NS_HALF, 1024);
}

struct NsBars {
  uint64_t tma, mma;
  uint32_t tmem_slot;
  int abort_flag;
  float red[4];
};

template <int NCH>   // number of 64-column chunks of X
__global__ void __launch_bounds__(128)
ns5_fused_kernel(const __grid_constant__ CUtensorMap tmX, __nv_bfloat16* __restrict__ out, long long n_tiles, int m,
                 int steps, float eps, int* status) {
  constexpr int N = NCH * 64;
  constexpr int TM_COLS = N <= 128 ? 128 : 256;            // TMEM columns of this CTA
  constexpr uint32_t A2_COL = TM_COLS == 256 ? 128 : 0;    // A*A lands beside A when there is room, else over it
  constexpr float ca = 3.4445f, cb = -4.7750f, cc = 2.0315f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sX = smem;
  uint8_t* sA = smem + NCH * NS_HALF;
  uint8_t* sB = sA;                                        // B replaces A in place
  NsBars* bars = reinterpret_cast<NsBars*>(sA + 2 * NS_HALF);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = threadIdx.x;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

  if (threadIdx.x == 0) {
    mbar_init(&bars->tma, 1);
    mbar_init(&bars->mma, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&bars->tmem_slot, TM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  const uint32_t x_base = smem_u32(sX), a_base = smem_u32(sA), b_base = smem_u32(sB);
  constexpr uint32_t idesc_aat = umma_idesc_bf16(128, 128, false, false);
  constexpr uint32_t idesc_bx = umma_idesc_bf16(128, N, false, true);

  uint32_t tma_phase = 0, mma_phase = 0;
  bool ok = true;
  for (long long tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
    if (threadIdx.x == 0) {
      mbar_expect_tx(&bars->tma, NCH * NS_HALF);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_3d(sX + c * NS_HALF, &tmX, &bars->tma, c * 64, 0, static_cast<int>(tile));
    }
    if (!mbar_wait(&bars->tma, tma_phase, abort_flag, status, 5)) { ok = false; break; }
    tma_phase ^= 1;

    // ---- Frobenius norm and normalisation (each thread owns one row of X)
    float ss = 0.f;
#pragma unroll 4
    for (int c = 0; c < NCH * 8; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(sX + ns_sw_off(row, c));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float a = bf16_lo(w[q]), b = bf16_hi(w[q]); ss += a * a + b * b; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) bars->red[warp] = ss;
    __syncthreads();
    const float tot = bars->red[0] + bars->red[1] + bars->red[2] + bars->red[3];
    const float inv = 1.f / (sqrtf(tot) + eps);
#pragma unroll 4
    for (int c = 0; c < NCH * 8; ++c) {
      uint4* ptr = reinterpret_cast<uint4*>(sX + ns_sw_off(row, c));
      uint4 v = *ptr;
      uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(bf16_lo(w[q]) * inv, bf16_hi(w[q]) * inv);
      *ptr = make_uint4(w[0], w[1], w[2], w[3]);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();

    for (int it = 0; it < steps; ++it) {
      // ---- A = X X^T  -> TMEM columns [0,128)
      if (threadIdx.x == 0) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < NCH * 4; ++ks) umma_ss(tmem, ns_desc_k(x_base, ks), ns_desc_k(x_base, ks), idesc_aat, ks > 0 ? 1u : 0u);
        umma_commit(&bars->mma);
      }
      if (!mbar_wait(&bars->mma, mma_phase, abort_flag, status, 5)) { ok = false; break; }
      mma_phase ^= 1;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem + lane_off + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(sA + ns_sw_off(row, c * 4 + q)) =
              make_uint4(pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1])),
                         pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])),
                         pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])),
                         pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncthreads();

      // ---- A2 = A A (A symmetric, so A doubles as the K-major B operand).  A's accumulator has been drained to
      // shared memory by every thread (the barrier above), so A2 may take its place.
      if (threadIdx.x == 0) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ss(tmem + A2_COL, ns_desc_k(a_base, ks), ns_desc_k(a_base, ks), idesc_aat, ks > 0 ? 1u : 0u);
        umma_commit(&bars->mma);
      }
      if (!mbar_wait(&bars->mma, mma_phase, abort_flag, status, 5)) { ok = false; break; }
      mma_phase ^= 1;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32], a4[16];
        tmem_ld32(tmem + A2_COL + lane_off + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 av = *reinterpret_cast<const uint4*>(sA + ns_sw_off(row, c * 4 + q));
          a4[4 * q] = av.x; a4[4 * q + 1] = av.y; a4[4 * q + 2] = av.z; a4[4 * q + 3] = av.w;
        }
        uint32_t o[16];
#pragma unroll
        for (int t = 0; t < 16; ++t)
          o[t] = pack_bf16x2(cc * __uint_as_float(v[2 * t]) + cb * bf16_lo(a4[t]),
                             cc * __uint_as_float(v[2 * t + 1]) + cb * bf16_hi(a4[t]));
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(sB + ns_sw_off(row, c * 4 + q)) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncthreads();

      // ---- X' = B X  -> TMEM columns [0,N); X read as an MN-major operand from the same bytes
      if (threadIdx.x == 0) {
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ss(tmem, ns_desc_k(b_base, ks), ns_desc_mn(x_base, ks), idesc_bx, ks > 0 ? 1u : 0u);
        umma_commit(&bars->mma);
      }
      if (!mbar_wait(&bars->mma, mma_phase, abort_flag, status, 5)) { ok = false; break; }
      mma_phase ^= 1;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < NCH * 2; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem + lane_off + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4* ptr = reinterpret_cast<uint4*>(sX + ns_sw_off(row, c * 4 + q));
          const uint4 xv = *ptr;
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
          uint32_t o[4];
#pragma unroll
          for (int t = 0; t < 4; ++t)
            o[t] = pack_bf16x2(round_bf16(__uint_as_float(v[8 * q + 2 * t])) + ca * bf16_lo(xw[t]),
                               round_bf16(__uint_as_float(v[8 * q + 2 * t + 1])) + ca * bf16_hi(xw[t]));
          *ptr = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncthreads();
    }
    if (!ok) break;

    // ---- result rows to global (row-contiguous 16-byte stores)
    if (row < m) {
      __nv_bfloat16* dst = out + (tile * m + row) * static_cast<long long>(N);
#pragma unroll 4
      for (int c = 0; c < NCH * 8; ++c)
        reinterpret_cast<uint4*>(dst)[c] = *reinterpret_cast<const uint4*>(sX + ns_sw_off(row, c));
    }
    fence_proxy_async_smem();
    __syncthreads();   // sX is reloaded by TMA for the next tile
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, TM_COLS);
  }
}

bool ns5_fused_supported(int m, int n) { return m >= 1 && m <= 128 && m <= n && n % 64 == 0 && n >= 64 && n <= 256; }

template <int NCH>
static void launch_ns5(const void* x_in, void* x_out, long long n_tiles, int m, int steps, float eps, cudaStream_t s) {
  constexpr int N = NCH * 64;
  constexpr size_t SMEM = 1024 + (NCH + 2) * NS_HALF + 256;
  constexpr int TM_COLS = N <= 128 ? 128 : 256;
  auto kern = ns5_fused_kernel<NCH>;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM); attr = true; }
  const uint64_t dims[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(m), static_cast<uint64_t>(n_tiles)};
  const uint64_t strides[2] = {static_cast<uint64_t>(N) * 2, static_cast<uint64_t>(N) * 2 * m};
  const uint32_t box[3] = {64, 128, 1};
  const CUtensorMap tm = make_tmap(x_in, 3, dims, strides, box, 2, true);
  // resident CTAs per SM: bounded by shared memory (227 KB, plus 1 KB the driver keeps per CTA) and by TMEM (512 columns)
  const int by_smem = static_cast<int>((227 * 1024) / (SMEM + 1024)), by_tmem = 512 / TM_COLS;
  const int per_sm = by_smem < by_tmem ? by_smem : by_tmem;
  const long long cap = static_cast<long long>(num_sms()) * per_sm;
  const int grid = static_cast<int>(n_tiles < cap ? n_tiles : cap);
  kern<<<grid, 128, SMEM, s>>>(tm, reinterpret_cast<__nv_bfloat16*>(x_out), n_tiles, m, steps, eps, status_word_ptr());
}

void ns5_fused(const void* x_in, void* x_out, long long n_tiles, int m, int n, int steps, float eps, cudaStream_t s) {
  if (n_tiles <= 0) return;
  if (!ns5_fused_supported(m, n)) throw std::runtime_error("himuon ns5_fused: unsupported tile shape");
  switch (n / 64) {
    case 1: launch_ns5<1>(x_in, x_out, n_tiles, m, steps, eps, s); break;
    case 2: launch_ns5<2>(x_in, x_out, n_tiles, m, steps, eps, s); break;
    case 3: launch_ns5<3>(x_in, x_out, n_tiles, m, steps, eps, s); break;
    default: launch_ns5<4>(x_in, x_out, n_tiles, m, steps, eps, s); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("himuon ns5_fused launch failed: ") + cudaGetErrorString(e));
}

}  // namespace himuon
