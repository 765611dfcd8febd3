// Persistent batched bf16 GEMM for sm_100a:  C[b] = alpha * op(A[b]) * op(B[b]) + beta * Aux[b]
//
//   * operands are staged by TMA (128-byte swizzle, no multicast) into a shared-memory ring,
//   * one elected thread issues tcgen05.mma (M=128, N=BN, K=16) into TMEM accumulators,
//   * four epilogue warps read TMEM with tcgen05.ld, apply the epilogue and store,
//   * two TMEM accumulators (2 x BN columns) let the epilogue of tile i overlap the MMAs of tile i+1.
//
// Either operand may be K-major (reduction dim contiguous) or MN-major (M/N contiguous),
// so forward (x W^T), dgrad (dy W) and wgrad (dy^T x) all run without a transpose pass.
// This one kernel replaces the reference's three Triton GEMM kernels
// (src/himuon/triton_kernels/XXT.py:12-75, ba_plus_cAA.py:12-89, fused_bmm_add.py:12-96)
// and the cuBLAS calls behind F.linear / torch.addmm.
#include "gemm_epilogue.cuh"
#include "himuon.h"
#include "sm100_common.cuh"
#include "tma_host.h"


namespace himuon {

__device__ int g_status_word = 0;

// AUX_TMA (bf16 output with an aux operand): the aux tile arrives by TMA in the very staging slab that its output slab
// leaves from.  Four slabs rotate through load -> combine in place -> store, with the load issued two slabs ahead
// (across tile boundaries), so the epilogue threads never wait on global memory.
template <int BN, int STAGES, bool A_MN, bool B_MN, bool AUX_TMA = false>
__global__ void __launch_bounds__(256, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX, GemmDev p) {
  constexpr int NSTG = AUX_TMA ? 4 : 2;       // staging slabs
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t CHUNK_BYTES = BK * 128;  // one 64-wide MN chunk of an MN-major tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_up_1024(smem_raw);
  uint8_t* sC = smem + STAGES * STAGE_BYTES;                      // two staging slabs for the TMA-store epilogue
  uint64_t* bars = reinterpret_cast<uint64_t*>(sC + NSTG * SLAB_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* aux_full = tempty + 2;            // AUX_TMA: one per staging slab
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_full + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    for (int a = 0; a < 4; ++a) mbar_init(&aux_full[a], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < p.total_items; item += gridDim.x) {
        const WorkItem w = decode_item(p, item);
        const TileCoord tc = decode_tile(p, w.tile, BN / BM);
        const int b = tc.b, mt = tc.mt, nt = tc.nt;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          if (!A_MN) {
            tma_load_3d(sA, &tmA, &full[stage], kb * BK, mt * BM, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sA + j * CHUNK_BYTES, &tmA, &full[stage], mt * BM + j * 64, kb * BK, b);
          }
          if (!B_MN) {
            tma_load_3d(sB, &tmB, &full[stage], kb * BK, nt * BN, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * CHUNK_BYTES, &tmB, &full[stage], nt * BN + j * 64, kb * BK, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < p.total_items; item += gridDim.x) {
        const WorkItem w = decode_item(p, item);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 2)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_smem_desc(a_base + k * 2048, CHUNK_BYTES, 1024)
                                        : umma_smem_desc(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + k * 2048, CHUNK_BYTES, 1024)
                                        : umma_smem_desc(b_base + k * 32, 16, 1024);
            umma_ss(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (warps 4..7 -> TMEM lanes 0..127)
    const int ew = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t slab_seq = 0;
    const bool issuer = (threadIdx.x == 128);
    if (issuer && p.tma_store) tma_prefetch_desc(&tmC);
    if constexpr (AUX_TMA) {
      constexpr int SW = 64, SLABS = BN / SW;
      const int row_in_tile = ew * 32 + lane;
      // Prefetch cursor (issuer only): the (tile, slab) pairs of this CTA in the order the epilogue visits them.
      int pf_item = blockIdx.x, pf_sl = 0;
      uint32_t pf_seq = 0;
      auto prefetch_next = [&]() {
        while (pf_item < p.total_items) {
          const TileCoord tc = decode_tile(p, pf_item, BN / BM);
          const int b = tc.b, mt = tc.mt, nt = tc.nt;
          const int col = nt * BN + pf_sl * SW;
          if (col < p.N) {
            const uint32_t buf = pf_seq & 3;
            mbar_expect_tx(&aux_full[buf], SLAB_BYTES);
            tma_load_3d(sC + buf * SLAB_BYTES, &tmX, &aux_full[buf], col, mt * BM, b);
            ++pf_seq;
            if (++pf_sl == SLABS) { pf_sl = 0; pf_item += gridDim.x; }
            return;
          }
          pf_sl = 0;                         // the rest of this tile lies past N
          pf_item += gridDim.x;
        }
      };
      if (issuer) {
        tma_prefetch_desc(&tmX);
        prefetch_next();
        prefetch_next();
      }
      uint32_t g = 0;                        // slabs finished by this CTA
      bool ok = true;
      for (int item = blockIdx.x; ok && item < p.total_items; item += gridDim.x) {
        const TileCoord tc = decode_tile(p, item, BN / BM);
        const int b = tc.b, mt = tc.mt, nt = tc.nt;
        __nv_bfloat16* mirror_c = tc.mirror ? reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(b) * p.strideC : nullptr;
        if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 3)) break;
        tc_fence_after();
        const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
        for (int sl = 0; sl < SLABS; ++sl) {
          const int col = nt * BN + sl * SW;
          if (col >= p.N) break;             // uniform over the 128 threads
          const uint32_t buf = g & 3;
          uint8_t* my_row = sC + buf * SLAB_BYTES + row_in_tile * 128;
          if (!mbar_wait(&aux_full[buf], (g >> 2) & 1, abort_flag, p.status, 5)) { ok = false; break; }
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t v[32];
            tmem_ld32(t_acc + sl * SW + ch * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4* cell = reinterpret_cast<uint4*>(my_row + (((ch * 4 + q) ^ (row_in_tile & 7)) << 4));
              const uint4 e = *cell;
              const uint32_t ew4[4] = {e.x, e.y, e.z, e.w};
              uint32_t o[4];
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                float f0 = p.alpha * __uint_as_float(v[8 * q + 2 * t]);
                float f1 = p.alpha * __uint_as_float(v[8 * q + 2 * t + 1]);
                if (p.round_acc) { f0 = round_bf16(f0); f1 = round_bf16(f1); }
                o[t] = pack_bf16x2(f0 + p.beta * bf16_lo(ew4[t]), f1 + p.beta * bf16_hi(ew4[t]));
              }
              *cell = make_uint4(o[0], o[1], o[2], o[3]);
              if (mirror_c != nullptr) mirror_store8(mirror_c, p.ldc, col + (ch * 4 + q) * 8, mt * BM + row_in_tile, p.N, o);
            }
          }
          fence_proxy_async_smem();
          named_barrier(1, 128);             // the whole slab is combined
          if (issuer) {
            tma_store_3d(&tmC, sC + buf * SLAB_BYTES, col, mt * BM, b);
            tma_store_commit();
            tma_store_wait_read<1>();        // the slab stored before this one is drained: its buffer takes slab g+2
            prefetch_next();
          }
          ++g;
        }
        if (!ok) break;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      if (issuer) tma_store_wait_read<0>();
    } else
    for (int item = blockIdx.x; item < p.total_items; item += gridDim.x) {
      const WorkItem w = decode_item(p, item);
      const TileCoord tc = decode_tile(p, w.tile, BN / BM);
      const int b = tc.b, mt = tc.mt, nt = tc.nt;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 3)) break;
      tc_fence_after();
      if (p.tma_store) {
        const int row_in_tile = ew * 32 + lane;
        const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + static_cast<uint32_t>(acc * BN);
        const long long aux_row = static_cast<long long>(b) * p.strideAux + static_cast<long long>(mt * BM + row_in_tile) * p.ldaux;
        if (p.out_fp32)
          epilogue_tile_tma<BN, true>(&tmC, sC, t_acc, row_in_tile, mt * BM, nt * BN, b, p.aux, aux_row, p.M, p.N,
                                      p.alpha, p.beta, p.round_acc, slab_seq, issuer);
        else
          epilogue_tile_tma<BN, false>(&tmC, sC, t_acc, row_in_tile, mt * BM, nt * BN, b, p.aux, aux_row, p.M, p.N,
                                       p.alpha, p.beta, p.round_acc, slab_seq, issuer, false,
                                       tc.mirror ? reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(b) * p.strideC : nullptr,
                                       p.ldc);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      }
      const int row = mt * BM + ew * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + static_cast<uint32_t>(acc * BN);
      const long long c_off = static_cast<long long>(b) * p.strideC + static_cast<long long>(row) * p.ldc;
      const long long x_off = static_cast<long long>(b) * p.strideAux + static_cast<long long>(row) * p.ldaux;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col = nt * BN + c0;
        if (col >= p.N) break;  // uniform over the warp
        uint32_t v[32];
        __syncwarp();
        tmem_ld32(t_row + c0, v);
        tmem_ld_wait();
        const bool full_vec = (col + 32 <= p.N);
        if (!row_ok) {
          // rows past M hold padding; nothing to store
        } else if (p.out_fp32) {
          float* cp = reinterpret_cast<float*>(p.C) + c_off + col;
          const float* xp = p.aux ? reinterpret_cast<const float*>(p.aux) + x_off + col : nullptr;
          if (full_vec && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0) &&
              (!xp || (reinterpret_cast<uintptr_t>(xp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 o;
              o.x = p.alpha * __uint_as_float(v[j + 0]);
              o.y = p.alpha * __uint_as_float(v[j + 1]);
              o.z = p.alpha * __uint_as_float(v[j + 2]);
              o.w = p.alpha * __uint_as_float(v[j + 3]);
              if (xp) {
                const float4 e = *reinterpret_cast<const float4*>(xp + j);
                o.x += p.beta * e.x; o.y += p.beta * e.y; o.z += p.beta * e.z; o.w += p.beta * e.w;
              }
              *reinterpret_cast<float4*>(cp + j) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < p.N) {
                float o = p.alpha * __uint_as_float(v[j]);
                if (xp) o += p.beta * xp[j];
                cp[j] = o;
              }
            }
          }
        } else {
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + col;
          const __nv_bfloat16* xp = p.aux ? reinterpret_cast<const __nv_bfloat16*>(p.aux) + x_off + col : nullptr;
          if (full_vec && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0) &&
              (!xp || (reinterpret_cast<uintptr_t>(xp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float f[8];
#pragma unroll
              for (int t = 0; t < 8; ++t) f[t] = p.alpha * __uint_as_float(v[j + t]);
              if (xp) {
                const uint4 e = *reinterpret_cast<const uint4*>(xp + j);
                const uint32_t ew4[4] = {e.x, e.y, e.z, e.w};
                if (p.round_acc) {
#pragma unroll
                  for (int t = 0; t < 8; ++t) f[t] = round_bf16(f[t]);
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  f[2 * t] += p.beta * bf16_lo(ew4[t]);
                  f[2 * t + 1] += p.beta * bf16_hi(ew4[t]);
                }
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(cp + j) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < p.N) {
                float o = p.alpha * __uint_as_float(v[j]);
                if (xp) {
                  if (p.round_acc) o = round_bf16(o);
                  o += p.beta * __bfloat162float(xp[j]);
                }
                cp[j] = __float2bfloat16_rn(o);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (!AUX_TMA && issuer && p.tma_store) tma_store_wait_read<0>();   // no store may still be reading shared memory at exit
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// bf16 output with a bf16 aux tile that TMA can fetch (16-byte aligned base, rows and batches)
static bool aux_tma_ok(const GemmArgs& a) {
  return a.aux != nullptr && !a.out_fp32 && a.ldaux % 8 == 0 && (a.batch == 1 || a.strideAux % 8 == 0) &&
         reinterpret_cast<uintptr_t>(a.aux) % 16 == 0 && a.ldc % 8 == 0 && (a.batch == 1 || a.strideC % 8 == 0) &&
         reinterpret_cast<uintptr_t>(a.C) % 16 == 0;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool AUX_TMA = false>
static void launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  constexpr uint32_t STAGE_BYTES = (BM + BN) * BK * 2;
  constexpr size_t SMEM = 1024 + STAGES * STAGE_BYTES + (AUX_TMA ? 4 : 2) * SLAB_BYTES + 256;
  static_assert(SMEM <= 232448, "shared memory budget of one CTA exceeded");
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, AUX_TMA>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM));
    attr_done = true;
  }
  // A: K-major storage (M rows x K) or MN-major storage (K rows x M).
  uint64_t dimsA[3], strA[2], dimsB[3], strB[2];
  uint32_t boxA[3], boxB[3];
  if (!A_MN) { dimsA[0] = a.K; dimsA[1] = a.M; boxA[0] = BK; boxA[1] = BM; }
  else       { dimsA[0] = a.M; dimsA[1] = a.K; boxA[0] = 64; boxA[1] = BK; }
  dimsA[2] = a.batch; boxA[2] = 1;
  strA[0] = static_cast<uint64_t>(a.lda) * 2;
  strA[1] = a.batch > 1 ? static_cast<uint64_t>(a.strideA) * 2 : strA[0] * dimsA[1];
  if (!B_MN) { dimsB[0] = a.K; dimsB[1] = a.N; boxB[0] = BK; boxB[1] = BN; }
  else       { dimsB[0] = a.N; dimsB[1] = a.K; boxB[0] = 64; boxB[1] = BK; }
  dimsB[2] = a.batch; boxB[2] = 1;
  strB[0] = static_cast<uint64_t>(a.ldb) * 2;
  strB[1] = a.batch > 1 ? static_cast<uint64_t>(a.strideB) * 2 : strB[0] * dimsB[1];
  CUtensorMap tmA = make_tmap(a.A, 3, dimsA, strA, boxA, 2, true);
  CUtensorMap tmB = make_tmap(a.B, 3, dimsB, strB, boxB, 2, true);

  GemmDev p{};
  p.C = a.C; p.aux = a.aux;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
  p.ldc = a.ldc; p.ldaux = a.ldaux; p.strideC = a.strideC; p.strideAux = a.strideAux;
  p.alpha = a.alpha; p.beta = a.beta; p.out_fp32 = a.out_fp32; p.round_acc = a.round_acc;
  p.tiles_m = (a.M + BM - 1) / BM;
  p.tiles_n = (a.N + BN - 1) / BN;
  p.kblocks = (a.K + BK - 1) / BK;
  p.status = status_word_ptr();
  // C tensor map for the TMA-store epilogue: rows of 128 bytes (64 bf16 / 32 fp32 columns) per slab.
  const int esz = a.out_fp32 ? 4 : 2;
  const int row_align = 16 / esz;
  p.tma_store = (a.ldc % row_align == 0) && (a.batch == 1 || a.strideC % row_align == 0) &&
                (reinterpret_cast<uintptr_t>(a.C) % 16 == 0) ? 1 : 0;
  CUtensorMap tmC = tmA;
  if (p.tma_store) {
    const uint64_t dimsC[3] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.batch)};
    const uint64_t strC[2] = {static_cast<uint64_t>(a.ldc) * esz,
                              a.batch > 1 ? static_cast<uint64_t>(a.strideC) * esz : static_cast<uint64_t>(a.ldc) * esz * a.M};
    const uint32_t boxC[3] = {static_cast<uint32_t>(128 / esz), BM, 1};
    tmC = make_tmap(a.C, 3, dimsC, strC, boxC, esz, true);
  }
  CUtensorMap tmX = tmC;
  if (AUX_TMA) {
    const uint64_t dimsX[3] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.batch)};
    const uint64_t strX[2] = {static_cast<uint64_t>(a.ldaux) * 2,
                              a.batch > 1 ? static_cast<uint64_t>(a.strideAux) * 2 : static_cast<uint64_t>(a.ldaux) * 2 * a.M};
    const uint32_t boxX[3] = {64, BM, 1};
    tmX = make_tmap(a.aux, 3, dimsX, strX, boxX, 2, true);
  }
  long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * a.batch;
  // Symmetric output: needs square bf16 C reachable by TMA stores and a tile width that is a whole number of tile
  // heights; otherwise every tile is computed (same result).
  p.sym = (a.symmetric && a.M == a.N && !a.out_fp32 && p.tma_store && BN % BM == 0 && p.tiles_n > 1) ? 1 : 0;
  p.sym_tiles = 0;
  if (p.sym) {
    for (int nt = 0; nt < p.tiles_n; ++nt) p.sym_tiles += p.tiles_m - nt * (BN / BM);
    total = static_cast<long long>(p.sym_tiles) * a.batch;
  }
  int sms = a.max_ctas > 0 ? a.max_ctas : num_sms();
  p.full_items = p.total_items = static_cast<int>(total);
  p.nslices = 1;
  const int grid = static_cast<int>(p.total_items < sms ? p.total_items : sms);
  kern<<<grid, 256, SMEM, stream>>>(tmA, tmB, tmC, tmX, p);
}

int num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (sms[dev] == 0) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev];
}

void gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.batch <= 0) return;
  if (a.K <= 0) throw std::runtime_error("himuon gemm: K must be positive");
  if (gemm2_supported(a)) {
    gemm2_bf16(a, stream);
    return;
  }
  // Tile width.  The main loop is bound by L2 -> shared-memory traffic, so the widest tile (highest arithmetic
  // intensity) wins even when it costs an extra partial wave; narrow tiles are only for narrow outputs.
  const int best_bn = a.N <= 128 ? 128 : (a.N <= 192 ? 192 : 256);
  const int sel = (a.a_mn ? 2 : 0) | (a.b_mn ? 1 : 0);
#define HM_LAUNCH(BN_, ST_)                                                        \
  switch (sel) {                                                                   \
    case 0: launch_gemm<BN_, ST_, false, false>(a, stream); break;                 \
    case 1: launch_gemm<BN_, ST_, false, true>(a, stream); break;                  \
    case 2: launch_gemm<BN_, ST_, true, false>(a, stream); break;                  \
    default: launch_gemm<BN_, ST_, true, true>(a, stream); break;                  \
  }
  if (best_bn == 256 && aux_tma_ok(a)) {
    switch (sel) {
      case 0: launch_gemm<256, 3, false, false, true>(a, stream); break;
      case 1: launch_gemm<256, 3, false, true, true>(a, stream); break;
      case 2: launch_gemm<256, 3, true, false, true>(a, stream); break;
      default: launch_gemm<256, 3, true, true, true>(a, stream); break;
    }
  } else if (best_bn == 128) { HM_LAUNCH(128, 6) }
  else if (best_bn == 192) { HM_LAUNCH(192, 4) }
  else { HM_LAUNCH(256, 4) }
#undef HM_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("himuon gemm launch failed: ") + cudaGetErrorString(e));
}

int* status_word_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess)
      throw std::runtime_error("himuon: cannot resolve the device status word");
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

int read_status_word(bool reset) {
  int v = 0;
  cudaMemcpy(&v, status_word_ptr(), sizeof(int), cudaMemcpyDeviceToHost);
  if (reset && v != 0) cudaMemset(status_word_ptr(), 0, sizeof(int));
  return v;
}

}  // namespace himuon
