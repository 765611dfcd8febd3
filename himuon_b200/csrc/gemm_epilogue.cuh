// Pieces shared by the one-CTA and the CTA-pair GEMM kernels: launch parameters, the work-item decoder and the
// TMA-store epilogue (TMEM -> registers -> fused epilogue -> swizzled shared-memory slab -> bulk tensor store).
#pragma once

#include "himuon.h"
#include "sm100_common.cuh"

namespace himuon {

struct GemmDev {
  void* C;
  const void* aux;
  int M, N, K, batch;
  long long ldc, ldaux, strideC, strideAux;
  float alpha, beta;
  int out_fp32;     // 1: C/aux are fp32, 0: bf16
  int round_acc;    // 1: round alpha*acc to bf16 before adding beta*aux
  int tiles_m, tiles_n, kblocks;
  int tma_store;    // 1: epilogue goes through shared-memory slabs and TMA stores (needs 16-byte aligned C rows)
  // Work list: items [0, full_items) are whole tiles; in the pair kernel each tile of a mostly empty last wave is cut
  // into `nslices` K-ranges, one item each, whose fp32 partial sums meet in a scratch tile.
  int full_items, total_items, nslices;
  int reduce_out;   // pair kernel, C += alpha*acc (aux == C, beta == 1; fp32 or bf16): tiles add into C with TMA reductions
  int stream_k;     // with reduce_out: every CTA pair takes an equal, contiguous range of (tile, k-block) units and
                    // adds each partial tile into C, so no wave of tiles is left partly idle
  // Symmetric output (C = C^T by construction: X X^T, c A A + b A with A symmetric; one-CTA kernel, bf16 out):
  // tiles that lie entirely above the diagonal are not computed; tiles entirely below it are also stored transposed.
  int sym;          // 1: symmetric mode
  int sym_tiles;    // computed tiles per batch entry
  int* status;
};

// Tile coordinates of work item `tile`.  In symmetric mode (tile width BN = R * BM) column block nt keeps the row
// blocks mt >= nt*R, enumerated mt-fastest; a tile with mt >= (nt+1)*R has no entry on or above the diagonal and
// its transpose covers exactly entries of tiles that were dropped.
struct TileCoord { int b, mt, nt; bool mirror; };
__device__ __forceinline__ TileCoord decode_tile(const GemmDev& p, int tile, int R) {
  TileCoord t;
  if (!p.sym) {
    const int per = p.tiles_m * p.tiles_n;
    t.b = tile / per;
    const int r = tile - t.b * per;
    t.mt = r % p.tiles_m;
    t.nt = r / p.tiles_m;
    t.mirror = false;
    return t;
  }
  t.b = tile / p.sym_tiles;
  int k = tile - t.b * p.sym_tiles;
  int nt = 0;
  for (;;) {
    const int cnt = p.tiles_m - nt * R;
    if (k < cnt || nt + 1 >= p.tiles_n) break;
    k -= cnt;
    ++nt;
  }
  t.nt = nt;
  t.mt = nt * R + k;
  t.mirror = t.mt >= (nt + 1) * R;
  return t;
}

// Transposed store of eight consecutive bf16 columns of one tile row: element j goes to C[row0 + j][col] (rows and
// col bounded by n).  The 32 lanes of a warp hold 32 consecutive `col`s, so each store instruction writes 64
// contiguous bytes.
__device__ __forceinline__ void mirror_store8(__nv_bfloat16* C, long long ldc, int row0, int col, int n,
                                              const uint32_t (&o)[4]) {
  if (col >= n) return;
  unsigned short* base = reinterpret_cast<unsigned short*>(C) + static_cast<long long>(row0) * ldc + col;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    if (row0 + 2 * t < n) base[static_cast<long long>(2 * t) * ldc] = static_cast<unsigned short>(o[t] & 0xFFFFu);
    if (row0 + 2 * t + 1 < n) base[static_cast<long long>(2 * t + 1) * ldc] = static_cast<unsigned short>(o[t] >> 16);
  }
}

struct WorkItem { int tile, kb0, kb1, slice, tail; bool split; };
__device__ __forceinline__ WorkItem decode_item(const GemmDev& p, int item) {
  WorkItem w;
  if (item < p.full_items) {
    w.tile = item; w.kb0 = 0; w.kb1 = p.kblocks; w.slice = 0; w.tail = 0; w.split = false;
  } else {
    const int t = item - p.full_items;
    w.tail = t / p.nslices;
    w.slice = t - w.tail * p.nslices;
    w.tile = p.full_items + w.tail;
    w.kb0 = static_cast<int>(static_cast<long long>(p.kblocks) * w.slice / p.nslices);
    w.kb1 = static_cast<int>(static_cast<long long>(p.kblocks) * (w.slice + 1) / p.nslices);
    w.split = true;
  }
  return w;
}

// Walks the work of one CTA (pair): either items first, first+stride, ... of the item list, or (stream_k) the
// contiguous share [total*first/stride, total*(first+1)/stride) of all (tile, k-block) units, cut at tile boundaries.
struct WorkCursor {
  const GemmDev& p;
  int item, stride;
  long long u, u1;
  __device__ __forceinline__ WorkCursor(const GemmDev& p_, int first, int stride_) : p(p_), item(first), stride(stride_), u(0), u1(0) {
    if (p.stream_k) {
      const long long total = static_cast<long long>(p.full_items) * p.kblocks;
      u = total * first / stride_;
      u1 = total * (first + 1) / stride_;
    }
  }
  __device__ __forceinline__ bool next(WorkItem& w) {
    if (p.stream_k) {
      if (u >= u1) return false;
      const int tile = static_cast<int>(u / p.kblocks);
      const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * p.kblocks);
      int len = p.kblocks - kb0;
      if (len > u1 - u) len = static_cast<int>(u1 - u);
      w.tile = tile; w.kb0 = kb0; w.kb1 = kb0 + len; w.slice = 0; w.tail = 0; w.split = false;
      u += len;
      return true;
    }
    if (item >= p.total_items) return false;
    w = decode_item(p, item);
    item += stride;
    return true;
  }
};

constexpr int BM = 128;
constexpr int BK = 64;
constexpr uint32_t SLAB_BYTES = BM * 128;   // one staging slab: 128 rows x 128 bytes (64 bf16 or 32 fp32 columns)

// Loads the 128 bytes of `aux` that belong to this thread's row of a slab (zeros when there is no aux).
template <bool OUT_FP32>
__device__ __forceinline__ void load_aux_slab(const void* aux, long long elem_off, bool row_ok, int valid_cols,
                                              uint4 (&x)[8]) {
  constexpr int SW = OUT_FP32 ? 32 : 64;
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = make_uint4(0, 0, 0, 0);
  if (aux == nullptr || !row_ok || valid_cols <= 0) return;
  if (OUT_FP32) {
    const float* ptr = reinterpret_cast<const float*>(aux) + elem_off;
    if (valid_cols >= SW && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = reinterpret_cast<const uint4*>(ptr)[j];
    } else {
      uint32_t* w = reinterpret_cast<uint32_t*>(x);
#pragma unroll
      for (int j = 0; j < 32; ++j) if (j < valid_cols) w[j] = __float_as_uint(ptr[j]);
    }
  } else {
    const __nv_bfloat16* ptr = reinterpret_cast<const __nv_bfloat16*>(aux) + elem_off;
    if (valid_cols >= SW && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = reinterpret_cast<const uint4*>(ptr)[j];
    } else {
      uint32_t* w = reinterpret_cast<uint32_t*>(x);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float lo = (2 * j < valid_cols) ? __bfloat162float(ptr[2 * j]) : 0.f;
        const float hi = (2 * j + 1 < valid_cols) ? __bfloat162float(ptr[2 * j + 1]) : 0.f;
        w[j] = pack_bf16x2(lo, hi);
      }
    }
  }
}

// Epilogue of one accumulator tile through swizzled shared-memory slabs and TMA stores.  Called by the 128
// epilogue threads together.  `slab_seq` numbers the slabs this CTA has stored so far (selects the staging buffer).
template <int BN, bool OUT_FP32>
__device__ __forceinline__ void epilogue_tile_tma(const CUtensorMap* tmC, uint8_t* sC, uint32_t t_row, int row_in_tile,
                                                  int m0, int n0, int b, const void* aux, long long aux_row_off,
                                                  int M, int N, float alpha, float beta, int round_acc,
                                                  uint32_t& slab_seq, bool issuer, bool reduce_add = false,
                                                  __nv_bfloat16* mirror_c = nullptr, long long mirror_ld = 0) {
  constexpr int SW = OUT_FP32 ? 32 : 64;
  constexpr int SLABS = BN / SW;
  const bool row_ok = (m0 + row_in_tile) < M;
  uint4 xa[8], xn[8];
  load_aux_slab<OUT_FP32>(aux, aux_row_off + n0, row_ok, N - n0, xa);
#pragma unroll 1
  for (int sl = 0; sl < SLABS; ++sl) {
    const int col = n0 + sl * SW;
    if (col >= N) break;                                   // uniform over the 128 threads
    if (sl + 1 < SLABS) load_aux_slab<OUT_FP32>(aux, aux_row_off + col + SW, row_ok, N - col - SW, xn);
    named_barrier(1, 128);                                 // the staging buffer is free (issuer waited on its reads)
    uint8_t* buf = sC + (slab_seq & 1) * SLAB_BYTES;
    uint8_t* my_row = buf + row_in_tile * 128;
#pragma unroll
    for (int ch = 0; ch < SW / 32; ++ch) {
      uint32_t v[32];
      tmem_ld32(t_row + sl * SW + ch * 32, v);
      tmem_ld_wait();
      if (OUT_FP32) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o;
          o.x = alpha * __uint_as_float(v[4 * j + 0]) + beta * __uint_as_float(xa[j].x);
          o.y = alpha * __uint_as_float(v[4 * j + 1]) + beta * __uint_as_float(xa[j].y);
          o.z = alpha * __uint_as_float(v[4 * j + 2]) + beta * __uint_as_float(xa[j].z);
          o.w = alpha * __uint_as_float(v[4 * j + 3]) + beta * __uint_as_float(xa[j].w);
          *reinterpret_cast<float4*>(my_row + ((j ^ (row_in_tile & 7)) << 4)) = o;
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 e = xa[ch * 4 + q];
          const uint32_t ew[4] = {e.x, e.y, e.z, e.w};
          uint32_t o[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            float f0 = alpha * __uint_as_float(v[8 * q + 2 * t]);
            float f1 = alpha * __uint_as_float(v[8 * q + 2 * t + 1]);
            if (round_acc) { f0 = round_bf16(f0); f1 = round_bf16(f1); }
            o[t] = pack_bf16x2(f0 + beta * bf16_lo(ew[t]), f1 + beta * bf16_hi(ew[t]));
          }
          const int j = ch * 4 + q;
          *reinterpret_cast<uint4*>(my_row + ((j ^ (row_in_tile & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          if (mirror_c != nullptr) mirror_store8(mirror_c, mirror_ld, col + j * 8, m0 + row_in_tile, N, o);
        }
      }
    }
    fence_proxy_async_smem();
    named_barrier(2, 128);                                 // the slab is complete
    if (issuer) {
      if (reduce_add) tma_reduce_add_3d(tmC, buf, col, m0, b);     // split-K: accumulate into the fp32 scratch tile
      else tma_store_3d(tmC, buf, col, m0, b);
      tma_store_commit();
      tma_store_wait_read<1>();                            // the other buffer's previous store has drained
    }
    ++slab_seq;
#pragma unroll
    for (int j = 0; j < 8; ++j) xa[j] = xn[j];
  }
}

}  // namespace himuon
