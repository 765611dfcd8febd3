// HBM-bound model kernels for the decoder (bf16 storage, fp32 math): RMSNorm, per-head
// RMSNorm fused with rotary embedding, SwiGLU, embedding gather / scatter-add and the
// softmax cross-entropy that turns a logits chunk into its gradient in place.
// In the reference these are PyTorch / HF library calls
// (transformers Qwen3/Llama modelling code reached from train.py:123-126).
#include "himuon.h"
#include "sm100_common.cuh"

namespace himuon {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float block_max_f(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    t = warp_max(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// ------------------------------------------------------------------------------------------------ RMSNorm
// One CTA per row; cols % 8 == 0.  y = bf16( bf16(x * rstd) * w )  (HF rounds to the input dtype before the weight).
// With `delta` the row normalised is h = bf16(x + delta) (the residual update), which is also written to `h_out`:
// the residual add and the norm that follows it share one pass.
__device__ __forceinline__ uint4 add_bf16x8(const uint4& a, const uint4& b) {
  const uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
  uint32_t o[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) o[q] = pack_bf16x2(bf16_lo(au[q]) + bf16_lo(bu[q]), bf16_hi(au[q]) + bf16_hi(bu[q]));
  return make_uint4(o[0], o[1], o[2], o[3]);
}
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int cols, float eps,
                   const __nv_bfloat16* __restrict__ delta, __nv_bfloat16* __restrict__ h_out) {
  __shared__ float red[32];
  const int nv = cols >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * cols);
    if (delta != nullptr) {
      const uint4* dr = reinterpret_cast<const uint4*>(delta + static_cast<long long>(r) * cols);
      uint4* hr = reinterpret_cast<uint4*>(h_out + static_cast<long long>(r) * cols);
      for (int i = threadIdx.x; i < nv; i += blockDim.x) hr[i] = add_bf16x8(xr[i], dr[i]);
      xr = hr;                              // each thread re-reads only what it wrote itself
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 v = xr[i];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float a = bf16_lo(u[q]), b = bf16_hi(u[q]); ss += a * a + b * b; }
    }
    const float tot = block_sum_f(ss, red);
    const float rs = rsqrtf(tot / cols + eps);
    if (threadIdx.x == 0 && rstd) rstd[r] = rs;
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<long long>(r) * cols);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 v = xr[i];
      const uint4 ww = wr[i];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
      const uint32_t k[4] = {ww.x, ww.y, ww.z, ww.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        o[q] = pack_bf16x2(round_bf16(bf16_lo(u[q]) * rs) * bf16_lo(k[q]), round_bf16(bf16_hi(u[q]) * rs) * bf16_hi(k[q]));
      yr[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat));  dw += sum_rows dy * xhat  (fp32 atomics into dw_accum).
// Each CTA owns a contiguous slab of rows and keeps its dw partial in registers (cols <= 8*256*kColIters).
constexpr int kNormColIters = 8;
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_accum, int rows, int cols,
                   const __nv_bfloat16* __restrict__ dres) {
  __shared__ float red[32];
  const int nv = cols >> 3;
  float dwp[kNormColIters][8];
#pragma unroll
  for (int a = 0; a < kNormColIters; ++a)
#pragma unroll
    for (int q = 0; q < 8; ++q) dwp[a][q] = 0.f;
  const int rows_per = (rows + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per;
  const int r1 = min(rows, r0 + rows_per);
  for (int r = r0; r < r1; ++r) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<long long>(r) * cols);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    const float rs = rstd[r];
    float dot = 0.f;
#pragma unroll
    for (int a = 0; a < kNormColIters; ++a) {
      const int i = threadIdx.x + a * 256;
      if (i < nv) {
        const uint4 xv = xr[i], gv = gr[i], wv = wr[i];
        const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w}, gu[4] = {gv.x, gv.y, gv.z, gv.w}, wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float xh0 = bf16_lo(xu[q]) * rs, xh1 = bf16_hi(xu[q]) * rs;
          const float g0 = bf16_lo(gu[q]), g1 = bf16_hi(gu[q]);
          dot += g0 * bf16_lo(wu[q]) * xh0 + g1 * bf16_hi(wu[q]) * xh1;
          dwp[a][2 * q] += g0 * xh0;
          dwp[a][2 * q + 1] += g1 * xh1;
        }
      }
    }
    const float mean = block_sum_f(dot, red) / cols;
    uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<long long>(r) * cols);
#pragma unroll
    for (int a = 0; a < kNormColIters; ++a) {
      const int i = threadIdx.x + a * 256;
      if (i < nv) {
        const uint4 xv = xr[i], gv = gr[i], wv = wr[i];
        const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w}, gu[4] = {gv.x, gv.y, gv.z, gv.w}, wu[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float xh0 = bf16_lo(xu[q]) * rs, xh1 = bf16_hi(xu[q]) * rs;
          o[q] = pack_bf16x2(rs * (bf16_lo(gu[q]) * bf16_lo(wu[q]) - xh0 * mean),
                             rs * (bf16_hi(gu[q]) * bf16_hi(wu[q]) - xh1 * mean));
        }
        uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        if (dres != nullptr)                  // gradient arriving on the residual path joins here
          ov = add_bf16x8(ov, reinterpret_cast<const uint4*>(dres + static_cast<long long>(r) * cols)[i]);
        dr[i] = ov;
      }
    }
  }
  if (dw_accum) {
#pragma unroll
    for (int a = 0; a < kNormColIters; ++a) {
      const int i = threadIdx.x + a * 256;
      if (i < nv) {
#pragma unroll
        for (int q = 0; q < 8; ++q) atomicAdd(dw_accum + i * 8 + q, dwp[a][q]);
      }
    }
  }
}

// Warp-per-row variant for hidden sizes up to 5120: a warp keeps its row of x in registers, reduces the dot product
// with shuffles (no block-wide barrier per row) and accumulates its dw contribution in registers over all the rows
// it processes (a lane always owns the same columns); dy is re-read for the second pass (it is still in L1).
// Eight rows are in flight per block; the block flushes dw once through shared memory.
template <int ITERS, bool WITH_DW>      // ITERS * 32 lanes * 8 elements columns at most
__global__ void __launch_bounds__(256)
rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_accum, int rows, int cols,
                        const __nv_bfloat16* __restrict__ dres) {
  extern __shared__ float s_dw[];
  const int nv = cols >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float dwp[ITERS][8];
#pragma unroll
  for (int a = 0; a < ITERS; ++a)
#pragma unroll
    for (int q = 0; q < 8; ++q) dwp[a][q] = 0.f;
  for (int r = blockIdx.x * 8 + warp; r < rows; r += gridDim.x * 8) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<long long>(r) * cols);
    uint4 xv[ITERS];
#pragma unroll
    for (int a = 0; a < ITERS; ++a) {
      const int i = lane + a * 32;
      if (i < nv) xv[a] = xr[i];
    }
    const float rs = rstd[r];
    float dot = 0.f;
#pragma unroll
    for (int a = 0; a < ITERS; ++a) {
      const int i = lane + a * 32;
      if (i < nv) {
        const uint4 wv = wr[i], gv = gr[i];
        const uint32_t xu[4] = {xv[a].x, xv[a].y, xv[a].z, xv[a].w}, gu[4] = {gv.x, gv.y, gv.z, gv.w},
                       wu[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float xh0 = bf16_lo(xu[q]) * rs, xh1 = bf16_hi(xu[q]) * rs;
          const float g0 = bf16_lo(gu[q]), g1 = bf16_hi(gu[q]);
          dot += g0 * bf16_lo(wu[q]) * xh0 + g1 * bf16_hi(wu[q]) * xh1;
          if (WITH_DW) {
            dwp[a][2 * q] += g0 * xh0;
            dwp[a][2 * q + 1] += g1 * xh1;
          }
        }
      }
    }
    const float mean = warp_sum(dot) / cols;
    uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<long long>(r) * cols);
#pragma unroll
    for (int a = 0; a < ITERS; ++a) {
      const int i = lane + a * 32;
      if (i < nv) {
        const uint4 wv = wr[i], gv = gr[i];
        const uint32_t xu[4] = {xv[a].x, xv[a].y, xv[a].z, xv[a].w}, gu[4] = {gv.x, gv.y, gv.z, gv.w},
                       wu[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float xh0 = bf16_lo(xu[q]) * rs, xh1 = bf16_hi(xu[q]) * rs;
          o[q] = pack_bf16x2(rs * (bf16_lo(gu[q]) * bf16_lo(wu[q]) - xh0 * mean),
                             rs * (bf16_hi(gu[q]) * bf16_hi(wu[q]) - xh1 * mean));
        }
        uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        if (dres != nullptr)                  // gradient arriving on the residual path joins here
          ov = add_bf16x8(ov, reinterpret_cast<const uint4*>(dres + static_cast<long long>(r) * cols)[i]);
        dr[i] = ov;
      }
    }
  }
  if (WITH_DW && dw_accum) {
#pragma unroll
    for (int a = 0; a < ITERS; ++a) {
      const int i = lane + a * 32;
      if (i < nv) {
#pragma unroll
        for (int q = 0; q < 8; ++q) atomicAdd(&s_dw[i * 8 + q], dwp[a][q]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < cols; i += blockDim.x) atomicAdd(dw_accum + i, s_dw[i]);
  }
}

// dw of RMSNorm as a column-strip reduction: block (cb, rb) covers 256 columns x `rows_per_block` rows, one warp per
// row at a time (a lane owns 8 adjacent columns), the eight warps meet in shared memory and each strip adds its sums
// with four-wide atomics.  Run next to the warp-per-row dx kernel, it keeps the per-row pass free of dw state
// (fewer registers, more rows in flight) and cuts the atomics per output cache line from thousands to a few hundred.
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dw_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const float* __restrict__ rstd, float* __restrict__ dw_accum, int rows, int cols,
                      int rows_per_block) {
  __shared__ float part[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float acc[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) acc[q] = 0.f;
  if (col < cols) {
#pragma unroll 4
    for (int r = r0 + warp; r < r1; r += 8) {
      const uint4 xv = *reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * cols + col);
      const uint4 gv = *reinterpret_cast<const uint4*>(dy + static_cast<long long>(r) * cols + col);
      const float rs = rstd[r];
      const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w}, gu[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += bf16_lo(gu[q]) * (bf16_lo(xu[q]) * rs);
        acc[2 * q + 1] += bf16_hi(gu[q]) * (bf16_hi(xu[q]) * rs);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) part[warp][lane * 8 + q] = acc[q];
  __syncthreads();
  if (threadIdx.x < 64) {
    const int c = threadIdx.x * 4;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) {
      sum.x += part[w8][c]; sum.y += part[w8][c + 1]; sum.z += part[w8][c + 2]; sum.w += part[w8][c + 3];
    }
    const int gc = blockIdx.x * 256 + c;
    if (gc + 3 < cols) atomicAdd(reinterpret_cast<float4*>(dw_accum + gc), sum);   // cols is a multiple of 8
  }
}

void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps, cudaStream_t s,
                 const void* delta, void* h_out) {
  if (rows <= 0) return;
  if (cols % 8) throw std::runtime_error("himuon rmsnorm: hidden size must be a multiple of 8");
  if ((delta == nullptr) != (h_out == nullptr)) throw std::runtime_error("himuon rmsnorm: delta and h_out go together");
  const int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  rmsnorm_fwd_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
                                          reinterpret_cast<__nv_bfloat16*>(y), rstd, rows, cols, eps,
                                          reinterpret_cast<const __nv_bfloat16*>(delta), reinterpret_cast<__nv_bfloat16*>(h_out));
}
void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_accum, int rows,
                 int cols, cudaStream_t s, const void* dres) {
  auto drp = reinterpret_cast<const __nv_bfloat16*>(dres);
  if (rows <= 0) return;
  if (cols % 8 || cols > 8 * 256 * kNormColIters) throw std::runtime_error("himuon rmsnorm_bwd: unsupported hidden size");
  if (cols <= 20 * 256) {
    const int blocks_needed = (rows + 7) / 8;
    const int grid = blocks_needed < num_sms() ? blocks_needed : num_sms();   // ~240 registers: one block per SM
    const size_t smem = cols * sizeof(float);
    auto dyp = reinterpret_cast<const __nv_bfloat16*>(dy);
    auto xp = reinterpret_cast<const __nv_bfloat16*>(x);
    auto wp = reinterpret_cast<const __nv_bfloat16*>(w);
    auto dxp = reinterpret_cast<__nv_bfloat16*>(dx);
    // dw goes to its own column-strip kernel (when its four-wide atomics are aligned); the row pass then carries none
    float* dw_rows = dw_accum;
    if (dw_accum != nullptr && reinterpret_cast<uintptr_t>(dw_accum) % 16 == 0) {
      const int rpb = 64;
      rmsnorm_bwd_dw_kernel<<<dim3((cols + 255) / 256, (rows + rpb - 1) / rpb), 256, 0, s>>>(dyp, xp, rstd, dw_accum, rows, cols, rpb);
      dw_rows = nullptr;
    }
    const int row_grid = dw_rows ? grid : blocks_needed;
#define HM_RMS_BWD(IT_)                                                                                              \
  if (dw_rows) rmsnorm_bwd_warp_kernel<IT_, true><<<row_grid, 256, smem, s>>>(dyp, xp, wp, rstd, dxp, dw_rows, rows, cols, drp); \
  else rmsnorm_bwd_warp_kernel<IT_, false><<<row_grid, 256, smem, s>>>(dyp, xp, wp, rstd, dxp, nullptr, rows, cols, drp);
    if (cols <= 10 * 256) { HM_RMS_BWD(10) }
    else if (cols <= 16 * 256) { HM_RMS_BWD(16) }
    else { HM_RMS_BWD(20) }
#undef HM_RMS_BWD
    return;
  }
  const int grid = rows < num_sms() * 4 ? rows : num_sms() * 4;
  rmsnorm_bwd_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
                                          reinterpret_cast<const __nv_bfloat16*>(w), rstd, reinterpret_cast<__nv_bfloat16*>(dx),
                                          dw_accum, rows, cols, drp);
}

// ------------------------------------------------------------------------------------------------ head-norm + RoPE
// Per-head RMSNorm (optional) + RoPE on (token, head) vectors of 128 elements.
// cos_sin: (seq_len, 64, 2) fp32.  Rotate-half convention:
//   y[i]      = xn[i]*cos[i] - xn[i+64]*sin[i]
//   y[i+64]   = xn[i+64]*cos[i] + xn[i]*sin[i]
// Layout of the two kernels below: sixteen lanes per head vector, lane l owning elements [8l, 8l+8) (one 16-byte
// access); lanes 0-7 hold the first half, lanes 8-15 the second half, so the rotation partner of every element sits
// at the same register index in lane l^8.  A warp therefore handles two vectors per pass.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z); f[5] = bf16_hi(u.z); f[6] = bf16_lo(u.w); f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

__global__ void __launch_bounds__(256)
headnorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, const float* __restrict__ cos_sin,
                         long long n_vec, int heads, int seq_len, long long ld_in, long long ld_out, float eps,
                         int use_norm) {
  const int sub = threadIdx.x & 15;                       // lane within the half warp
  const bool second = sub >= 8;
  const long long hw0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const long long nhw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  float wv[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) wv[q] = 1.f;
  if (use_norm) unpack8(reinterpret_cast<const uint4*>(w)[sub], wv);
  const long long n_iter = (n_vec + nhw - 1) / nhw;       // the same trip count for every lane (shuffles inside)
  for (long long it = 0; it < n_iter; ++it) {
    const long long vi = hw0 + it * nhw;
    const bool live = vi < n_vec;
    const uint32_t vi32 = live ? static_cast<uint32_t>(vi) : 0u;          // n_vec < 2^31 (checked by the launcher)
    const uint32_t tok = vi32 / static_cast<uint32_t>(heads);
    const int head = static_cast<int>(vi32 - tok * static_cast<uint32_t>(heads));
    const int pos = static_cast<int>(tok % static_cast<uint32_t>(seq_len));
    float xv[8];
    unpack8(reinterpret_cast<const uint4*>(x + static_cast<long long>(tok) * ld_in + head * 128)[sub], xv);
    const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + static_cast<long long>(pos) * 128 + (sub & 7) * 16);
    const float4 c0 = cs4[0], c1 = cs4[1], c2 = cs4[2], c3 = cs4[3];   // (cos, sin) of this lane's eight frequencies
    const float cs[16] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w, c2.x, c2.y, c2.z, c2.w, c3.x, c3.y, c3.z, c3.w};
    if (use_norm) {
      float ss = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) ss += xv[q] * xv[q];
      ss = half_warp_sum(ss);
      const float rs = rsqrtf(ss * (1.f / 128.f) + eps);
      if (sub == 0 && live && rstd) rstd[vi] = rs;
#pragma unroll
      for (int q = 0; q < 8; ++q) xv[q] = round_bf16(round_bf16(xv[q] * rs) * wv[q]);
    }
    float out[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float other = __shfl_xor_sync(0xffffffffu, xv[q], 8);
      out[q] = second ? xv[q] * cs[2 * q] + other * cs[2 * q + 1] : xv[q] * cs[2 * q] - other * cs[2 * q + 1];
    }
    if (live) reinterpret_cast<uint4*>(y + static_cast<long long>(tok) * ld_out + head * 128)[sub] = pack8(out);
  }
}

__global__ void __launch_bounds__(256)
headnorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                         const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                         __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_accum,
                         const float* __restrict__ cos_sin, long long n_vec, int heads, int seq_len, long long ld_dy,
                         long long ld_x, long long ld_dx, int use_norm) {
  __shared__ float sdw[8][128];                         // one row of partial dw per warp
  const int sub = threadIdx.x & 15;
  const bool second = sub >= 8;
  const long long hw0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const long long nhw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 4;
  float wv[8], acc[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) { wv[q] = 1.f; acc[q] = 0.f; }
  if (use_norm) unpack8(reinterpret_cast<const uint4*>(w)[sub], wv);
  const long long n_iter = (n_vec + nhw - 1) / nhw;
  for (long long it = 0; it < n_iter; ++it) {
    const long long vi = hw0 + it * nhw;
    const bool live = vi < n_vec;
    const uint32_t vi32 = live ? static_cast<uint32_t>(vi) : 0u;          // n_vec < 2^31 (checked by the launcher)
    const uint32_t tok = vi32 / static_cast<uint32_t>(heads);
    const int head = static_cast<int>(vi32 - tok * static_cast<uint32_t>(heads));
    const int pos = static_cast<int>(tok % static_cast<uint32_t>(seq_len));
    float g[8];
    unpack8(reinterpret_cast<const uint4*>(dy + static_cast<long long>(tok) * ld_dy + head * 128)[sub], g);
    const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + static_cast<long long>(pos) * 128 + (sub & 7) * 16);
    const float4 c0 = cs4[0], c1 = cs4[1], c2 = cs4[2], c3 = cs4[3];
    const float cs[16] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w, c2.x, c2.y, c2.z, c2.w, c3.x, c3.y, c3.z, c3.w};
    float d[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {                          // transpose of the rotation
      const float other = __shfl_xor_sync(0xffffffffu, g[q], 8);
      d[q] = second ? g[q] * cs[2 * q] - other * cs[2 * q + 1] : g[q] * cs[2 * q] + other * cs[2 * q + 1];
    }
    if (use_norm) {
      float h[8];
      unpack8(reinterpret_cast<const uint4*>(x + static_cast<long long>(tok) * ld_x + head * 128)[sub], h);
      const float rs = live ? rstd[vi] : 0.f;
      float dot = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        h[q] *= rs;
        if (live) acc[q] += d[q] * h[q];
        dot += d[q] * wv[q] * h[q];
      }
      const float mean = half_warp_sum(dot) * (1.f / 128.f);
#pragma unroll
      for (int q = 0; q < 8; ++q) d[q] = rs * (d[q] * wv[q] - h[q] * mean);
    }
    if (live) reinterpret_cast<uint4*>(dx + static_cast<long long>(tok) * ld_dx + head * 128)[sub] = pack8(d);
  }
  if (use_norm && dw_accum) {
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], 16);   // the warp's two half warps
    if ((threadIdx.x & 31) < 16) {
#pragma unroll
      for (int q = 0; q < 8; ++q) sdw[threadIdx.x >> 5][sub * 8 + q] = acc[q];
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) {
        v.x += sdw[w8][4 * threadIdx.x]; v.y += sdw[w8][4 * threadIdx.x + 1];
        v.z += sdw[w8][4 * threadIdx.x + 2]; v.w += sdw[w8][4 * threadIdx.x + 3];
      }
      if (reinterpret_cast<uintptr_t>(dw_accum) % 16 == 0) {
        atomicAdd(reinterpret_cast<float4*>(dw_accum) + threadIdx.x, v);   // 8 atomics per cache line and block
      } else {
        atomicAdd(dw_accum + 4 * threadIdx.x, v.x); atomicAdd(dw_accum + 4 * threadIdx.x + 1, v.y);
        atomicAdd(dw_accum + 4 * threadIdx.x + 2, v.z); atomicAdd(dw_accum + 4 * threadIdx.x + 3, v.w);
      }
    }
  }
}

void headnorm_rope_fwd(const void* x, const void* w, void* y, float* rstd, const float* cos_sin, int tokens, int heads,
                       int seq_len, long long ld_in, long long ld_out, float eps, int use_norm, cudaStream_t s) {
  const long long n_vec = static_cast<long long>(tokens) * heads;
  if (n_vec <= 0) return;
  if (n_vec >= (1LL << 31)) throw std::runtime_error("himuon headnorm_rope: too many head vectors for one launch");
  const long long blocks = (n_vec + 15) / 16;
  const int grid = static_cast<int>(blocks < num_sms() * 8 ? blocks : num_sms() * 8);
  headnorm_rope_fwd_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
                                                reinterpret_cast<__nv_bfloat16*>(y), rstd, cos_sin, n_vec, heads, seq_len,
                                                ld_in, ld_out, eps, use_norm);
}
void headnorm_rope_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_accum,
                       const float* cos_sin, int tokens, int heads, int seq_len, long long ld_dy, long long ld_x,
                       long long ld_dx, int use_norm, cudaStream_t s) {
  const long long n_vec = static_cast<long long>(tokens) * heads;
  if (n_vec <= 0) return;
  if (n_vec >= (1LL << 31)) throw std::runtime_error("himuon headnorm_rope: too many head vectors for one launch");
  const long long blocks = (n_vec + 15) / 16;
  const int grid = static_cast<int>(blocks < num_sms() * 4 ? blocks : num_sms() * 4);
  headnorm_rope_bwd_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
                                                reinterpret_cast<const __nv_bfloat16*>(w), rstd, reinterpret_cast<__nv_bfloat16*>(dx),
                                                dw_accum, cos_sin, n_vec, heads, seq_len, ld_dy, ld_x, ld_dx, use_norm);
}

// ------------------------------------------------------------------------------------------------ SwiGLU
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                  __nv_bfloat16* __restrict__ out, long long rows, int cols, long long ld_g, long long ld_u, long long ld_o) {
  const int vpr = cols >> 3;
  const long long total = rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int c = static_cast<int>(i - r * vpr) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gate + r * ld_g + c);
    const uint4 u = *reinterpret_cast<const uint4*>(up + r * ld_u + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float g0 = bf16_lo(gw[q]), g1 = bf16_hi(gw[q]);
      const float s0 = round_bf16(g0 / (1.f + __expf(-g0))), s1 = round_bf16(g1 / (1.f + __expf(-g1)));
      o[q] = pack_bf16x2(s0 * bf16_lo(uw[q]), s1 * bf16_hi(uw[q]));
    }
    *reinterpret_cast<uint4*>(out + r * ld_o + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gate,
                  const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dup,
                  long long rows, int cols, long long ld_do, long long ld_g, long long ld_u, long long ld_dg, long long ld_du) {
  const int vpr = cols >> 3;
  const long long total = rows * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;
    const int c = static_cast<int>(i - r * vpr) * 8;
    const uint4 d = *reinterpret_cast<const uint4*>(dout + r * ld_do + c);
    const uint4 g = *reinterpret_cast<const uint4*>(gate + r * ld_g + c);
    const uint4 u = *reinterpret_cast<const uint4*>(up + r * ld_u + c);
    const uint32_t dw[4] = {d.x, d.y, d.z, d.w}, gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float gg[2] = {bf16_lo(gw[q]), bf16_hi(gw[q])}, uu[2] = {bf16_lo(uw[q]), bf16_hi(uw[q])}, dd[2] = {bf16_lo(dw[q]), bf16_hi(dw[q])};
      float rg[2], ru[2];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const float sig = 1.f / (1.f + __expf(-gg[t]));
        const float silu = gg[t] * sig;
        ru[t] = dd[t] * silu;
        rg[t] = dd[t] * uu[t] * (sig * (1.f + gg[t] * (1.f - sig)));
      }
      og[q] = pack_bf16x2(rg[0], rg[1]);
      ou[q] = pack_bf16x2(ru[0], ru[1]);
    }
    *reinterpret_cast<uint4*>(dgate + r * ld_dg + c) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dup + r * ld_du + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}
static int ew_grid(long long work_items) {
  const long long blocks = (work_items + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}
void swiglu_fwd(const void* gate, const void* up, void* out, long long rows, int cols, long long ld_g, long long ld_u,
                long long ld_o, cudaStream_t s) {
  if (rows <= 0) return;
  if (cols % 8 || ld_g % 8 || ld_u % 8 || ld_o % 8) throw std::runtime_error("himuon swiglu: sizes must be multiples of 8");
  swiglu_fwd_kernel<<<ew_grid(rows * (cols / 8)), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(gate),
      reinterpret_cast<const __nv_bfloat16*>(up), reinterpret_cast<__nv_bfloat16*>(out), rows, cols, ld_g, ld_u, ld_o);
}
void swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, long long rows, int cols,
                long long ld_do, long long ld_g, long long ld_u, long long ld_dg, long long ld_du, cudaStream_t s) {
  if (rows <= 0) return;
  if (cols % 8 || ld_do % 8 || ld_g % 8 || ld_u % 8 || ld_dg % 8 || ld_du % 8)
    throw std::runtime_error("himuon swiglu: sizes must be multiples of 8");
  swiglu_bwd_kernel<<<ew_grid(rows * (cols / 8)), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
      reinterpret_cast<const __nv_bfloat16*>(gate), reinterpret_cast<const __nv_bfloat16*>(up),
      reinterpret_cast<__nv_bfloat16*>(dgate), reinterpret_cast<__nv_bfloat16*>(dup), rows, cols, ld_do, ld_g, ld_u, ld_dg, ld_du);
}

// ------------------------------------------------------------------------------------------------ embedding
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                     __nv_bfloat16* __restrict__ out, long long tokens, int dim) {
  const int vpr = dim >> 3;
  const long long total = tokens * vpr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vpr;
    const int c = static_cast<int>(i - t * vpr);
    reinterpret_cast<uint4*>(out + t * dim)[c] = reinterpret_cast<const uint4*>(table + ids[t] * dim)[c];
  }
}
template <typename T>
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout, T* __restrict__ dtable,
                     long long tokens, int dim) {
  const int ppr = dim >> 1;
  const long long total = tokens * ppr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / ppr;
    const int c = static_cast<int>(i - t * ppr) * 2;
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(dout + t * dim + c);
    if constexpr (sizeof(T) == 2) {
      atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable + ids[t] * dim + c), g);
    } else {
      atomicAdd(reinterpret_cast<float*>(dtable) + ids[t] * dim + c, __low2float(g));
      atomicAdd(reinterpret_cast<float*>(dtable) + ids[t] * dim + c + 1, __high2float(g));
    }
  }
}
void embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int dim, cudaStream_t s) {
  if (tokens <= 0) return;
  if (dim % 8) throw std::runtime_error("himuon embedding: dim must be a multiple of 8");
  embedding_fwd_kernel<<<ew_grid(tokens * (dim / 8)), 256, 0, s>>>(ids, reinterpret_cast<const __nv_bfloat16*>(table),
                                                                  reinterpret_cast<__nv_bfloat16*>(out), tokens, dim);
}
void embedding_bwd(const long long* ids, const void* dout, void* dtable, long long tokens, int dim, int table_fp32,
                   cudaStream_t s) {
  if (tokens <= 0) return;
  if (table_fp32)
    embedding_bwd_kernel<float><<<ew_grid(tokens * (dim / 2)), 256, 0, s>>>(ids, reinterpret_cast<const __nv_bfloat16*>(dout),
                                                                           reinterpret_cast<float*>(dtable), tokens, dim);
  else
    embedding_bwd_kernel<__nv_bfloat16><<<ew_grid(tokens * (dim / 2)), 256, 0, s>>>(ids, reinterpret_cast<const __nv_bfloat16*>(dout),
                                                                                   reinterpret_cast<__nv_bfloat16*>(dtable), tokens, dim);
}

// ------------------------------------------------------------------------------------------------ cross entropy
// One CTA per row of a (rows, vocab) bf16 logits chunk: online max / sum-exp in pass 1, then the row is
// rewritten as grad_scale * (softmax - onehot) in pass 2 (the re-read is served from L2).
__global__ void __launch_bounds__(1024)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                     float* __restrict__ loss_sum, float* __restrict__ count, float* __restrict__ lse_out,
                     long long rows, int vocab, long long ld, float grad_scale, const float* __restrict__ scale_dev,
                     long long ignore_index) {
  __shared__ float red[32];
  if (scale_dev) grad_scale *= *scale_dev;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    __nv_bfloat16* row = logits + r * ld;
    const long long label = labels[r];
    const bool valid = label != ignore_index;   // uniform over the block
    const bool vec = ((vocab & 7) == 0) && ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
    if (!valid) {
      if (vec) {
        for (int i = threadIdx.x; i < (vocab >> 3); i += blockDim.x) reinterpret_cast<uint4*>(row)[i] = make_uint4(0, 0, 0, 0);
      } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) row[i] = __float2bfloat16_rn(0.f);
      }
      if (threadIdx.x == 0 && lse_out) lse_out[r] = 0.f;
      continue;
    }
    float mx = -INFINITY, sum = 0.f;
    if (vec) {
      for (int i = threadIdx.x; i < (vocab >> 3); i += blockDim.x) {
        const uint4 v = reinterpret_cast<const uint4*>(row)[i];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) { f[2 * q] = bf16_lo(u[q]); f[2 * q + 1] = bf16_hi(u[q]); }
        float lm = f[0];
#pragma unroll
        for (int q = 1; q < 8; ++q) lm = fmaxf(lm, f[q]);
        if (lm > mx) { sum *= __expf(mx - lm); mx = lm; }
#pragma unroll
        for (int q = 0; q < 8; ++q) sum += __expf(f[q] - mx);
      }
    } else {
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float f = __bfloat162float(row[i]);
        if (f > mx) { sum *= __expf(mx - f); mx = f; }
        sum += __expf(f - mx);
      }
    }
    const float gmx = block_max_f(mx, red);
    sum = (mx == -INFINITY) ? 0.f : sum * __expf(mx - gmx);
    const float gsum = block_sum_f(sum, red);
    const float lse = gmx + logf(gsum);
    if (threadIdx.x == 0) {
      const float tgt = __bfloat162float(row[label]);
      atomicAdd(loss_sum, lse - tgt);
      atomicAdd(count, 1.f);
      if (lse_out) lse_out[r] = lse;
    }
    __syncthreads();  // the target logit is read before anyone overwrites it
    if (vec) {
      for (int i = threadIdx.x; i < (vocab >> 3); i += blockDim.x) {
        const uint4 v = reinterpret_cast<const uint4*>(row)[i];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float p0 = __expf(bf16_lo(u[q]) - lse), p1 = __expf(bf16_hi(u[q]) - lse);
          const long long c = static_cast<long long>(i) * 8 + 2 * q;
          if (c == label) p0 -= 1.f;
          if (c + 1 == label) p1 -= 1.f;
          o[q] = pack_bf16x2(p0 * grad_scale, p1 * grad_scale);
        }
        reinterpret_cast<uint4*>(row)[i] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    } else {
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float p = __expf(__bfloat162float(row[i]) - lse);
        if (i == label) p -= 1.f;
        row[i] = __float2bfloat16_rn(p * grad_scale);
      }
    }
    __syncthreads();
  }
}
void cross_entropy_fwd_bwd(void* logits, const long long* labels, float* loss_sum, float* count, float* lse_out,
                           long long rows, int vocab, long long ld, float grad_scale, const float* scale_dev,
                           long long ignore_index, cudaStream_t s) {
  if (rows <= 0) return;
  const long long cap = static_cast<long long>(num_sms()) * 2;
  const int grid = static_cast<int>(rows < cap ? rows : cap);
  cross_entropy_kernel<<<grid, 1024, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(logits), labels, loss_sum, count, lse_out, rows,
                                             vocab, ld, grad_scale, scale_dev, ignore_index);
}

// ------------------------------------------------------------------------------------------------ head-group sum
// out[t, hk, :] = sum_g in[t, hk*G + g, :] for 128-wide heads (gradients of grouped K/V heads).
__global__ void __launch_bounds__(256)
group_sum_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long tokens, int hkv, int G,
                 long long ld_in, long long ld_out) {
  const long long total = tokens * hkv * 16;      // 16 vectors of 8 elements per head
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vec = static_cast<int>(i & 15);
    const long long th = i >> 4;
    const int hk = static_cast<int>(th % hkv);
    const long long t = th / hkv;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int g = 0; g < G; ++g) {
      const uint4 v = *reinterpret_cast<const uint4*>(in + t * ld_in + (hk * G + g) * 128 + vec * 8);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) { acc[2 * q] += bf16_lo(u[q]); acc[2 * q + 1] += bf16_hi(u[q]); }
    }
    *reinterpret_cast<uint4*>(out + t * ld_out + hk * 128 + vec * 8) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}
void group_sum_heads(const void* in, void* out, long long tokens, int hkv, int G, long long ld_in, long long ld_out,
                     cudaStream_t s) {
  if (tokens <= 0) return;
  group_sum_kernel<<<ew_grid(tokens * hkv * 16), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                            reinterpret_cast<__nv_bfloat16*>(out), tokens, hkv, G, ld_in, ld_out);
}

// ------------------------------------------------------------------------------------------------ casts
template <typename S, typename D>
__global__ void cast_copy_kernel(const S* __restrict__ src, D* __restrict__ dst, long long n, float scale) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v;
    if constexpr (sizeof(S) == 2) v = __bfloat162float(src[i]); else v = src[i];
    v *= scale;
    if constexpr (sizeof(D) == 2) dst[i] = __float2bfloat16_rn(v); else dst[i] = v;
  }
}
void cast_copy(const void* src, void* dst, long long n, int src_fp32, int dst_fp32, float scale, cudaStream_t s) {
  if (n <= 0) return;
  const int grid = ew_grid(n);
  if (src_fp32 && dst_fp32) cast_copy_kernel<float, float><<<grid, 256, 0, s>>>((const float*)src, (float*)dst, n, scale);
  else if (src_fp32) cast_copy_kernel<float, __nv_bfloat16><<<grid, 256, 0, s>>>((const float*)src, (__nv_bfloat16*)dst, n, scale);
  else if (dst_fp32) cast_copy_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>((const __nv_bfloat16*)src, (float*)dst, n, scale);
  else cast_copy_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, n, scale);
}
__global__ void bf16_add_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] += __bfloat162float(src[i]);
}
void bf16_add_to_f32(const void* src, float* dst, long long n, cudaStream_t s) {
  if (n <= 0) return;
  bf16_add_to_f32_kernel<<<ew_grid(n), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(src), dst, n);
}

}  // namespace himuon
