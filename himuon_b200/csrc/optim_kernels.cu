// Multi-tensor optimizer kernels (HBM-bound): each runs ONE launch over every matrix of a
// bucket, driven by a device-resident entry table.
//
//   momentum_tile : sum of gradient replicas (this rank's and, under sharding, the peers' through
//                   peer pointers) -> scale -> momentum update -> Nesterov -> zero-padded tile layout
//                   (the reference's separate launches: src/himuon/optimizers/himuon.py:350-357, 713-719)
//   ns_normalize  : per-tile Frobenius normalisation (himuon.py:241 / triton_kernels/ns5_smem.py:84-88)
//   untile_apply  : untile + crop + lr-scale + decoupled weight decay + parameter update
//                   (himuon.py:315-348, 215-228) with lr / wd read from a device table, so a captured
//                   CUDA graph follows the LR schedule without recapture
//   adamw_multi   : the three AdamW conventions used by the optimizers (himuon.py:359-372,
//                   muon.py:171-193, adamw.py:86-116)
#include "himuon.h"
#include "sm100_common.cuh"

namespace himuon {

constexpr int kRowsPerUnit = 16;

int momentum_tile_units(int R, int C, int Th) { return R * C * ((Th + kRowsPerUnit - 1) / kRowsPerUnit); }

template <typename Entry>
__device__ __forceinline__ int find_entry(const Entry* e, int n, long long unit) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (static_cast<long long>(e[mid].unit_begin) <= unit) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ------------------------------------------------------------------------------------------------
template <typename G>
__global__ void __launch_bounds__(256)
momentum_tile_kernel(const MomTileEntry* __restrict__ entries, int n_entries, int total_units, int Th, int Tw,
                     __nv_bfloat16* __restrict__ tiles, float mu, int nesterov, float gscale, int n_src) {
  const int row_blocks = (Th + kRowsPerUnit - 1) / kRowsPerUnit;
  for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
    const int ei = find_entry(entries, n_entries, unit);
    const MomTileEntry e = entries[ei];
    const int local = unit - e.unit_begin;
    const int t = local / row_blocks;
    const int rb = local - t * row_blocks;
    const int tr = t / e.C, tc = t - tr * e.C;
    __nv_bfloat16* out = tiles + (e.tile_base + t) * static_cast<long long>(Th) * Tw;
    G* mom = reinterpret_cast<G*>(e.mom);
    const int i0 = rb * kRowsPerUnit;
    const int i1 = min(Th, i0 + kRowsPerUnit);
    const bool vec = (sizeof(G) == 2) && (Tw % 8 == 0) && (e.ld % 8 == 0) && (e.w % 8 == 0);
    if (vec) {
      const int vec_per_row = Tw / 8;
      const int nvec = (i1 - i0) * vec_per_row;
      // two vectors per thread and pass, their loads issued together
      for (int x0 = threadIdx.x; x0 < nvec; x0 += 2 * blockDim.x) {
        int xs[2] = {x0, x0 + static_cast<int>(blockDim.x)};
        bool live[2], inside[2];
        int ii[2], jj[2];
        long long off[2], moff[2];
        float g[2][8];
        uint4 mv[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          live[u] = xs[u] < nvec;
          ii[u] = i0 + xs[u] / vec_per_row;
          jj[u] = (xs[u] % vec_per_row) * 8;
          const int gi = tr * Th + ii[u], gj = tc * Tw + jj[u];
          inside[u] = live[u] && gi < e.h && gj < e.w;
          off[u] = static_cast<long long>(gi) * e.ld + gj;
          moff[u] = static_cast<long long>(gi) * e.w + gj;
#pragma unroll
          for (int q = 0; q < 8; ++q) g[u][q] = 0.f;
          mv[u] = make_uint4(0, 0, 0, 0);
          if (inside[u]) mv[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(mom) + moff[u]);
        }
        for (int sidx = 0; sidx < n_src; ++sidx) {
          uint4 gv[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
#pragma unroll
          for (int u = 0; u < 2; ++u)
            if (inside[u]) gv[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e.grad[sidx]) + off[u]);
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const uint32_t gw[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) { g[u][2 * q] += bf16_lo(gw[q]); g[u][2 * q + 1] += bf16_hi(gw[q]); }
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (!live[u]) continue;
          uint4 o = make_uint4(0, 0, 0, 0);
          if (inside[u]) {
            const uint32_t mw[4] = {mv[u].x, mv[u].y, mv[u].z, mv[u].w};
            float r[8], m[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) { m[2 * q] = bf16_lo(mw[q]); m[2 * q + 1] = bf16_hi(mw[q]); }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              // the gradient as the optimizer would see it (stored precision), then buf = mu*buf + g
              const float gq = round_bf16(g[u][q] * gscale);
              const float bq = round_bf16(round_bf16(m[q] * mu) + gq);
              m[q] = bq;
              r[q] = nesterov ? round_bf16(gq + mu * bq) : bq;
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(mom) + moff[u]) =
                make_uint4(pack_bf16x2(m[0], m[1]), pack_bf16x2(m[2], m[3]), pack_bf16x2(m[4], m[5]), pack_bf16x2(m[6], m[7]));
            o = make_uint4(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]), pack_bf16x2(r[4], r[5]), pack_bf16x2(r[6], r[7]));
          }
          *reinterpret_cast<uint4*>(out + static_cast<long long>(ii[u]) * Tw + jj[u]) = o;
        }
      }
    } else {
      const int n = (i1 - i0) * Tw;
      for (int x = threadIdx.x; x < n; x += blockDim.x) {
        const int i = i0 + x / Tw;
        const int j = x % Tw;
        const int gi = tr * Th + i, gj = tc * Tw + j;
        float r = 0.f;
        if (gi < e.h && gj < e.w) {
          const long long off = static_cast<long long>(gi) * e.ld + gj;
          float g = 0.f;
          for (int s = 0; s < n_src; ++s) g += ldf(reinterpret_cast<const G*>(e.grad[s]) + off);
          g *= gscale;
          const long long moff = static_cast<long long>(gi) * e.w + gj;
          float b;
          if (sizeof(G) == 2) {
            g = round_bf16(g);
            b = round_bf16(round_bf16(ldf(mom + moff) * mu) + g);
            r = nesterov ? round_bf16(g + mu * b) : b;
          } else {
            b = ldf(mom + moff) * mu + g;
            r = nesterov ? g + mu * b : b;
          }
          stf(mom + moff, b);
        }
        out[static_cast<long long>(i) * Tw + j] = __float2bfloat16_rn(r);
      }
    }
  }
}

void momentum_tile(const MomTileEntry* entries, int n_entries, int total_units, int Th, int Tw, void* tiles,
                   float momentum, int nesterov, float grad_scale, int n_src, int grad_fp32, cudaStream_t stream) {
  if (total_units <= 0) return;
  const int grid = total_units < num_sms() * 16 ? total_units : num_sms() * 16;
  if (grad_fp32)
    momentum_tile_kernel<float><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, Th, Tw,
                                                          reinterpret_cast<__nv_bfloat16*>(tiles), momentum, nesterov,
                                                          grad_scale, n_src);
  else
    momentum_tile_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, Th, Tw,
                                                                  reinterpret_cast<__nv_bfloat16*>(tiles), momentum,
                                                                  nesterov, grad_scale, n_src);
}

// ------------------------------------------------------------------------------------------------
template <typename P>
__global__ void __launch_bounds__(256)
untile_apply_kernel(const ApplyEntry* __restrict__ entries, int n_entries, int total_units, int Th, int Tw,
                    const __nv_bfloat16* __restrict__ tiles, const float* __restrict__ hyper) {
  const int row_blocks = (Th + kRowsPerUnit - 1) / kRowsPerUnit;
  for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
    const int ei = find_entry(entries, n_entries, unit);
    const ApplyEntry e = entries[ei];
    const float lr = hyper[8 * e.group], wd = hyper[8 * e.group + 1];
    const float decay = wd > 0.f ? 1.f - lr * wd : 1.f;
    const float step = lr * e.scale;
    const int local = unit - e.unit_begin;
    const int t = local / row_blocks;
    const int rb = local - t * row_blocks;
    const int tr = t / e.C, tc = t - tr * e.C;
    const __nv_bfloat16* in = tiles + (e.tile_base + t) * static_cast<long long>(Th) * Tw;
    P* param = reinterpret_cast<P*>(e.param);
    const int i0 = rb * kRowsPerUnit;
    const int i1 = min(Th, i0 + kRowsPerUnit);
    const bool vec = (sizeof(P) == 2) && (Tw % 8 == 0) && (e.ld % 8 == 0) && (e.w % 8 == 0);
    if (vec) {
      const int vec_per_row = Tw / 8;
      const int nvec = (i1 - i0) * vec_per_row;
      for (int x = threadIdx.x; x < nvec; x += blockDim.x) {
        const int i = i0 + x / vec_per_row;
        const int j = (x % vec_per_row) * 8;
        const int gi = tr * Th + i, gj = tc * Tw + j;
        if (gi >= e.h || gj >= e.w) continue;
        const uint4 uv = *reinterpret_cast<const uint4*>(in + static_cast<long long>(i) * Tw + j);
        __nv_bfloat16* pp = reinterpret_cast<__nv_bfloat16*>(param) + static_cast<long long>(gi) * e.ld + gj;
        uint4 pv = *reinterpret_cast<const uint4*>(pp);
        const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float a = bf16_lo(pw[q]), b = bf16_hi(pw[q]);
          if (wd > 0.f) { a = round_bf16(a * decay); b = round_bf16(b * decay); }
          a -= step * bf16_lo(uw[q]);
          b -= step * bf16_hi(uw[q]);
          pw[q] = pack_bf16x2(a, b);
        }
        pv.x = pw[0]; pv.y = pw[1]; pv.z = pw[2]; pv.w = pw[3];
        *reinterpret_cast<uint4*>(pp) = pv;
      }
    } else {
      const int n = (i1 - i0) * Tw;
      for (int x = threadIdx.x; x < n; x += blockDim.x) {
        const int i = i0 + x / Tw;
        const int j = x % Tw;
        const int gi = tr * Th + i, gj = tc * Tw + j;
        if (gi >= e.h || gj >= e.w) continue;
        const float u = __bfloat162float(in[static_cast<long long>(i) * Tw + j]);
        P* pp = param + static_cast<long long>(gi) * e.ld + gj;
        float v = ldf(pp);
        if (wd > 0.f) { v *= decay; if (sizeof(P) == 2) v = round_bf16(v); }
        stf(pp, v - step * u);
      }
    }
  }
}

void untile_apply(const ApplyEntry* entries, int n_entries, int total_units, int Th, int Tw, const void* tiles,
                  const float* hyper, int param_fp32, cudaStream_t stream) {
  if (total_units <= 0) return;
  const int grid = total_units < num_sms() * 16 ? total_units : num_sms() * 16;
  if (param_fp32)
    untile_apply_kernel<float><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, Th, Tw,
                                                         reinterpret_cast<const __nv_bfloat16*>(tiles), hyper);
  else
    untile_apply_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, Th, Tw,
                                                                 reinterpret_cast<const __nv_bfloat16*>(tiles), hyper);
}

// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

__global__ void __launch_bounds__(1024)
ns_normalize_kernel(const __nv_bfloat16* tiles, __nv_bfloat16* out, long long n_tiles, long long tile_elems, float eps) {
  __shared__ float red[32];
  for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const __nv_bfloat16* x = tiles + t * tile_elems;
    __nv_bfloat16* y = out + t * tile_elems;             // may alias x (in place)
    float ss = 0.f;
    if ((tile_elems & 7) == 0) {
      const long long nv = tile_elems >> 3;
      const uint4* xv = reinterpret_cast<const uint4*>(x);
      long long i = threadIdx.x;
      for (; i + 3 * blockDim.x < nv; i += 4 * blockDim.x) {      // four independent loads in flight per thread
        uint4 v4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v4[u] = xv[i + u * blockDim.x];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t w[4] = {v4[u].x, v4[u].y, v4[u].z, v4[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) { const float a = bf16_lo(w[q]), b = bf16_hi(w[q]); ss += a * a + b * b; }
        }
      }
      for (; i < nv; i += blockDim.x) {
        const uint4 v = xv[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float a = bf16_lo(w[q]), b = bf16_hi(w[q]); ss += a * a + b * b; }
      }
    } else {
      for (long long i = threadIdx.x; i < tile_elems; i += blockDim.x) { const float a = __bfloat162float(x[i]); ss += a * a; }
    }
    const float tot = block_sum(ss, red);
    // an all-zero (padding) tile stays exactly zero (inv = 0 also covers the out-of-place copy); uniform over the block
    if (tot == 0.f && y == x) continue;
    const float inv = tot == 0.f ? 0.f : 1.f / (sqrtf(tot) + eps);
    if ((tile_elems & 7) == 0) {
      const long long nv = tile_elems >> 3;
      const uint4* xv = reinterpret_cast<const uint4*>(x);
      uint4* yv = reinterpret_cast<uint4*>(y);
      long long i = threadIdx.x;
      for (; i + 3 * blockDim.x < nv; i += 4 * blockDim.x) {
        uint4 v4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v4[u] = xv[i + u * blockDim.x];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint32_t w[4] = {v4[u].x, v4[u].y, v4[u].z, v4[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(bf16_lo(w[q]) * inv, bf16_hi(w[q]) * inv);
          yv[i + u * blockDim.x] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      for (; i < nv; i += blockDim.x) {
        uint4 v = xv[i];
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(bf16_lo(w[q]) * inv, bf16_hi(w[q]) * inv);
        yv[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
      for (long long i = threadIdx.x; i < tile_elems; i += blockDim.x) y[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * inv);
    }
  }
}

void ns_normalize(void* tiles, long long n_tiles, long long tile_elems, float eps, cudaStream_t stream, void* out) {
  if (n_tiles <= 0) return;
  const long long cap = static_cast<long long>(num_sms()) * 2;
  const int grid = static_cast<int>(n_tiles < cap ? n_tiles : cap);
  const int threads = tile_elems >= 8192 ? 1024 : 256;
  ns_normalize_kernel<<<grid, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(tiles),
                                                    reinterpret_cast<__nv_bfloat16*>(out ? out : tiles), n_tiles, tile_elems, eps);
}

// ------------------------------------------------------------------------------------------------
constexpr int kAdamUnit = 4096;  // elements per work unit

// The three parameter-update conventions (0: HiMuon's fallback, 1: Muon / MuonFsdp, 2: plain AdamW, decay after the step).
__device__ __forceinline__ float adam_apply(int mode, float pi, float mi, float vi, float lr, float wd, float eps,
                                            float bc1, float bc2) {
  if (mode == 0) {
    const float u = (mi / bc1) / (sqrtf(vi) / sqrtf(bc2) + eps);
    if (wd > 0.f) pi *= 1.f - lr * wd;
    pi -= lr * u;
  } else if (mode == 1) {
    const float u = mi / (eps + sqrtf(vi));
    const float scale = bc1 / sqrtf(bc2);
    if (wd > 0.f) pi *= 1.f - lr * wd;
    pi -= (lr / scale) * u;
  } else {
    const float u = mi / (sqrtf(vi) + eps);
    pi -= lr * sqrtf(bc2) / bc1 * u;
    if (wd > 0.f) pi -= lr * wd * pi;
  }
  return pi;
}

template <typename P, typename S>
__global__ void __launch_bounds__(256)
adamw_multi_kernel(const AdamEntry* __restrict__ entries, int n_entries, long long total_units,
                   const float* __restrict__ hyper, const float* __restrict__ step_ptr, int mode) {
  const float t = *step_ptr + 1.f;  // this step's index; the counter itself is advanced by adamw_step_advance
  for (long long unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
    int lo = 0, hi = n_entries - 1;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (entries[mid].unit_begin <= unit) lo = mid; else hi = mid - 1;
    }
    const AdamEntry e = entries[lo];
    const float* h = hyper + 8 * e.group;
    const float lr = h[0], wd = h[1], b1 = h[2], b2 = h[3], eps = h[4];
    const float bc1 = 1.f - powf(b1, t), bc2 = 1.f - powf(b2, t);
    const long long base = (unit - e.unit_begin) * kAdamUnit;
    const long long end = min(e.numel, base + kAdamUnit);
    P* p = reinterpret_cast<P*>(e.param);
    const S* g = reinterpret_cast<const S*>(e.grad);
    S* m = reinterpret_cast<S*>(e.m);
    S* v = reinterpret_cast<S*>(e.v);
    long long scalar_from = base;
    if (sizeof(P) == 2 && sizeof(S) == 2 &&
        ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
          reinterpret_cast<uintptr_t>(v)) & 15) == 0) {
      // all-bf16 tensors: eight elements per thread and access (units start on multiples of 4096 elements)
      const long long nvec = (end - base) >> 3;
      for (long long k = threadIdx.x; k < nvec; k += blockDim.x) {
        const long long i = base + (k << 3);
        const uint4 g4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e.grad) + i);
        uint4 m4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e.m) + i);
        uint4 v4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e.v) + i);
        uint4 p4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e.param) + i);
        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
        uint32_t mw[4] = {m4.x, m4.y, m4.z, m4.w}, vw[4] = {v4.x, v4.y, v4.z, v4.w}, pw[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float mo[2], vo[2], po[2];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const float gi = hh ? bf16_hi(gw[q]) : bf16_lo(gw[q]);
            float mi = hh ? bf16_hi(mw[q]) : bf16_lo(mw[q]);
            float vi = hh ? bf16_hi(vw[q]) : bf16_lo(vw[q]);
            float pi = hh ? bf16_hi(pw[q]) : bf16_lo(pw[q]);
            mi = round_bf16(mi + (gi - mi) * (1.f - b1));
            vi = round_bf16(vi + (gi * gi - vi) * (1.f - b2));
            pi = adam_apply(mode, pi, mi, vi, lr, wd, eps, bc1, bc2);
            mo[hh] = mi; vo[hh] = vi; po[hh] = pi;
          }
          mw[q] = pack_bf16x2(mo[0], mo[1]);
          vw[q] = pack_bf16x2(vo[0], vo[1]);
          pw[q] = pack_bf16x2(po[0], po[1]);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(e.m) + i) = make_uint4(mw[0], mw[1], mw[2], mw[3]);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(e.v) + i) = make_uint4(vw[0], vw[1], vw[2], vw[3]);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(e.param) + i) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      }
      scalar_from = base + (nvec << 3);
    }
    for (long long i = scalar_from + threadIdx.x; i < end; i += blockDim.x) {
      const float gi = ldf(g + i);
      float mi = ldf(m + i), vi = ldf(v + i);
      mi = mi + (gi - mi) * (1.f - b1);
      vi = vi + (gi * gi - vi) * (1.f - b2);
      if (sizeof(S) == 2) { mi = round_bf16(mi); vi = round_bf16(vi); }
      stf(m + i, mi);
      stf(v + i, vi);
      stf(p + i, adam_apply(mode, ldf(p + i), mi, vi, lr, wd, eps, bc1, bc2));
    }
  }
}

__global__ void adamw_step_advance_kernel(float* step) { *step += 1.f; }

void adamw_step_advance(float* step, cudaStream_t stream) { adamw_step_advance_kernel<<<1, 1, 0, stream>>>(step); }

void adamw_multi(const AdamEntry* entries, int n_entries, long long total_units, const float* hyper, float* step,
                 int mode, int param_fp32, int state_fp32, cudaStream_t stream) {
  if (total_units <= 0) return;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  const int grid = static_cast<int>(total_units < cap ? total_units : cap);
  if (param_fp32 && state_fp32)
    adamw_multi_kernel<float, float><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, hyper, step, mode);
  else if (!param_fp32 && !state_fp32)
    adamw_multi_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, hyper, step, mode);
  else if (!param_fp32 && state_fp32)
    adamw_multi_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, hyper, step, mode);
  else
    adamw_multi_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(entries, n_entries, total_units, hyper, step, mode);
}

}  // namespace himuon
