// Element-wise kernels of SOAP's step in the eigenbasis (bf16 tensors, fp32 arithmetic, 16-byte accesses).
//
//   soap_moments : m <- b1*m + (1-b1)*g          (first moment, kept in the parameter basis)
//                  v <- b2*v + (1-b2)*g_rot^2    (second moment, kept in the eigenbasis)
//   soap_ratio   : r <- m_rot / (sqrt(v) + eps)  (the Adam direction in the eigenbasis)
//
// The rotations around them (Q_L^T G Q_R, Q_L R Q_R^T), the Gram-matrix statistics and the parameter update are
// GEMMs with fused epilogues (gemm_sm100.cu).  Reference: src/himuon/optimizers/soap.py:142-200 (the same
// arithmetic as a chain of eager PyTorch ops).
#include "himuon.h"
#include "sm100_common.cuh"

namespace himuon {

__global__ void __launch_bounds__(256)
soap_moments_kernel(const uint4* __restrict__ g, const uint4* __restrict__ g_rot, uint4* __restrict__ m,
                    uint4* __restrict__ v, long long n_vec, float b1, float b2) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 gg = g[i], gr = g_rot[i], mm = m[i], vv = v[i];
    const uint32_t gw[4] = {gg.x, gg.y, gg.z, gg.w}, rw[4] = {gr.x, gr.y, gr.z, gr.w};
    const uint32_t mw[4] = {mm.x, mm.y, mm.z, mm.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
    uint32_t mo[4], vo[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float m0 = b1 * bf16_lo(mw[q]) + (1.f - b1) * bf16_lo(gw[q]);
      const float m1 = b1 * bf16_hi(mw[q]) + (1.f - b1) * bf16_hi(gw[q]);
      const float r0 = bf16_lo(rw[q]), r1 = bf16_hi(rw[q]);
      const float v0 = b2 * bf16_lo(vw[q]) + (1.f - b2) * r0 * r0;
      const float v1 = b2 * bf16_hi(vw[q]) + (1.f - b2) * r1 * r1;
      mo[q] = pack_bf16x2(m0, m1);
      vo[q] = pack_bf16x2(v0, v1);
    }
    m[i] = make_uint4(mo[0], mo[1], mo[2], mo[3]);
    v[i] = make_uint4(vo[0], vo[1], vo[2], vo[3]);
  }
}

__global__ void __launch_bounds__(256)
soap_ratio_kernel(const uint4* __restrict__ m_rot, const uint4* __restrict__ v, uint4* __restrict__ out,
                  long long n_vec, float eps) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 mm = m_rot[i], vv = v[i];
    const uint32_t mw[4] = {mm.x, mm.y, mm.z, mm.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
      o[q] = pack_bf16x2(bf16_lo(mw[q]) / (sqrtf(bf16_lo(vw[q])) + eps), bf16_hi(mw[q]) / (sqrtf(bf16_hi(vw[q])) + eps));
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

static int ew_blocks(long long n_vec) {
  long long b = (n_vec + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

void soap_moments(const void* g, const void* g_rot, void* m, void* v, long long n_elems, float b1, float b2,
                  cudaStream_t s) {
  if (n_elems <= 0) return;
  if (n_elems % 8) throw std::runtime_error("himuon soap_moments: element count must be a multiple of 8");
  const long long nv = n_elems / 8;
  soap_moments_kernel<<<ew_blocks(nv), 256, 0, s>>>(reinterpret_cast<const uint4*>(g), reinterpret_cast<const uint4*>(g_rot),
                                                    reinterpret_cast<uint4*>(m), reinterpret_cast<uint4*>(v), nv, b1, b2);
}

void soap_ratio(const void* m_rot, const void* v, void* out, long long n_elems, float eps, cudaStream_t s) {
  if (n_elems <= 0) return;
  if (n_elems % 8) throw std::runtime_error("himuon soap_ratio: element count must be a multiple of 8");
  const long long nv = n_elems / 8;
  soap_ratio_kernel<<<ew_blocks(nv), 256, 0, s>>>(reinterpret_cast<const uint4*>(m_rot), reinterpret_cast<const uint4*>(v),
                                                  reinterpret_cast<uint4*>(out), nv, eps);
}

}  // namespace himuon
