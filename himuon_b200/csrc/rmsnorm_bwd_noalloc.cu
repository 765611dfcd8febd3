// Allocation-free variant of the RMSNorm backward pass (see himuon_noalloc.h for who needs it).
// The ordinary path (bindings.cpp -> rmsnorm_bwd) accumulates the weight gradient in a caller-allocated
// fp32 buffer; here that buffer is a fixed array in the library image, addressed through
// cudaGetSymbolAddress, and nothing in this file calls cudaMalloc, cudaFree or any allocating routine.
#include "himuon_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>

#include "himuon.h"

namespace {

// Scratch: one fp32 running sum per column.  64 KiB, resident on every GPU that loads the library.
static __device__ __align__(256) float g_colsum_scratch[HIMUON_NOALLOC_MAX_COLS];

thread_local std::string t_last_error;

// Host code must not use g_colsum_scratch as a pointer: the name is only a host-side handle.  The
// device address is looked up once per device, with that device current, and cached for the life of the process
// (a cudaDeviceReset in between would leave the cached address stale; the library does not support that).
float* scratch_address() {
  static float* per_device[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_scratch);
    if (e != cudaSuccess) {
      t_last_error = std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e);
      return nullptr;
    }
    per_device[dev] = static_cast<float*>(p);
  }
  return per_device[dev];
}

__global__ void colsum_to_bf16_kernel(const float* __restrict__ sums, __nv_bfloat16* __restrict__ dw, int cols) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cols) dw[i] = __float2bfloat16_rn(sums[i]);
}

}  // namespace

extern "C" int himuon_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                          void* dw, int rows, int cols, void* stream) {
  t_last_error.clear();
  if (!dy || !x || !w || !rstd || !dx || !dw) { t_last_error = "null pointer argument"; return 1; }
  if (rows <= 0 || cols <= 0) { t_last_error = "rows and cols must be positive"; return 2; }
  if (cols > HIMUON_NOALLOC_MAX_COLS) {
    t_last_error = "cols = " + std::to_string(cols) + " exceeds the built-in scratch of " +
                   std::to_string(HIMUON_NOALLOC_MAX_COLS) + " columns";
    return 3;
  }
  if (cols % 8) { t_last_error = "cols must be a multiple of 8"; return 4; }
  // The kernels move 16 bytes per access.  Callers of this C symbol bypass the tensor checks of the Python
  // bindings, so a misaligned pointer is refused here, on the host, before anything is launched.
  const void* vec_ptrs[5] = {dy, x, w, dx, dw};
  const char* vec_names[5] = {"dy", "x", "w", "dx", "dw"};
  for (int i = 0; i < 5; ++i) {
    if (reinterpret_cast<uintptr_t>(vec_ptrs[i]) % 16 != 0) {
      t_last_error = std::string(vec_names[i]) + " must be 16-byte aligned";
      return 9;
    }
  }
  if (reinterpret_cast<uintptr_t>(rstd) % 4 != 0) { t_last_error = "rstd must be 4-byte aligned"; return 9; }
  float* scratch = scratch_address();
  if (scratch == nullptr) {
    if (t_last_error.empty()) t_last_error = "cannot resolve the scratch array on the current device";
    return 5;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the sums must start at zero and the array still holds the previous call's values
  cudaError_t e = cudaMemsetAsync(scratch, 0, static_cast<size_t>(cols) * sizeof(float), s);
  if (e != cudaSuccess) { t_last_error = std::string("cudaMemsetAsync: ") + cudaGetErrorString(e); return 6; }
  try {
    himuon::rmsnorm_bwd(dy, x, w, rstd, dx, scratch, rows, cols, s);
  } catch (const std::exception& ex) {
    t_last_error = ex.what();
    return 7;
  }
  colsum_to_bf16_kernel<<<(cols + 255) / 256, 256, 0, s>>>(scratch, static_cast<__nv_bfloat16*>(dw), cols);
  e = cudaGetLastError();
  if (e != cudaSuccess) { t_last_error = std::string("kernel launch: ") + cudaGetErrorString(e); return 8; }
  return 0;
}

extern "C" const char* himuon_noalloc_last_error(void) { return t_last_error.c_str(); }
