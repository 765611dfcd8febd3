// Host-side TMA tensor-map encoding without linking libcuda: the driver entry point
// is fetched at run time through the CUDA runtime, so the library also builds on a
// machine that has no driver installed.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace himuon {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
      throw std::runtime_error("himuon: cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct TmapKey {
  const void* ptr;
  uint64_t d0, d1, d2, d3;     // extents (innermost first)
  uint64_t s1, s2, s3;         // byte strides of dims 1..3
  uint32_t b0, b1, b2, b3;     // box
  int rank, elem_bytes, swizzle;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && d3 == o.d3 && s1 == o.s1 && s2 == o.s2 &&
           s3 == o.s3 && b0 == o.b0 && b1 == o.b1 && b2 == o.b2 && b3 == o.b3 && rank == o.rank &&
           elem_bytes == o.elem_bytes && swizzle == o.swizzle;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    auto mix = [&h](uint64_t v) { h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2); };
    mix(k.d0); mix(k.d1); mix(k.d2); mix(k.d3); mix(k.s1); mix(k.s2); mix(k.s3);
    mix((uint64_t(k.b0) << 32) | k.b1); mix((uint64_t(k.b2) << 32) | k.b3);
    mix((uint64_t(k.rank) << 16) | (uint64_t(k.elem_bytes) << 8) | uint64_t(k.swizzle));
    return static_cast<size_t>(h);
  }
};

// Encodes (and caches) a tiled tensor map of rank 3 or 4 over 16-bit or 32-bit elements.
// dims/box are innermost-first; strides[i] is the byte stride of dimension i+1.
// Requirements checked here: base 16-byte aligned, strides multiples of 16 bytes,
// inner box extent * element size a multiple of 16 bytes and at most 128 bytes when swizzled.
inline CUtensorMap make_tmap(const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                             const uint32_t* box, int elem_bytes, bool swizzle128) {
  TmapKey key{ptr, dims[0], dims[1], rank > 2 ? dims[2] : 1, rank > 3 ? dims[3] : 1,
              strides_bytes[0], rank > 2 ? strides_bytes[1] : 0, rank > 3 ? strides_bytes[2] : 0,
              box[0], box[1], rank > 2 ? box[2] : 1, rank > 3 ? box[3] : 1, rank, elem_bytes, swizzle128 ? 1 : 0};
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  if (reinterpret_cast<uintptr_t>(ptr) & 15) throw std::runtime_error("himuon: TMA base address must be 16-byte aligned");
  for (int i = 0; i < rank - 1; ++i)
    if (strides_bytes[i] & 15)
      throw std::runtime_error("himuon: TMA stride " + std::to_string(strides_bytes[i]) + " is not a multiple of 16 bytes");
  if ((box[0] * elem_bytes) & 15) throw std::runtime_error("himuon: TMA inner box must be a multiple of 16 bytes");
  cuuint64_t gdim[4];
  cuuint64_t gstr[3];
  cuuint32_t gbox[4];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; gbox[i] = box[i]; }
  for (int i = 0; i < rank - 1; ++i) gstr[i] = strides_bytes[i];
  CUtensorMap tm;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = get_encode_fn()(&tm, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(ptr), gdim, gstr, gbox, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE,
                               swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("himuon: cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, tm);
  }
  return tm;
}

}  // namespace himuon
