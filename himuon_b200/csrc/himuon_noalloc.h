// C entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference; it exists for users of this library who
// embed it somewhere device allocation is off limits: a host runtime that has already handed all
// device memory to its own pool (so a cudaMalloc here would fail or fragment it), or a latency
// critical loop that cannot afford the implicit device-wide synchronisation of cudaMalloc/cudaFree.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest `cols` the entry point accepts (the size of its built-in scratch, in floats).
#define HIMUON_NOALLOC_MAX_COLS 16384

// RMSNorm backward without any allocation.
//   dy, x : (rows, cols) bf16, contiguous      w : (cols) bf16      rstd : (rows) fp32 from the forward pass
//   dx    : (rows, cols) bf16 output            dw : (cols) bf16 output (gradient of the weight)
//   stream: a cudaStream_t (may be 0)
// dy, x, w, dx and dw must be 16-byte aligned (the kernels use 16-byte accesses) and cols a multiple of 8; a call
// that breaks either rule is refused with an error code before any kernel is launched.
// The per-column fp32 sums that the ordinary entry point keeps in a caller-allocated buffer live in a
// fixed 64 KiB array inside the library image (every GPU that loads the library holds it until
// exit).  Returns 0 on success; on failure returns non-zero and himuon_noalloc_last_error() says why
// (for instance cols > HIMUON_NOALLOC_MAX_COLS or cols not a multiple of 8).
//
// The first call on each device resolves the device address of that array (with that device
// current); make this first call before starting any stream capture.  All calls share the one
// array and it keeps whatever the previous call left, so each call clears the part it uses first,
// and two calls whose kernels overlap on the GPU (different streams, no ordering) race on it:
// serialise them.
int himuon_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                               int rows, int cols, void* stream);

// Message of the last failure on the calling thread (empty string when none).
const char* himuon_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
