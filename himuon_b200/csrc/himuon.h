// Host-side C++ interface of the sm_100a kernel library.  Every launcher takes raw
// device pointers and a stream; nothing here depends on PyTorch.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

namespace himuon {

// ---------------------------------------------------------------- runtime helpers
int num_sms();
int* status_word_ptr();              // device address of the bounded-wait status word
int read_status_word(bool reset);    // synchronous read (0 = healthy)

// ---------------------------------------------------------------- GEMM
// C[b] = alpha * op(A[b]) * op(B[b]) + beta * aux[b], bf16 operands, fp32 accumulate.
// a_mn = false: A stored (M x K) with K contiguous;  true: stored (K x M) with M contiguous.
// b_mn = false: B stored (N x K) with K contiguous;  true: stored (K x N) with N contiguous.
// lda/ldb are the element strides between stored rows; all leading dims and batch strides
// must be multiples of 8 elements (TMA needs 16-byte strides).
struct GemmArgs {
  const void* A = nullptr;
  const void* B = nullptr;
  void* C = nullptr;
  const void* aux = nullptr;
  int M = 0, N = 0, K = 0, batch = 1;
  long long lda = 0, ldb = 0, ldc = 0, ldaux = 0;
  long long strideA = 0, strideB = 0, strideC = 0, strideAux = 0;
  bool a_mn = false, b_mn = false;
  float alpha = 1.f, beta = 0.f;
  int out_fp32 = 0;
  int round_acc = 0;
  int max_ctas = 0;   // 0 = one CTA per SM
  int symmetric = 0;  // the caller guarantees C = C^T (X X^T, or c A A + b A with A symmetric): the one-CTA kernel then
                      // computes only the tiles that touch the lower triangle and mirrors the rest
};
void gemm_bf16(const GemmArgs& args, cudaStream_t stream);
// CTA-pair (cta_group::2) variant for 256 x 256 tiles; gemm_bf16 dispatches to it when gemm2_supported().
bool gemm2_supported(const GemmArgs& args);
void gemm2_bf16(const GemmArgs& args, cudaStream_t stream);


// ---------------------------------------------------------------- optimizer kernels
constexpr int kMaxSrc = 8;

// One matrix whose gradient is folded into momentum and written out as NS tiles.
struct MomTileEntry {
  const void* grad[kMaxSrc];  // gradient replicas to sum (this rank's plus peers'), same dtype
  void* mom;                  // momentum buffer, same dtype as the gradient
  long long tile_base;        // index of this matrix' first tile in the tile buffer
  int h, w;                   // matrix shape
  int R, C;                   // tile grid (ceil(h/Th), ceil(w/Tw))
  int unit_begin;             // first work unit of this entry
  int ld;                     // element stride between gradient rows
};
void momentum_tile(const MomTileEntry* entries, int n_entries, int total_units, int Th, int Tw, void* tiles_bf16,
                   float momentum, int nesterov, float grad_scale, int n_src, int grad_fp32, cudaStream_t stream);
int momentum_tile_units(int R, int C, int Th);

struct ApplyEntry {
  void* param;
  long long tile_base;
  int h, w;
  int R, C;
  int unit_begin;
  int group;        // row of the hyper-parameter table
  float scale;      // lr multiplier (0.2*sqrt(max(block)) or 1)
  int ld;
};
// p <- p*(1 - lr*wd) - lr*scale*U with U read from the tile buffer; lr = hyper[8g], wd = hyper[8g+1]
// (the same 8-float rows as adamw_multi).
void untile_apply(const ApplyEntry* entries, int n_entries, int total_units, int Th, int Tw, const void* tiles_bf16,
                  const float* hyper, int param_fp32, cudaStream_t stream);

// In-place per-tile Frobenius normalisation of a (B, m, n) bf16 buffer: X <- bf16(X / (||X||_F + eps)).
// `out` (same shape, optional): write the normalised tiles there instead of in place.
void ns_normalize(void* tiles_bf16, long long n_tiles, long long tile_elems, float eps, cudaStream_t stream,
                  void* out = nullptr);

struct AdamEntry {
  void* param;
  const void* grad;
  void* m;
  void* v;
  long long numel;
  long long unit_begin;
  int group;
  int pad;
};
// mode 0: HiMuon fallback (lerp moments, u = (m/bc1)/(sqrt(v)/sqrt(bc2)+eps), wd first)
// mode 1: Muon fallback   (u = m/(eps+sqrt(v)), step = lr/(bc1/sqrt(bc2)), wd first)
// mode 2: AdamW class     (u = m/(sqrt(v)+eps), step = lr*sqrt(bc2)/bc1, wd after the step)
// `step` is a device scalar that the kernel's first thread increments after use (graph-replay safe);
// hyper rows are (lr, wd, beta1, beta2, eps, unused...) with stride 8 floats per group.
void adamw_multi(const AdamEntry* entries, int n_entries, long long total_units, const float* hyper, float* step,
                 int mode, int param_fp32, int state_fp32, cudaStream_t stream);
void adamw_step_advance(float* step, cudaStream_t stream);

// SOAP in the eigenbasis (bf16, contiguous, 16-byte aligned, element counts multiples of 8):
// m <- b1*m + (1-b1)*g ; v <- b2*v + (1-b2)*g_rot^2            and            out <- m_rot / (sqrt(v) + eps)
void soap_moments(const void* g, const void* g_rot, void* m, void* v, long long n_elems, float b1, float b2,
                  cudaStream_t s);
void soap_ratio(const void* m_rot, const void* v, void* out, long long n_elems, float eps, cudaStream_t s);

// ---------------------------------------------------------------- model kernels
// With `delta`/`h_out`: h_out = bf16(x + delta) is written and normalised instead of x (fused residual update).
void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps, cudaStream_t s,
                 const void* delta = nullptr, void* h_out = nullptr);
// With `dres` (same shape as dx): dx = dres + the norm's input gradient (the residual path's gradient joins here).
void rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_accum,
                 int rows, int cols, cudaStream_t s, const void* dres = nullptr);
// Per-head RMSNorm (optional) + rotary embedding on a (tokens, heads, 128) view with row stride `ld`.
void headnorm_rope_fwd(const void* x, const void* w, void* y, float* rstd, const float* cos_sin, int tokens,
                       int heads, int seq_len, long long ld_in, long long ld_out, float eps, int use_norm,
                       cudaStream_t s);
void headnorm_rope_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_accum,
                       const float* cos_sin, int tokens, int heads, int seq_len, long long ld_dy, long long ld_x,
                       long long ld_dx, int use_norm, cudaStream_t s);
void swiglu_fwd(const void* gate, const void* up, void* out, long long rows, int cols, long long ld_g, long long ld_u,
                long long ld_o, cudaStream_t s);
void swiglu_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, long long rows, int cols,
                long long ld_do, long long ld_g, long long ld_u, long long ld_dg, long long ld_du, cudaStream_t s);
void embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int dim, cudaStream_t s);
void embedding_bwd(const long long* ids, const void* dout, void* dtable, long long tokens, int dim, int table_fp32,
                   cudaStream_t s);
// Row-wise softmax cross-entropy on bf16 logits; overwrites logits with scale*(softmax - onehot).
// Rows whose label is `ignore_index` get zero gradient.  loss_sum/count accumulate with atomics.
// The gradient scale is grad_scale * (*scale_dev) when scale_dev is given (a device scalar such as 1/n_valid).
void cross_entropy_fwd_bwd(void* logits, const long long* labels, float* loss_sum, float* count, float* lse_out,
                           long long rows, int vocab, long long ld, float grad_scale, const float* scale_dev,
                           long long ignore_index, cudaStream_t s);
void group_sum_heads(const void* in, void* out, long long tokens, int hkv, int G, long long ld_in, long long ld_out,
                     cudaStream_t s);
void cast_copy(const void* src, void* dst, long long n, int src_fp32, int dst_fp32, float scale, cudaStream_t s);
void bf16_add_to_f32(const void* src_bf16, float* dst, long long n, cudaStream_t s);

// ---------------------------------------------------------------- attention (causal GQA, head_dim 128)
// q: (B, S, Hq, 128), k/v: (B, S, Hkv, 128), o like q; all bf16 with token stride ld_* elements
// (so q/k/v may be column slices of one fused projection output).  lse: (B, Hq, S) fp32, the base-2 log-sum-exp of the
// scaled scores (log2 of the softmax denominator plus the row maximum in base-2 units), as the backward kernels use it.
struct AttnArgs {
  const void* q; const void* k; const void* v; void* o; float* lse;
  const void* d_o; void* dq; void* dk; void* dv; float* delta;
  void* dk_part; void* dv_part;       // optional (B*S, Hq*128) scratch: per-query-head dK/dV, summed over each group afterwards
  long long ld_part;
  int B, S, Hq, Hkv;
  long long ld_q, ld_k, ld_v, ld_o, ld_do, ld_dq, ld_dk, ld_dv;
  float scale;
};
void flash_attn_fwd(const AttnArgs& a, cudaStream_t s);
void flash_attn_bwd(const AttnArgs& a, cudaStream_t s);

// ---------------------------------------------------------------- collectives over peer-mapped memory
constexpr int kCommMaxBlocks = 256;
// Flag area of one rank: int[2][kCommMaxBlocks][8] (phase, block slot, writing rank), zero-initialised.
constexpr long long kCommFlagBytes = 2LL * kCommMaxBlocks * 8 * sizeof(int);
struct CommPeers {
  int* flags[kMaxSrc];            // every rank's flag area as mapped into this process
  int world, rank;
  unsigned long long limit_ns;    // bound of each wait on a peer flag
  int* status;                    // status word (code 6 on expiry)
};
struct CommBufs { void* ptr[kMaxSrc]; };
struct CopySeg { const void* src; void* dst; long long bytes; long long unit_begin; };
// epoch_local: int[2*kCommMaxBlocks] private to this rank, zero-initialised, advanced by the kernels.
void peer_barrier(const CommPeers& peers, int* epoch_local, cudaStream_t s, int channel = 0);
// algo 0 and 2: two-shot (every size), 1: one-shot (regions up to 2 MiB; never chosen automatically).
void allreduce_symm(const CommPeers& peers, const CommBufs& bufs, long long n_elems, int is_fp32, float scale,
                    int* epoch_local, int max_blocks, cudaStream_t s, int algo = 0);
// NVLS variants: `mc_region` is the multicast address of the region (all ranks' copies behind one address, vmm.cpp).
void allreduce_nvls(const CommPeers& peers, void* mc_region, long long n_elems, int is_fp32, float scale, int* epoch_local,
                    int max_blocks, cudaStream_t s);
void reduce_nvls(const void* mc_region, void* out, long long n_elems, int is_fp32, float scale, float beta, cudaStream_t s);
// out = beta * out + scale * sum of the n_src replicas.
void reduce_replicas(const CommBufs& srcs, int n_src, void* out, long long n_elems, int is_fp32, float scale,
                     cudaStream_t s, float beta = 0.f);
long long multi_copy_units(long long bytes);
void multi_copy(const CopySeg* segs_dev, int n_segs, long long total_units, int max_blocks, cudaStream_t s);

// ---------------------------------------------------------------- fused tile-resident NS5
// Five quintic Newton-Schulz iterations on (B, m, n) bf16 tiles with m <= n, m <= 128, n <= 128*... kept in
// shared memory for the whole computation (see ns5_sm100.cu).
bool ns5_fused_supported(int m, int n);
void ns5_fused(const void* x_in, void* x_out, long long n_tiles, int m, int n, int steps, float eps, cudaStream_t s);

}  // namespace himuon
