// PyTorch bindings: tensors in, raw pointers + current stream out.  All checks that would
// otherwise become device faults (dtype, contiguity, alignment, shape agreement) happen here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "himuon.h"
#include "symm.h"

namespace py = pybind11;
using himuon::GemmArgs;

#define HM_CHECK(cond, msg) TORCH_CHECK(cond, "himuon: ", msg)

static cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static bool is_bf16(const at::Tensor& t) { return t.scalar_type() == at::kBFloat16; }
static bool is_f32(const at::Tensor& t) { return t.scalar_type() == at::kFloat; }

// out = alpha * op(a) @ op(b) + beta * aux.   a: (.., M, K) or (.., K, M) when trans_a; b: (.., K, N) or (.., N, K) when trans_b.
static void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& out, const c10::optional<at::Tensor>& aux,
                 bool trans_a, bool trans_b, double alpha, double beta, bool round_acc, int64_t max_ctas,
                 bool symmetric) {
  HM_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm operands must be CUDA tensors");
  HM_CHECK(is_bf16(a) && is_bf16(b), "gemm operands must be bf16");
  HM_CHECK(is_bf16(out) || is_f32(out), "gemm output must be bf16 or fp32");
  HM_CHECK(a.dim() == b.dim() && a.dim() == out.dim() && (a.dim() == 2 || a.dim() == 3), "gemm takes 2-D or 3-D operands");
  const c10::cuda::CUDAGuard guard(a.device());
  const int nd = a.dim();
  GemmArgs g;
  g.batch = nd == 3 ? static_cast<int>(a.size(0)) : 1;
  const int64_t a_rows = a.size(nd - 2), a_cols = a.size(nd - 1);
  const int64_t b_rows = b.size(nd - 2), b_cols = b.size(nd - 1);
  g.M = static_cast<int>(trans_a ? a_cols : a_rows);
  g.K = static_cast<int>(trans_a ? a_rows : a_cols);
  g.N = static_cast<int>(trans_b ? b_rows : b_cols);
  HM_CHECK((trans_b ? b_cols : b_rows) == g.K, "gemm inner dimensions disagree");
  HM_CHECK(out.size(nd - 2) == g.M && out.size(nd - 1) == g.N, "gemm output has the wrong shape");
  HM_CHECK(a.stride(nd - 1) == 1 && b.stride(nd - 1) == 1 && out.stride(nd - 1) == 1, "gemm needs unit inner strides");
  if (nd == 3) HM_CHECK(b.size(0) == g.batch && out.size(0) == g.batch, "gemm batch sizes disagree");
  g.A = a.data_ptr(); g.B = b.data_ptr(); g.C = out.data_ptr();
  g.lda = a.stride(nd - 2); g.ldb = b.stride(nd - 2); g.ldc = out.stride(nd - 2);
  g.strideA = nd == 3 ? a.stride(0) : 0; g.strideB = nd == 3 ? b.stride(0) : 0; g.strideC = nd == 3 ? out.stride(0) : 0;
  HM_CHECK(g.lda % 8 == 0 && g.ldb % 8 == 0 && g.strideA % 8 == 0 && g.strideB % 8 == 0,
           "gemm operand strides must be multiples of 8 elements (16 bytes)");
  HM_CHECK(reinterpret_cast<uintptr_t>(g.A) % 16 == 0 && reinterpret_cast<uintptr_t>(g.B) % 16 == 0,
           "gemm operand base addresses must be 16-byte aligned");
  g.a_mn = trans_a;     // stored (K, M): M contiguous
  g.b_mn = !trans_b;    // stored (K, N): N contiguous
  g.alpha = static_cast<float>(alpha); g.beta = static_cast<float>(beta);
  g.out_fp32 = is_f32(out) ? 1 : 0;
  g.round_acc = round_acc ? 1 : 0;
  g.max_ctas = static_cast<int>(max_ctas);
  g.symmetric = symmetric ? 1 : 0;
  if (symmetric) HM_CHECK(g.M == g.N, "gemm: a symmetric output must be square");
  if (aux.has_value() && beta != 0.0) {
    const at::Tensor& x = aux.value();
    HM_CHECK(x.scalar_type() == out.scalar_type() && x.dim() == nd && x.stride(nd - 1) == 1, "gemm aux must match the output dtype/rank");
    HM_CHECK(x.size(nd - 2) == g.M && x.size(nd - 1) == g.N, "gemm aux has the wrong shape");
    g.aux = x.data_ptr(); g.ldaux = x.stride(nd - 2); g.strideAux = nd == 3 ? x.stride(0) : 0;
  }
  himuon::gemm_bf16(g, cur_stream());
}

static void momentum_tile(const at::Tensor& entries, int64_t n_entries, int64_t total_units, int64_t Th, int64_t Tw,
                          at::Tensor& tiles, double mu, bool nesterov, double gscale, int64_t n_src, bool grad_fp32) {
  HM_CHECK(entries.is_cuda() && tiles.is_cuda() && is_bf16(tiles), "momentum_tile: bad buffers");
  HM_CHECK(entries.numel() >= n_entries * (int64_t)sizeof(himuon::MomTileEntry), "momentum_tile: entry table too small");
  HM_CHECK(n_src >= 1 && n_src <= himuon::kMaxSrc, "momentum_tile: unsupported number of gradient replicas");
  const c10::cuda::CUDAGuard guard(tiles.device());
  himuon::momentum_tile(reinterpret_cast<const himuon::MomTileEntry*>(entries.data_ptr()), (int)n_entries, (int)total_units,
                        (int)Th, (int)Tw, tiles.data_ptr(), (float)mu, nesterov ? 1 : 0, (float)gscale, (int)n_src,
                        grad_fp32 ? 1 : 0, cur_stream());
}
static void untile_apply(const at::Tensor& entries, int64_t n_entries, int64_t total_units, int64_t Th, int64_t Tw,
                         const at::Tensor& tiles, const at::Tensor& hyper, bool param_fp32) {
  HM_CHECK(entries.is_cuda() && tiles.is_cuda() && is_bf16(tiles) && hyper.is_cuda() && is_f32(hyper), "untile_apply: bad buffers");
  HM_CHECK(entries.numel() >= n_entries * (int64_t)sizeof(himuon::ApplyEntry), "untile_apply: entry table too small");
  const c10::cuda::CUDAGuard guard(tiles.device());
  himuon::untile_apply(reinterpret_cast<const himuon::ApplyEntry*>(entries.data_ptr()), (int)n_entries, (int)total_units,
                       (int)Th, (int)Tw, tiles.data_ptr(), hyper.data_ptr<float>(), param_fp32 ? 1 : 0, cur_stream());
}
static void ns_normalize(at::Tensor& tiles, int64_t n_tiles, int64_t tile_elems, double eps, const c10::optional<at::Tensor>& out) {
  HM_CHECK(tiles.is_cuda() && is_bf16(tiles) && tiles.is_contiguous(), "ns_normalize: tiles must be contiguous bf16");
  HM_CHECK(tiles.numel() >= n_tiles * tile_elems, "ns_normalize: buffer too small");
  if (out.has_value())
    HM_CHECK(out->is_cuda() && is_bf16(*out) && out->is_contiguous() && out->numel() >= n_tiles * tile_elems, "ns_normalize: bad out");
  const c10::cuda::CUDAGuard guard(tiles.device());
  himuon::ns_normalize(tiles.data_ptr(), n_tiles, tile_elems, (float)eps, cur_stream(), out.has_value() ? out->data_ptr() : nullptr);
}
static void adamw_multi(const at::Tensor& entries, int64_t n_entries, int64_t total_units, const at::Tensor& hyper,
                        at::Tensor& step, int64_t mode, bool param_fp32, bool state_fp32) {
  HM_CHECK(entries.is_cuda() && hyper.is_cuda() && is_f32(hyper) && step.is_cuda() && is_f32(step), "adamw_multi: bad buffers");
  HM_CHECK(entries.numel() >= n_entries * (int64_t)sizeof(himuon::AdamEntry), "adamw_multi: entry table too small");
  const c10::cuda::CUDAGuard guard(hyper.device());
  himuon::adamw_multi(reinterpret_cast<const himuon::AdamEntry*>(entries.data_ptr()), (int)n_entries, total_units,
                      hyper.data_ptr<float>(), step.data_ptr<float>(), (int)mode, param_fp32 ? 1 : 0, state_fp32 ? 1 : 0,
                      cur_stream());
}
static void adamw_step_advance(at::Tensor& step) {
  const c10::cuda::CUDAGuard guard(step.device());
  himuon::adamw_step_advance(step.data_ptr<float>(), cur_stream());
}

static void rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, at::Tensor& y, at::Tensor& rstd, double eps,
                        const c10::optional<at::Tensor>& delta, const c10::optional<at::Tensor>& h_out) {
  HM_CHECK(x.is_cuda() && is_bf16(x) && is_bf16(w) && is_bf16(y) && is_f32(rstd) && x.is_contiguous() && y.is_contiguous(), "rmsnorm_fwd: bad tensors");
  const int cols = (int)x.size(-1);
  const int rows = (int)(x.numel() / cols);
  HM_CHECK(rstd.numel() >= rows && w.numel() == cols, "rmsnorm_fwd: shape mismatch");
  HM_CHECK(delta.has_value() == h_out.has_value(), "rmsnorm_fwd: delta and h_out go together");
  if (delta.has_value())
    HM_CHECK(is_bf16(*delta) && is_bf16(*h_out) && delta->is_contiguous() && h_out->is_contiguous() &&
                 delta->numel() == x.numel() && h_out->numel() == x.numel(), "rmsnorm_fwd: bad delta / h_out");
  const c10::cuda::CUDAGuard guard(x.device());
  himuon::rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, cols, (float)eps, cur_stream(),
                      delta.has_value() ? delta->data_ptr() : nullptr, h_out.has_value() ? h_out->data_ptr() : nullptr);
}
static void rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd,
                        at::Tensor& dx, at::Tensor& dw_accum, const c10::optional<at::Tensor>& dres) {
  if (dres.has_value())
    HM_CHECK(is_bf16(*dres) && dres->is_contiguous() && dres->numel() == x.numel(), "rmsnorm_bwd: bad residual gradient");
  HM_CHECK(dy.is_cuda() && is_bf16(dy) && is_bf16(x) && is_bf16(w) && is_bf16(dx) && is_f32(dw_accum) && dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous(), "rmsnorm_bwd: bad tensors");
  const int cols = (int)x.size(-1);
  const int rows = (int)(x.numel() / cols);
  HM_CHECK(dw_accum.numel() == cols, "rmsnorm_bwd: dw_accum must have one fp32 per column");
  const c10::cuda::CUDAGuard guard(x.device());
  himuon::rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), dw_accum.data_ptr<float>(), rows, cols, cur_stream(),
                      dres.has_value() ? dres->data_ptr() : nullptr);
}
// x, y: (tokens, heads*128) views with unit inner stride and row stride ld
static void headnorm_rope_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& w, at::Tensor& y,
                              const c10::optional<at::Tensor>& rstd, const at::Tensor& cos_sin, int64_t heads,
                              int64_t seq_len, double eps) {
  HM_CHECK(x.is_cuda() && is_bf16(x) && is_bf16(y) && x.dim() == 2 && y.dim() == 2 && x.stride(1) == 1 && y.stride(1) == 1, "headnorm_rope_fwd: bad tensors");
  HM_CHECK(x.size(1) == heads * 128 && y.size(1) == heads * 128, "headnorm_rope_fwd: head_dim must be 128");
  HM_CHECK(is_f32(cos_sin) && cos_sin.is_contiguous() && cos_sin.numel() >= seq_len * 128, "headnorm_rope_fwd: bad rope table");
  HM_CHECK(x.stride(0) % 8 == 0 && y.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(y.data_ptr()) % 16 == 0,
           "headnorm_rope_fwd: rows must start on 16-byte boundaries");
  const bool use_norm = w.has_value();
  if (use_norm) HM_CHECK(rstd.has_value() && rstd->numel() >= x.size(0) * heads && is_bf16(*w) && w->numel() == 128, "headnorm_rope_fwd: norm needs weight[128] and rstd");
  const c10::cuda::CUDAGuard guard(x.device());
  himuon::headnorm_rope_fwd(x.data_ptr(), use_norm ? w->data_ptr() : nullptr, y.data_ptr(), use_norm ? rstd->data_ptr<float>() : nullptr,
                            cos_sin.data_ptr<float>(), (int)x.size(0), (int)heads, (int)seq_len, x.stride(0), y.stride(0), (float)eps,
                            use_norm ? 1 : 0, cur_stream());
}
static void headnorm_rope_bwd(const at::Tensor& dy, const c10::optional<at::Tensor>& x, const c10::optional<at::Tensor>& w,
                              const c10::optional<at::Tensor>& rstd, at::Tensor& dx, const c10::optional<at::Tensor>& dw_accum,
                              const at::Tensor& cos_sin, int64_t heads, int64_t seq_len) {
  HM_CHECK(dy.is_cuda() && is_bf16(dy) && is_bf16(dx) && dy.dim() == 2 && dx.dim() == 2 && dy.stride(1) == 1 && dx.stride(1) == 1, "headnorm_rope_bwd: bad tensors");
  HM_CHECK(dy.size(1) == heads * 128 && dx.size(1) == heads * 128, "headnorm_rope_bwd: head_dim must be 128");
  HM_CHECK(dy.stride(0) % 8 == 0 && dx.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(dy.data_ptr()) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(dx.data_ptr()) % 16 == 0 &&
               (!x.has_value() || (x->stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(x->data_ptr()) % 16 == 0)),
           "headnorm_rope_bwd: rows must start on 16-byte boundaries");
  const bool use_norm = w.has_value();
  if (use_norm) HM_CHECK(x.has_value() && rstd.has_value() && dw_accum.has_value() && is_f32(*dw_accum) && dw_accum->numel() == 128 && x->stride(1) == 1, "headnorm_rope_bwd: norm needs x, rstd, dw_accum");
  const c10::cuda::CUDAGuard guard(dy.device());
  himuon::headnorm_rope_bwd(dy.data_ptr(), use_norm ? x->data_ptr() : nullptr, use_norm ? w->data_ptr() : nullptr,
                            use_norm ? rstd->data_ptr<float>() : nullptr, dx.data_ptr(), use_norm ? dw_accum->data_ptr<float>() : nullptr,
                            cos_sin.data_ptr<float>(), (int)dy.size(0), (int)heads, (int)seq_len, dy.stride(0),
                            use_norm ? x->stride(0) : 0, dx.stride(0), use_norm ? 1 : 0, cur_stream());
}
static void swiglu_fwd(const at::Tensor& gate, const at::Tensor& up, at::Tensor& out) {
  HM_CHECK(gate.is_cuda() && is_bf16(gate) && is_bf16(up) && is_bf16(out) && gate.dim() == 2 && up.dim() == 2 && out.dim() == 2, "swiglu_fwd: 2-D bf16 tensors");
  HM_CHECK(gate.stride(1) == 1 && up.stride(1) == 1 && out.stride(1) == 1 && gate.sizes() == up.sizes() && gate.sizes() == out.sizes(), "swiglu_fwd: shape/stride mismatch");
  const c10::cuda::CUDAGuard guard(gate.device());
  himuon::swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.size(0), (int)gate.size(1), gate.stride(0), up.stride(0), out.stride(0), cur_stream());
}
static void swiglu_bwd(const at::Tensor& dout, const at::Tensor& gate, const at::Tensor& up, at::Tensor& dgate, at::Tensor& dup) {
  HM_CHECK(dout.is_cuda() && is_bf16(dout) && is_bf16(gate) && is_bf16(up) && is_bf16(dgate) && is_bf16(dup), "swiglu_bwd: bf16 tensors");
  HM_CHECK(dout.stride(1) == 1 && gate.stride(1) == 1 && up.stride(1) == 1 && dgate.stride(1) == 1 && dup.stride(1) == 1, "swiglu_bwd: unit inner strides");
  HM_CHECK(dout.sizes() == gate.sizes() && gate.sizes() == up.sizes() && dgate.sizes() == gate.sizes() && dup.sizes() == gate.sizes(), "swiglu_bwd: shape mismatch");
  const c10::cuda::CUDAGuard guard(gate.device());
  himuon::swiglu_bwd(dout.data_ptr(), gate.data_ptr(), up.data_ptr(), dgate.data_ptr(), dup.data_ptr(), gate.size(0), (int)gate.size(1),
                     dout.stride(0), gate.stride(0), up.stride(0), dgate.stride(0), dup.stride(0), cur_stream());
}
static void embedding_fwd(const at::Tensor& ids, const at::Tensor& table, at::Tensor& out) {
  HM_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && is_bf16(table) && table.is_contiguous() && is_bf16(out) && out.is_contiguous(), "embedding_fwd: bad tensors");
  HM_CHECK(out.numel() == ids.numel() * table.size(1), "embedding_fwd: output shape");
  const c10::cuda::CUDAGuard guard(ids.device());
  himuon::embedding_fwd(ids.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()) : nullptr, table.data_ptr(), out.data_ptr(), ids.numel(), (int)table.size(1), cur_stream());
}
static void embedding_bwd(const at::Tensor& ids, const at::Tensor& dout, at::Tensor& dtable) {
  HM_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && is_bf16(dout) && dout.is_contiguous() && dtable.is_contiguous() && (is_bf16(dtable) || is_f32(dtable)), "embedding_bwd: bad tensors");
  HM_CHECK(dtable.size(1) % 2 == 0 && dout.numel() == ids.numel() * dtable.size(1), "embedding_bwd: shapes");
  const c10::cuda::CUDAGuard guard(ids.device());
  himuon::embedding_bwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), dout.data_ptr(), dtable.data_ptr(), ids.numel(), (int)dtable.size(1), is_f32(dtable) ? 1 : 0, cur_stream());
}
static void cross_entropy(at::Tensor& logits, const at::Tensor& labels, at::Tensor& loss_sum, at::Tensor& count,
                          const c10::optional<at::Tensor>& lse, double grad_scale,
                          const c10::optional<at::Tensor>& scale_dev, int64_t ignore_index) {
  HM_CHECK(logits.is_cuda() && is_bf16(logits) && logits.dim() == 2 && logits.stride(1) == 1, "cross_entropy: logits must be 2-D bf16");
  HM_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0), "cross_entropy: labels");
  HM_CHECK(is_f32(loss_sum) && is_f32(count), "cross_entropy: accumulators must be fp32");
  if (scale_dev.has_value()) HM_CHECK(scale_dev->is_cuda() && is_f32(*scale_dev) && scale_dev->numel() == 1, "cross_entropy: scale_dev must be one fp32 on the device");
  const c10::cuda::CUDAGuard guard(logits.device());
  himuon::cross_entropy_fwd_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), loss_sum.data_ptr<float>(),
                                count.data_ptr<float>(), lse.has_value() ? lse->data_ptr<float>() : nullptr, logits.size(0),
                                (int)logits.size(1), logits.stride(0), (float)grad_scale,
                                scale_dev.has_value() ? scale_dev->data_ptr<float>() : nullptr, ignore_index, cur_stream());
}

static void flash_attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& o, at::Tensor& lse,
                           int64_t B, int64_t S, int64_t Hq, int64_t Hkv, double scale) {
  HM_CHECK(q.is_cuda() && is_bf16(q) && is_bf16(k) && is_bf16(v) && is_bf16(o) && is_f32(lse), "flash_attn_fwd: dtypes");
  HM_CHECK(q.dim() == 2 && k.dim() == 2 && v.dim() == 2 && o.dim() == 2, "flash_attn_fwd: (tokens, heads*128) views expected");
  HM_CHECK(q.size(0) == B * S && q.size(1) == Hq * 128 && k.size(1) == Hkv * 128 && v.size(1) == Hkv * 128 && o.size(1) == Hq * 128, "flash_attn_fwd: shapes (head_dim 128)");
  HM_CHECK(q.stride(1) == 1 && k.stride(1) == 1 && v.stride(1) == 1 && o.stride(1) == 1, "flash_attn_fwd: unit inner strides");
  HM_CHECK(Hq % Hkv == 0 && lse.numel() >= B * Hq * S, "flash_attn_fwd: heads / lse size");
  const c10::cuda::CUDAGuard guard(q.device());
  himuon::AttnArgs a{};
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr(); a.lse = lse.data_ptr<float>();
  a.B = (int)B; a.S = (int)S; a.Hq = (int)Hq; a.Hkv = (int)Hkv;
  a.ld_q = q.stride(0); a.ld_k = k.stride(0); a.ld_v = v.stride(0); a.ld_o = o.stride(0);
  a.scale = (float)scale;
  himuon::flash_attn_fwd(a, cur_stream());
}
static void flash_attn_bwd(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                           const at::Tensor& o, const at::Tensor& lse, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv,
                           at::Tensor& delta, const c10::optional<at::Tensor>& dkv_part, int64_t B, int64_t S, int64_t Hq,
                           int64_t Hkv, double scale) {
  HM_CHECK(q.is_cuda() && is_bf16(q) && is_bf16(k) && is_bf16(v) && is_bf16(o) && is_bf16(d_o) && is_bf16(dq) && is_bf16(dk) && is_bf16(dv) && is_f32(lse) && is_f32(delta), "flash_attn_bwd: dtypes");
  HM_CHECK(q.stride(1) == 1 && k.stride(1) == 1 && v.stride(1) == 1 && o.stride(1) == 1 && d_o.stride(1) == 1 && dq.stride(1) == 1 && dk.stride(1) == 1 && dv.stride(1) == 1, "flash_attn_bwd: unit inner strides");
  HM_CHECK(q.size(0) == B * S && q.size(1) == Hq * 128 && k.size(1) == Hkv * 128 && delta.numel() >= B * Hq * S, "flash_attn_bwd: shapes");
  const c10::cuda::CUDAGuard guard(q.device());
  himuon::AttnArgs a{};
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = const_cast<void*>(o.data_ptr()); a.lse = lse.data_ptr<float>();
  a.d_o = d_o.data_ptr(); a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr(); a.delta = delta.data_ptr<float>();
  a.B = (int)B; a.S = (int)S; a.Hq = (int)Hq; a.Hkv = (int)Hkv;
  a.ld_q = q.stride(0); a.ld_k = k.stride(0); a.ld_v = v.stride(0); a.ld_o = o.stride(0); a.ld_do = d_o.stride(0);
  a.ld_dq = dq.stride(0); a.ld_dk = dk.stride(0); a.ld_dv = dv.stride(0);
  if (dkv_part.has_value()) {
    const at::Tensor& t = dkv_part.value();     // (2, B*S, Hq*128): per-query-head dK and dV
    HM_CHECK(t.is_cuda() && is_bf16(t) && t.is_contiguous() && t.dim() == 3 && t.size(0) == 2 && t.size(1) == B * S && t.size(2) == Hq * 128,
             "flash_attn_bwd: dkv_part must be a contiguous (2, B*S, Hq*128) bf16 tensor");
    a.dk_part = t.data_ptr();
    a.dv_part = static_cast<char*>(t.data_ptr()) + t.stride(0) * 2;
    a.ld_part = t.stride(1);
  }
  a.scale = (float)scale;
  himuon::flash_attn_bwd(a, cur_stream());
}

static bool ns5_fused_supported(int64_t m, int64_t n) { return himuon::ns5_fused_supported((int)m, (int)n); }
static void ns5_fused(const at::Tensor& x, at::Tensor& out, int64_t steps, double eps) {
  HM_CHECK(x.is_cuda() && is_bf16(x) && is_bf16(out) && x.is_contiguous() && out.is_contiguous() && x.dim() == 3 && x.sizes() == out.sizes(), "ns5_fused: contiguous (B, m, n) bf16 tensors");
  HM_CHECK(himuon::ns5_fused_supported((int)x.size(1), (int)x.size(2)), "ns5_fused: tile shape not supported");
  const c10::cuda::CUDAGuard guard(x.device());
  himuon::ns5_fused(x.data_ptr(), out.data_ptr(), x.size(0), (int)x.size(1), (int)x.size(2), (int)steps, (float)eps, cur_stream());
}

static int64_t status(bool reset) { return himuon::read_status_word(reset); }

static void soap_moments(const at::Tensor& g, const at::Tensor& g_rot, at::Tensor& m, at::Tensor& v, double b1, double b2) {
  HM_CHECK(g.is_cuda() && is_bf16(g) && is_bf16(g_rot) && is_bf16(m) && is_bf16(v), "soap_moments: bf16 CUDA tensors");
  HM_CHECK(g.is_contiguous() && g_rot.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "soap_moments: contiguous tensors");
  HM_CHECK(g.numel() == g_rot.numel() && g.numel() == m.numel() && g.numel() == v.numel() && g.numel() % 8 == 0,
           "soap_moments: equal element counts, multiples of 8");
  const at::Tensor* all4[4] = {&g, &g_rot, &m, &v};
  for (const at::Tensor* t : all4)
    HM_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "soap_moments: 16-byte aligned tensors");
  const c10::cuda::CUDAGuard guard(g.device());
  himuon::soap_moments(g.data_ptr(), g_rot.data_ptr(), m.data_ptr(), v.data_ptr(), g.numel(), (float)b1, (float)b2, cur_stream());
}
static void soap_ratio(const at::Tensor& m_rot, const at::Tensor& v, at::Tensor& out, double eps) {
  HM_CHECK(m_rot.is_cuda() && is_bf16(m_rot) && is_bf16(v) && is_bf16(out), "soap_ratio: bf16 CUDA tensors");
  HM_CHECK(m_rot.is_contiguous() && v.is_contiguous() && out.is_contiguous(), "soap_ratio: contiguous tensors");
  HM_CHECK(m_rot.numel() == v.numel() && m_rot.numel() == out.numel() && m_rot.numel() % 8 == 0,
           "soap_ratio: equal element counts, multiples of 8");
  const at::Tensor* all3[3] = {&m_rot, &v, &out};
  for (const at::Tensor* t : all3)
    HM_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "soap_ratio: 16-byte aligned tensors");
  const c10::cuda::CUDAGuard guard(m_rot.device());
  himuon::soap_ratio(m_rot.data_ptr(), v.data_ptr(), out.data_ptr(), m_rot.numel(), (float)eps, cur_stream());
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("soap_moments", &soap_moments);
  m.def("soap_ratio", &soap_ratio);
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("aux") = py::none(), py::arg("trans_a") = false,
        py::arg("trans_b") = false, py::arg("alpha") = 1.0, py::arg("beta") = 0.0, py::arg("round_acc") = false,
        py::arg("max_ctas") = 0, py::arg("symmetric") = false);
  m.def("momentum_tile", &momentum_tile);
  m.def("untile_apply", &untile_apply);
  m.def("ns_normalize", &ns_normalize, py::arg("tiles"), py::arg("n_tiles"), py::arg("tile_elems"), py::arg("eps"),
        py::arg("out") = py::none());
  m.def("adamw_multi", &adamw_multi);
  m.def("adamw_step_advance", &adamw_step_advance);
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("w"), py::arg("y"), py::arg("rstd"), py::arg("eps"),
        py::arg("delta") = py::none(), py::arg("h_out") = py::none());
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"), py::arg("dx"),
        py::arg("dw_accum"), py::arg("dres") = py::none());
  m.def("headnorm_rope_fwd", &headnorm_rope_fwd);
  m.def("headnorm_rope_bwd", &headnorm_rope_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("cross_entropy", &cross_entropy);
  m.def("flash_attn_fwd", &flash_attn_fwd);
  m.def("flash_attn_bwd", &flash_attn_bwd);
  m.def("ns5_fused_supported", &ns5_fused_supported);
  m.def("ns5_fused", &ns5_fused);
  m.def("status", &status, py::arg("reset") = true);
  m.def("num_sms", [] { return himuon::num_sms(); });
  m.def("momentum_tile_units", [](int64_t R, int64_t C, int64_t Th) { return himuon::momentum_tile_units((int)R, (int)C, (int)Th); });
  m.def("sizeof_entries", [] {
    return std::vector<int64_t>{(int64_t)sizeof(himuon::MomTileEntry), (int64_t)sizeof(himuon::ApplyEntry), (int64_t)sizeof(himuon::AdamEntry)};
  });
  himuon::bind_symm(m);
}
