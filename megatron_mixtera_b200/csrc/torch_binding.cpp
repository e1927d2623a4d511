// torch custom-op front of libb200_decode.so: TORCH_LIBRARY(b200_decode, ...).
//
// Each op checks device, dtype and contiguity of its tensors on the host, takes the CURRENT CUDA stream of the
// tensors' device, calls the C-ABI entry point of include/b200_decode.h with raw pointers and sizes, and turns a
// non-zero return code into a c10::Error (TORCH_CHECK).  No kernel lives here and nothing is allocated here: outputs
// and workspaces are tensors the caller passes in.  The shim is a separate shared object that links the C-ABI library,
// so the same kernels stay reachable without torch (ctypes, cgo, JNI ...).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include "../../include/b200_decode.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

inline b200_stream_t stream_of(const Tensor& t) {
  return reinterpret_cast<b200_stream_t>(at::cuda::getCurrentCUDAStream(t.get_device()).stream());
}
inline void need(const Tensor& t, at::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda(), "b200_decode: ", name, " must be a CUDA tensor (no CPU fallback exists)");
  TORCH_CHECK(t.scalar_type() == dt, "b200_decode: ", name, " must be ", dt, ", got ", t.scalar_type());
  TORCH_CHECK(t.is_contiguous(), "b200_decode: ", name, " must be contiguous");
}
inline void need_opt(const OptTensor& t, at::ScalarType dt, const char* name) {
  if (t.has_value()) need(*t, dt, name);
}
// split-K partial sums live in the caller's byte workspace: fp32 values in a uint8 (or float) tensor
inline void need_partials(const OptTensor& t) {
  if (!t.has_value()) return;
  TORCH_CHECK(t->is_cuda() && t->is_contiguous() && (t->scalar_type() == at::kByte || t->scalar_type() == at::kFloat),
              "b200_decode: partials must be a contiguous CUDA tensor of uint8 or float32");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "b200_decode: partials must be 16-byte aligned");
}
inline void* ptr(const Tensor& t) { return t.data_ptr(); }
inline void* ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
inline void ok(int code, const char* fn) {
  TORCH_CHECK(code == B200_OK, fn, " failed: ", b200_error_string(code), " (", code, ")");
}
constexpr auto BF16 = at::kBFloat16;
constexpr auto U8 = at::kByte;
constexpr auto F32 = at::kFloat;
constexpr auto I64 = at::kLong;
constexpr auto I32 = at::kInt;

// ---------------------------------------------------------------------------------------------------------------
// row kernels
// ---------------------------------------------------------------------------------------------------------------
void gather_rows(const Tensor& table, const Tensor& ids, Tensor out, int64_t vocab_start, int64_t vocab_end,
                 const OptTensor& add_table, const OptTensor& add_ids) {
  need(table, BF16, "table");
  need(ids, I64, "ids");
  need(out, BF16, "out");
  need_opt(add_table, BF16, "add_table");
  need_opt(add_ids, I64, "add_ids");
  c10::cuda::CUDAGuard guard(table.device());
  ok(b200_gather_rows_bf16(ptr(table), static_cast<const int64_t*>(ptr(ids)), ptr(out), static_cast<int>(ids.numel()),
                           static_cast<int>(table.size(1)), vocab_start, vocab_end, ptr(add_table),
                           static_cast<const int64_t*>(ptr(add_ids)), stream_of(table)),
     "b200_gather_rows_bf16");
}

// x (bf16) or split-K partial sums (fp32 [splits][rows][hidden]) -> hidden / normed (bf16) or quantised (q_mode 1 / 2)
void add_norm(const OptTensor& x, const OptTensor& partials, int64_t num_splits, const OptTensor& bias,
              const OptTensor& residual, const OptTensor& gamma, const OptTensor& beta, const OptTensor& hidden_out,
              const OptTensor& normed_out, const OptTensor& q_out, const OptTensor& scales_out, int64_t q_mode,
              int64_t m_pad, int64_t rows, int64_t hidden, double eps) {
  TORCH_CHECK(x.has_value() != partials.has_value(), "b200_decode.add_norm: exactly one of x / partials");
  need_opt(x, BF16, "x");
  need_partials(partials);
  need_opt(bias, BF16, "bias");
  need_opt(residual, BF16, "residual");
  need_opt(gamma, BF16, "gamma");
  need_opt(beta, BF16, "beta");
  need_opt(hidden_out, BF16, "hidden_out");
  need_opt(normed_out, BF16, "normed_out");
  need_opt(q_out, U8, "q_out");
  const Tensor& any = x.has_value() ? *x : *partials;
  c10::cuda::CUDAGuard guard(any.device());
  auto s = stream_of(any);
  const int r = static_cast<int>(rows), h = static_cast<int>(hidden), ns = static_cast<int>(num_splits);
  const float e = static_cast<float>(eps);
  int rc;
  if (q_mode == 0) {
    rc = x.has_value() ? b200_add_norm_bf16(ptr(x), ptr(bias), ptr(residual), ptr(gamma), ptr(beta), ptr(hidden_out),
                                            ptr(normed_out), r, h, e, s)
                       : b200_add_norm_splitk_bf16(static_cast<const float*>(ptr(partials)), ns, ptr(bias), ptr(residual),
                                                   ptr(gamma), ptr(beta), ptr(hidden_out), ptr(normed_out), r, h, e, s);
  } else if (q_mode == 1) {
    need_opt(scales_out, U8, "scales_out");
    rc = x.has_value() ? b200_add_norm_mxfp8(ptr(x), ptr(bias), ptr(residual), ptr(gamma), ptr(beta), ptr(hidden_out),
                                             ptr(q_out), ptr(scales_out), r, h, e, s)
                       : b200_add_norm_splitk_mxfp8(static_cast<const float*>(ptr(partials)), ns, ptr(bias), ptr(residual),
                                                    ptr(gamma), ptr(beta), ptr(hidden_out), ptr(q_out), ptr(scales_out), r,
                                                    h, e, s);
  } else {
    need_opt(scales_out, F32, "scales_out");
    rc = x.has_value()
             ? b200_add_norm_fp8_rowblock(ptr(x), ptr(bias), ptr(residual), ptr(gamma), ptr(beta), ptr(hidden_out),
                                          ptr(q_out), static_cast<float*>(ptr(scales_out)), static_cast<int>(m_pad), r, h, e, s)
             : b200_add_norm_splitk_fp8_rowblock(static_cast<const float*>(ptr(partials)), ns, ptr(bias), ptr(residual),
                                                 ptr(gamma), ptr(beta), ptr(hidden_out), ptr(q_out),
                                                 static_cast<float*>(ptr(scales_out)), static_cast<int>(m_pad), r, h, e, s);
  }
  ok(rc, "b200_add_norm");
}

void activation(const OptTensor& x, const OptTensor& partials, int64_t num_splits, const OptTensor& bias,
                const OptTensor& out, const OptTensor& q_out, const OptTensor& scales_out, int64_t q_mode, int64_t m_pad,
                int64_t rows, int64_t F, int64_t kind) {
  TORCH_CHECK(x.has_value() != partials.has_value(), "b200_decode.activation: exactly one of x / partials");
  need_opt(x, BF16, "x");
  need_partials(partials);
  need_opt(bias, BF16, "bias");
  need_opt(out, BF16, "out");
  need_opt(q_out, U8, "q_out");
  const Tensor& any = x.has_value() ? *x : *partials;
  c10::cuda::CUDAGuard guard(any.device());
  auto s = stream_of(any);
  const int r = static_cast<int>(rows), f = static_cast<int>(F), k = static_cast<int>(kind), ns = static_cast<int>(num_splits);
  const float* p = static_cast<const float*>(ptr(partials));
  int rc;
  if (q_mode == 0) {
    rc = x.has_value() ? b200_activation_bf16(ptr(x), ptr(bias), ptr(out), r, f, k, s)
                       : b200_activation_splitk_bf16(p, ns, ptr(bias), ptr(out), r, f, k, s);
  } else if (q_mode == 1) {
    need_opt(scales_out, U8, "scales_out");
    rc = x.has_value() ? b200_activation_mxfp8(ptr(x), ptr(bias), ptr(q_out), ptr(scales_out), r, f, k, s)
                       : b200_activation_splitk_mxfp8(p, ns, ptr(bias), ptr(q_out), ptr(scales_out), r, f, k, s);
  } else {
    need_opt(scales_out, F32, "scales_out");
    float* sc = static_cast<float*>(ptr(scales_out));
    rc = x.has_value() ? b200_activation_fp8_rowblock(ptr(x), ptr(bias), ptr(q_out), sc, static_cast<int>(m_pad), r, f, k, s)
                       : b200_activation_splitk_fp8_rowblock(p, ns, ptr(bias), ptr(q_out), sc, static_cast<int>(m_pad), r, f, k, s);
  }
  ok(rc, "b200_activation");
}

// mode 1: MXFP8 activation rows; 2: 1 x 128 fp32-scaled rows; 3: MXFP8 weight (tile-major); 4: 128 x 128 block weight
void quantize(int64_t mode, const Tensor& x, Tensor q, Tensor scales, int64_t rows, int64_t K, int64_t m_pad) {
  need(x, BF16, "x");
  need(q, U8, "q");
  c10::cuda::CUDAGuard guard(x.device());
  auto s = stream_of(x);
  const int r = static_cast<int>(rows), k = static_cast<int>(K);
  int rc;
  switch (mode) {
    case 1: need(scales, U8, "scales"); rc = b200_quantize_mxfp8(ptr(x), K, ptr(q), ptr(scales), r, k, s); break;
    case 2:
      need(scales, F32, "scales");
      rc = b200_quantize_fp8_rowblock(ptr(x), K, ptr(q), static_cast<float*>(ptr(scales)), r, k, static_cast<int>(m_pad), s);
      break;
    case 3: need(scales, U8, "scales"); rc = b200_quantize_mxfp8_weight(ptr(x), ptr(q), ptr(scales), r, k, s); break;
    case 4:
      need(scales, F32, "scales");
      rc = b200_quantize_fp8_weight_block128(ptr(x), ptr(q), static_cast<float*>(ptr(scales)), r, k, s);
      break;
    default: TORCH_CHECK(false, "b200_decode.quantize: unknown mode ", mode);
  }
  ok(rc, "b200_quantize");
}

// ---------------------------------------------------------------------------------------------------------------
// GEMMs.  kind 0: bf16, 1: MXFP8 (x_scales / w_scales = E8M0 tile bytes), 2: 128-block recipe (fp32 scales)
// ---------------------------------------------------------------------------------------------------------------
void gemm(int64_t kind, const Tensor& x, const OptTensor& x_scales, int64_t m_pad, const Tensor& w, const OptTensor& w_scales,
          const OptTensor& bias, Tensor out, const OptTensor& workspace, int64_t M, int64_t N, int64_t K) {
  need(out, BF16, "out");
  need_opt(bias, BF16, "bias");
  need_opt(workspace, U8, "workspace");
  c10::cuda::CUDAGuard guard(x.device());
  auto s = stream_of(x);
  const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
  void* ws = ptr(workspace);
  const size_t ws_bytes = workspace.has_value() ? static_cast<size_t>(workspace->numel()) : 0;
  TORCH_CHECK(out.numel() >= M * N, "b200_decode.gemm: out is too small");
  int rc;
  if (kind == 0) {
    need(x, BF16, "x");
    need(w, BF16, "w");
    TORCH_CHECK(w.dim() == 2 && w.size(0) == N && w.size(1) == K && x.numel() == M * K, "b200_decode.gemm: shape mismatch");
    rc = b200_gemm_bf16(ptr(x), K, ptr(w), ptr(bias), ptr(out), N, m, n, k, ws, ws_bytes, s);
  } else if (kind == 1) {
    need(x, U8, "xq");
    need(w, U8, "wq");
    TORCH_CHECK(x_scales.has_value() && w_scales.has_value(), "b200_decode.gemm: MXFP8 needs both scale tensors");
    need(*x_scales, U8, "x_scales");
    need(*w_scales, U8, "w_scales");
    TORCH_CHECK(static_cast<size_t>(w.numel()) >= b200_fp8_weight_bytes(n, k) && x.numel() >= M * K, "b200_decode.gemm: operand too small");
    rc = b200_gemm_mxfp8(ptr(x), ptr(x_scales), ptr(w), ptr(w_scales), ptr(bias), ptr(out), N, m, n, k, ws, ws_bytes, s);
  } else {
    need(x, U8, "xq");
    need(w, U8, "wq");
    TORCH_CHECK(x_scales.has_value() && w_scales.has_value(), "b200_decode.gemm: the 128-block recipe needs both scale tensors");
    need(*x_scales, F32, "x_scales");
    need(*w_scales, F32, "w_scales");
    TORCH_CHECK(static_cast<size_t>(w.numel()) >= b200_fp8_weight_bytes(n, k) && x.numel() >= M * K, "b200_decode.gemm: operand too small");
    rc = b200_gemm_fp8_block(ptr(x), static_cast<const float*>(ptr(x_scales)), static_cast<int>(m_pad), ptr(w),
                             static_cast<const float*>(ptr(w_scales)), ptr(bias), ptr(out), N, m, n, k, ws, ws_bytes, s);
  }
  ok(rc, "b200_gemm");
}

// split-K partial sums [splits][M][N] fp32 into `partials`; returns the number of splits
int64_t gemm_splitk(int64_t kind, const Tensor& x, const OptTensor& x_scales, int64_t m_pad, const Tensor& w,
                    const OptTensor& w_scales, Tensor partials, int64_t M, int64_t N, int64_t K) {
  need_partials(partials);
  c10::cuda::CUDAGuard guard(x.device());
  auto s = stream_of(x);
  const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
  float* p = static_cast<float*>(ptr(partials));
  const size_t bytes = static_cast<size_t>(partials.numel()) * partials.element_size();
  int splits = 0, rc;
  if (kind == 0) {
    need(x, BF16, "x");
    need(w, BF16, "w");
    rc = b200_gemm_bf16_splitk(ptr(x), K, ptr(w), m, n, k, p, bytes, &splits, s);
  } else if (kind == 1) {
    need(x, U8, "xq");
    need(w, U8, "wq");
    TORCH_CHECK(x_scales.has_value() && w_scales.has_value(), "b200_decode.gemm_splitk: MXFP8 needs both scale tensors");
    rc = b200_gemm_mxfp8_splitk(ptr(x), ptr(x_scales), ptr(w), ptr(w_scales), m, n, k, p, bytes, &splits, s);
  } else {
    need(x, U8, "xq");
    need(w, U8, "wq");
    TORCH_CHECK(x_scales.has_value() && w_scales.has_value(), "b200_decode.gemm_splitk: the 128-block recipe needs both scale tensors");
    rc = b200_gemm_fp8_block_splitk(ptr(x), static_cast<const float*>(ptr(x_scales)), static_cast<int>(m_pad), ptr(w),
                                    static_cast<const float*>(ptr(w_scales)), m, n, k, p, bytes, &splits, s);
  }
  ok(rc, "b200_gemm_splitk");
  return splits;
}

void gemm_bf16_swiglu(const Tensor& x, const Tensor& w_interleaved, Tensor out) {
  need(x, BF16, "x");
  need(w_interleaved, BF16, "w");
  need(out, BF16, "out");
  const int64_t K = x.size(-1), M = x.numel() / K, N = w_interleaved.size(0);
  c10::cuda::CUDAGuard guard(x.device());
  ok(b200_gemm_bf16_swiglu(ptr(x), K, ptr(w_interleaved), ptr(out), N / 2, static_cast<int>(M), static_cast<int>(N),
                           static_cast<int>(K), stream_of(x)),
     "b200_gemm_bf16_swiglu");
}

void gemm_mxfp8_swiglu(const Tensor& xq, const Tensor& x_sf, const Tensor& wq, const Tensor& w_sf, const OptTensor& q_out,
                       const OptTensor& sf_out, const OptTensor& y_out, int64_t M, int64_t F, int64_t K) {
  need(xq, U8, "xq");
  need(x_sf, U8, "x_sf");
  need(wq, U8, "wq");
  need(w_sf, U8, "w_sf");
  need_opt(q_out, U8, "q_out");
  need_opt(sf_out, U8, "sf_out");
  need_opt(y_out, BF16, "y_out");
  c10::cuda::CUDAGuard guard(xq.device());
  ok(b200_gemm_mxfp8_swiglu(ptr(xq), ptr(x_sf), ptr(wq), ptr(w_sf), ptr(q_out), ptr(sf_out), ptr(y_out), F, static_cast<int>(M),
                            static_cast<int>(F), static_cast<int>(K), stream_of(xq)),
     "b200_gemm_mxfp8_swiglu");
}

// ---------------------------------------------------------------------------------------------------------------
// Paged attention.  `args` is a CPU uint8 tensor holding one b200_attention_args (the caller fills it from tensors it
// keeps alive); `anchor` is any CUDA tensor of the call (device + stream).  which: 0 rope_append, 1 decode attention,
// 2 prefill attention (needs `units`, int32 [num_units][4] on the device).
// ---------------------------------------------------------------------------------------------------------------
void attention(const Tensor& args, const Tensor& anchor, int64_t which, const OptTensor& units, int64_t num_units) {
  TORCH_CHECK(args.is_cpu() && args.scalar_type() == U8 && args.is_contiguous() &&
                  args.numel() == static_cast<int64_t>(sizeof(b200_attention_args)),
              "b200_decode.attention: args must be a CPU uint8 tensor of sizeof(b200_attention_args) = ",
              sizeof(b200_attention_args), " bytes");
  TORCH_CHECK(anchor.is_cuda(), "b200_decode.attention: anchor must be a CUDA tensor (no CPU fallback exists)");
  const auto* a = static_cast<const b200_attention_args*>(args.data_ptr());
  c10::cuda::CUDAGuard guard(anchor.device());
  auto s = stream_of(anchor);
  if (which == 0) {
    ok(b200_rope_append(a, s), "b200_rope_append");
  } else if (which == 1) {
    ok(b200_paged_attention(a, s), "b200_paged_attention");
  } else {
    TORCH_CHECK(units.has_value(), "b200_decode.attention: the prefill kernel needs `units`");
    need(*units, I32, "units");
    TORCH_CHECK(units->numel() >= 4 * num_units, "b200_decode.attention: `units` holds fewer than num_units entries");
    ok(b200_paged_prefill_attention(a, static_cast<const int32_t*>(ptr(units)), static_cast<int>(num_units), s),
       "b200_paged_prefill_attention");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Sampling
// ---------------------------------------------------------------------------------------------------------------
inline void need_logits(const Tensor& logits) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == BF16 && logits.dim() == 2 && logits.stride(1) == 1,
              "b200_decode: logits must be a 2-D bf16 CUDA tensor with unit inner stride");
}
void argmax(const Tensor& logits, Tensor out) {
  need_logits(logits);
  need(out, I64, "out");
  TORCH_CHECK(out.numel() >= logits.size(0), "b200_decode.argmax: out is too small");
  c10::cuda::CUDAGuard guard(logits.device());
  ok(b200_argmax_bf16(ptr(logits), logits.stride(0), static_cast<int64_t*>(ptr(out)), static_cast<int>(logits.size(0)),
                      static_cast<int>(logits.size(1)), stream_of(logits)),
     "b200_argmax_bf16");
}
void argmax_shard(const Tensor& logits, Tensor keys, int64_t index_offset) {
  need_logits(logits);
  need(keys, I64, "keys");  // 64-bit keys carried in an int64 tensor
  TORCH_CHECK(keys.numel() >= logits.size(0), "b200_decode.argmax_shard: keys is too small");
  c10::cuda::CUDAGuard guard(logits.device());
  ok(b200_argmax_shard_bf16(ptr(logits), logits.stride(0), static_cast<uint64_t*>(ptr(keys)), static_cast<int>(logits.size(0)),
                            static_cast<int>(logits.size(1)), index_offset, stream_of(logits)),
     "b200_argmax_shard_bf16");
}
void argmax_merge(const Tensor& keys, int64_t shards, int64_t rows, Tensor out) {
  need(keys, I64, "keys");
  need(out, I64, "out");
  TORCH_CHECK(keys.numel() >= shards * rows && out.numel() >= rows, "b200_decode.argmax_merge: tensor too small");
  c10::cuda::CUDAGuard guard(keys.device());
  ok(b200_argmax_merge(static_cast<const uint64_t*>(ptr(keys)), static_cast<int>(shards), static_cast<int>(rows),
                       static_cast<int64_t*>(ptr(out)), stream_of(keys)),
     "b200_argmax_merge");
}
// top_k > 0: top-k filter; otherwise nucleus filter with top_p
void filtered_probs(const Tensor& logits, Tensor probs, int64_t top_k, double top_p, double temperature) {
  need_logits(logits);
  need(probs, F32, "probs");
  TORCH_CHECK(probs.numel() >= logits.size(0) * logits.size(1), "b200_decode.filtered_probs: probs is too small");
  c10::cuda::CUDAGuard guard(logits.device());
  const int rows = static_cast<int>(logits.size(0)), vocab = static_cast<int>(logits.size(1));
  if (top_k > 0)
    ok(b200_topk_probs_bf16(ptr(logits), logits.stride(0), static_cast<float*>(ptr(probs)), rows, vocab, static_cast<int>(top_k),
                            static_cast<float>(temperature), stream_of(logits)),
       "b200_topk_probs_bf16");
  else
    ok(b200_topp_probs_bf16(ptr(logits), logits.stride(0), static_cast<float*>(ptr(probs)), rows, vocab,
                            static_cast<float>(top_p), static_cast<float>(temperature), stream_of(logits)),
       "b200_topp_probs_bf16");
}

// ---------------------------------------------------------------------------------------------------------------
// Tensor-parallel all-reduce fused with add + norm.  `comm` is a CPU uint8 tensor holding a b200_tp_comm (one-shot,
// two_shot == 0) or a b200_tp_exchange (two-shot); its peer pointers come from b200_peer_buffer_open.
// ---------------------------------------------------------------------------------------------------------------
void allreduce_add_norm(const Tensor& comm, int64_t two_shot, int64_t slot, const OptTensor& bias, const OptTensor& residual,
                        const Tensor& gamma, const OptTensor& beta, const OptTensor& hidden_out, const OptTensor& normed_out,
                        const OptTensor& q_out, const OptTensor& scales_out, int64_t q_mode, int64_t m_pad, int64_t rows,
                        int64_t hidden, double eps, const OptTensor& partials, int64_t num_splits) {
  need_partials(partials);
  TORCH_CHECK(!partials.has_value() || two_shot, "b200_decode.allreduce_add_norm: split-K input needs the two-shot form");
  const int64_t want = two_shot ? sizeof(b200_tp_exchange) : sizeof(b200_tp_comm);
  TORCH_CHECK(comm.is_cpu() && comm.scalar_type() == U8 && comm.is_contiguous() && comm.numel() == want,
              "b200_decode.allreduce_add_norm: comm must be a CPU uint8 tensor of ", want, " bytes");
  need(gamma, BF16, "gamma");
  need_opt(bias, BF16, "bias");
  need_opt(residual, BF16, "residual");
  need_opt(beta, BF16, "beta");
  need_opt(hidden_out, BF16, "hidden_out");
  need_opt(normed_out, BF16, "normed_out");
  need_opt(q_out, U8, "q_out");
  c10::cuda::CUDAGuard guard(gamma.device());
  auto s = stream_of(gamma);
  const int r = static_cast<int>(rows), h = static_cast<int>(hidden);
  const float e = static_cast<float>(eps);
  int rc;
  if (two_shot) {
    const auto* x = static_cast<const b200_tp_exchange*>(comm.data_ptr());
    rc = partials.has_value()
             ? b200_allreduce2_add_norm_splitk(x, static_cast<const float*>(ptr(partials)), static_cast<int>(num_splits),
                                               ptr(bias), ptr(residual), ptr(gamma), ptr(beta), static_cast<int>(q_mode), r, h, e, s)
             : b200_allreduce2_add_norm(x, ptr(bias), ptr(residual), ptr(gamma), ptr(beta), static_cast<int>(q_mode), r, h, e, s);
  } else {
    const auto* c = static_cast<const b200_tp_comm*>(comm.data_ptr());
    const int sl = static_cast<int>(slot);
    if (q_mode == 0) {
      rc = b200_allreduce_add_norm_bf16(c, sl, ptr(bias), ptr(residual), ptr(gamma), ptr(beta), ptr(hidden_out),
                                        ptr(normed_out), r, h, e, s);
    } else if (q_mode == 1) {
      need_opt(scales_out, U8, "scales_out");
      rc = b200_allreduce_add_norm_mxfp8(c, sl, ptr(bias), ptr(residual), ptr(gamma), ptr(beta), ptr(hidden_out), ptr(q_out),
                                         ptr(scales_out), r, h, e, s);
    } else {
      need_opt(scales_out, F32, "scales_out");
      rc = b200_allreduce_add_norm_fp8_rowblock(c, sl, ptr(bias), ptr(residual), ptr(gamma), ptr(beta), ptr(hidden_out),
                                                ptr(q_out), static_cast<float*>(ptr(scales_out)), static_cast<int>(m_pad), r, h,
                                                e, s);
    }
  }
  ok(rc, "b200_allreduce_add_norm");
}

}  // namespace

// Schemas: every tensor an op writes is an argument marked (x!), nothing is returned except the split count of
// gemm_splitk, and only the CUDA dispatch key has kernels: a call with CPU tensors alone fails in the dispatcher.
TORCH_LIBRARY(b200_decode, m) {
  m.def("gather_rows(Tensor table, Tensor ids, Tensor(a!) out, int vocab_start, int vocab_end, Tensor? add_table, "
        "Tensor? add_ids) -> ()");
  m.def("add_norm(Tensor? x, Tensor? partials, int num_splits, Tensor? bias, Tensor? residual, Tensor? gamma, Tensor? beta, "
        "Tensor(a!)? hidden_out, Tensor(b!)? normed_out, Tensor(c!)? q_out, Tensor(d!)? scales_out, int q_mode, int m_pad, "
        "int rows, int hidden, float eps) -> ()");
  m.def("activation(Tensor? x, Tensor? partials, int num_splits, Tensor? bias, Tensor(a!)? out, Tensor(b!)? q_out, "
        "Tensor(c!)? scales_out, int q_mode, int m_pad, int rows, int F, int kind) -> ()");
  m.def("quantize(int mode, Tensor x, Tensor(a!) q, Tensor(b!) scales, int rows, int K, int m_pad) -> ()");
  m.def("gemm(int kind, Tensor x, Tensor? x_scales, int m_pad, Tensor w, Tensor? w_scales, Tensor? bias, Tensor(a!) out, "
        "Tensor(b!)? workspace, int M, int N, int K) -> ()");
  m.def("gemm_splitk(int kind, Tensor x, Tensor? x_scales, int m_pad, Tensor w, Tensor? w_scales, Tensor(a!) partials, "
        "int M, int N, int K) -> int");
  m.def("gemm_bf16_swiglu(Tensor x, Tensor w_interleaved, Tensor(a!) out) -> ()");
  m.def("gemm_mxfp8_swiglu(Tensor xq, Tensor x_sf, Tensor wq, Tensor w_sf, Tensor(a!)? q_out, Tensor(b!)? sf_out, "
        "Tensor(c!)? y_out, int M, int F, int K) -> ()");
  m.def("attention(Tensor args, Tensor(a!) anchor, int which, Tensor? units, int num_units) -> ()");
  m.def("argmax(Tensor logits, Tensor(a!) out) -> ()");
  m.def("argmax_shard(Tensor logits, Tensor(a!) keys, int index_offset) -> ()");
  m.def("argmax_merge(Tensor keys, int shards, int rows, Tensor(a!) out) -> ()");
  m.def("filtered_probs(Tensor logits, Tensor(a!) probs, int top_k, float top_p, float temperature) -> ()");
  m.def("allreduce_add_norm(Tensor comm, int two_shot, int slot, Tensor? bias, Tensor? residual, Tensor gamma, Tensor? beta, "
        "Tensor(a!)? hidden_out, Tensor(b!)? normed_out, Tensor(c!)? q_out, Tensor(d!)? scales_out, int q_mode, int m_pad, "
        "int rows, int hidden, float eps, Tensor? partials, int num_splits) -> ()");
}

TORCH_LIBRARY_IMPL(b200_decode, CUDA, m) {
  m.impl("gather_rows", &gather_rows);
  m.impl("add_norm", &add_norm);
  m.impl("activation", &activation);
  m.impl("quantize", &quantize);
  m.impl("gemm", &gemm);
  m.impl("gemm_splitk", &gemm_splitk);
  m.impl("gemm_bf16_swiglu", &gemm_bf16_swiglu);
  m.impl("gemm_mxfp8_swiglu", &gemm_mxfp8_swiglu);
  m.impl("attention", &attention);
  m.impl("argmax", &argmax);
  m.impl("argmax_shard", &argmax_shard);
  m.impl("argmax_merge", &argmax_merge);
  m.impl("filtered_probs", &filtered_probs);
  m.impl("allreduce_add_norm", &allreduce_add_norm);
}
