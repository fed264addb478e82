// C++ face of libmxb200 at nanochat-cpp's kernel seam.
//
// nanochat-cpp keeps its CUDA kernels behind free functions in namespace nanochat::kernels whose headers include
// only <cstdint> and <cuda_runtime_api.h> (src/nanochat/model/fp8/fp8_kernel.h:1-10, mx_gemm_kernel.h:5-9,
// ops/residual_norm_kernel.h:1-10). This header offers the MX subset of that seam with the SAME names, parameter lists and conventions, implemented as
// inline calls into the C ABI of include/mxb200.h: a translation unit of the reference that includes this header
// instead of fp8_kernel.h / mx_gemm_kernel.h, and links libmxb200.so, runs its MX path on the B200 engine.
//   - quantizer launchers return void and leave errors to cudaGetLastError-style checks in the reference
//     (fp8.cpp:152); here a failing status is kept in a thread-local that last_status() returns.
//   - GEMMs return a static message or nullptr, as cutlass_mx_gemm_* do (mx_gemm_kernel.h:12).
#pragma once

#include <cstdint>

#include <cuda_runtime_api.h>

#include "mxb200.h"

namespace nanochat::kernels {

// src/nanochat/model/fp8/fp8_kernel.h:28-33; the C struct has the same four fields in the same order.
struct MxOut {
  void* data;
  int64_t ld;
  void* scale;
  int64_t scale_tiles;
};
static_assert(sizeof(MxOut) == sizeof(mxb200_mx_out), "MxOut and mxb200_mx_out share one layout");

namespace b200_detail {
inline int& status_slot() {
  static thread_local int status = MXB200_OK;
  return status;
}
inline mxb200_mx_out view(const MxOut& o) {
  return mxb200_mx_out{o.data, o.ld, o.scale, o.scale_tiles};
}
inline const char* message(int status) {
  return status == MXB200_OK ? nullptr : mxb200_strerror(status);
}
}  // namespace b200_detail

// Status of this thread's most recent quantizer call (MXB200_OK when it launched).
inline int last_status() {
  return b200_detail::status_slot();
}

// src/nanochat/model/fp8/fp8_kernel.h:35-39
inline void quantize_mx(const void* x, bool x_bf16, int64_t rows, int64_t cols, MxOut out, MxOut out_t, bool relu_square,
                        cudaStream_t stream) {
  b200_detail::status_slot() =
        mxb200_quantize_mx(x, x_bf16 ? 1 : 0, rows, cols, b200_detail::view(out), b200_detail::view(out_t),
                           relu_square ? MXB200_PROLOGUE_RELU_SQUARE : MXB200_PROLOGUE_NONE, MXB200_SCALE_REFERENCE, stream);
}

// src/nanochat/model/fp8/fp8_kernel.h:41-43
inline void quantize_mx_relu_square_bwd(const void* g, const void* h, int64_t rows, int64_t cols, MxOut out, MxOut out_t,
                                        cudaStream_t stream) {
  b200_detail::status_slot() = mxb200_quantize_mx_relu_square_bwd(g, h, rows, cols, b200_detail::view(out),
                                                                  b200_detail::view(out_t), MXB200_SCALE_REFERENCE, stream);
}

// Same contract as cutlass_mx_gemm_bf16 (src/nanochat/model/fp8/mx_gemm_kernel.h:13-17).
inline const char* b200_mx_gemm_bf16(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d,
                                     int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
  return b200_detail::message(mxb200_gemm_bf16(a, a_scale, b, b_scale, d, nullptr, M, N, K, stream));
}

// ... with the residual add fused into the epilogue: d = bf16(float(bf16(acc)) + float(resid)), the rounding of the
// reference's separate add (src/nanochat/model/ops/residual_norm_kernel.cu:96-104). resid may alias d.
inline const char* b200_mx_gemm_bf16_residual(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                              void* d, const void* resid, int64_t M, int64_t N, int64_t K,
                                              cudaStream_t stream) {
  return b200_detail::message(mxb200_gemm_bf16(a, a_scale, b, b_scale, d, resid, M, N, K, stream));
}

// Same contract as cutlass_mx_gemm_f32 (src/nanochat/model/fp8/mx_gemm_kernel.h:19-22): needs no workspace; the
// K dimension is not split, so long-K shapes with few tiles (weight gradients) are better served by the next one.
inline const char* b200_mx_gemm_f32(const void* a, const void* a_scale, const void* b, const void* b_scale, float* d,
                                    int64_t M, int64_t N, int64_t K, const float* alpha, bool accumulate,
                                    cudaStream_t stream) {
  return b200_detail::message(mxb200_gemm_f32(a, a_scale, b, b_scale, d, M, N, K, alpha, accumulate ? 1 : 0, stream));
}

// The weight-gradient form: deterministic split-K over a caller workspace (the reference borrows torch's cuBLASLt
// workspace for the same purpose, src/nanochat/model/fp8/mx_gemm.cpp:236-237). splits <= 0: the library chooses;
// workspace_bytes must cover mxb200_gemm_workspace_bytes(M, N, K, splits).
inline const char* b200_mx_gemm_f32_splitk(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                           float* d, int64_t M, int64_t N, int64_t K, const float* alpha,
                                           bool accumulate, int splits, void* workspace, size_t workspace_bytes,
                                           cudaStream_t stream) {
  if (splits <= 0)
    splits = mxb200_gemm_splits(M, N, K);
  return b200_detail::message(mxb200_gemm_splitk(a, a_scale, b, b_scale, d, MXB200_OUT_F32, nullptr, M, N, K, alpha,
                                                 accumulate ? 1 : 0, splits, workspace, workspace_bytes, stream));
}

// Same contract as cutlass_mx_gemm_relu_square (src/nanochat/model/fp8/mx_gemm_kernel.h:24-27): h = a . b^T in bf16 and,
// from the same epilogue, quantize_mx(h, relu_square = true) into q (M, N) and q_t (N, M), bit for bit.
inline const char* b200_mx_gemm_relu_square(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                            void* h, void* q, void* q_scale, void* q_t, void* q_t_scale, int64_t M,
                                            int64_t N, int64_t K, cudaStream_t stream) {
  return b200_detail::message(
        mxb200_gemm_relu_square(a, a_scale, b, b_scale, h, q, q_scale, q_t, q_t_scale, M, N, K, stream));
}

// Same contract as cutlass_mx_gemm_relu_square_bwd (src/nanochat/model/fp8/mx_gemm_kernel.h:29-32): ga = a . b^T is not
// written; with h (M, N) bf16 the epilogue gives quantize_mx_relu_square_bwd(ga, h) into dh (M, N) and dh_t (N, M).
inline const char* b200_mx_gemm_relu_square_bwd(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                                const void* h, void* dh, void* dh_scale, void* dh_t, void* dh_t_scale,
                                                int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
  return b200_detail::message(
        mxb200_gemm_relu_square_bwd(a, a_scale, b, b_scale, h, dh, dh_scale, dh_t, dh_t_scale, M, N, K, stream));
}

// src/nanochat/model/ops/residual_norm_kernel.h:17-31 and :33-41, field for field.
struct ResidualNormFwd {
  const void *x, *r, *x0;
  const float *lr, *l0;
  void* s;
  void *res, *n;
  float* rstd;
  int64_t rows;
  int cols;
  float eps;
};

struct ResidualNormMxFwd {
  ResidualNormFwd base;
  MxOut out, out_t;
  int n_cols;
};

// This library's limit on cols (the reference's kResidualNormMxMaxCols is 1536, residual_norm_kernel.h:15).
inline constexpr int kResidualNormMxMaxCols = 2048;

// src/nanochat/model/ops/residual_norm_kernel.h:44; a failing status is kept for last_status(), as for the quantizer.
inline void residual_norm_mx_fwd(const ResidualNormMxFwd& a, cudaStream_t stream) {
  const mxb200_residual_norm_mx args{a.base.x,    a.base.r,    a.base.x0,  a.base.lr,
                                     a.base.l0,   a.base.s,    a.base.res, a.base.n,
                                     a.base.rstd, a.base.rows, a.base.cols, a.base.eps,
                                     b200_detail::view(a.out), b200_detail::view(a.out_t), a.n_cols};
  b200_detail::status_slot() = mxb200_residual_norm_mx_fwd(&args, stream);
}

// src/nanochat/model/ops/softcap_ce_kernel.h:13-22, the form the MX branch calls (grad = false: loss and lse only; the
// gradient then comes from softcap_ce_grad_mx). A call with grad = true is refused (MXB200_ERR_ARGUMENT in
// last_status()): writing the bf16 gradient belongs to the recipes this library does not replace.
inline void softcap_ce(void* logits, int64_t rows, int64_t ld, const int64_t* targets, int vocab, int padded,
                       float softcap, float* loss, const float* /*grad_scale*/, int64_t /*grad_scale_stride*/,
                       const int64_t* /*num_valid*/, bool grad, float* /*grad_amax*/, float* lse, cudaStream_t stream) {
  b200_detail::status_slot() =
        grad ? MXB200_ERR_ARGUMENT
             : mxb200_softcap_ce_loss(logits, rows, ld, targets, vocab, padded, softcap, loss, lse, stream);
}

// src/nanochat/model/ops/softcap_ce_kernel.h:24-29
inline void softcap_ce_grad_mx(const void* logits, int64_t rows, int64_t ld, const int64_t* targets, const float* lse,
                               int vocab, int padded, float softcap, const float* grad_scale,
                               int64_t grad_scale_stride, const int64_t* num_valid, MxOut out, MxOut out_t,
                               cudaStream_t stream) {
  b200_detail::status_slot() =
        mxb200_softcap_ce_grad_mx(logits, rows, ld, targets, lse, vocab, padded, softcap, grad_scale, grad_scale_stride,
                                  num_valid, b200_detail::view(out), b200_detail::view(out_t), MXB200_SCALE_REFERENCE,
                                  stream);
}

}  // namespace nanochat::kernels
