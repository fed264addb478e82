// C-callable door into the reference's own MX quantizer, fused residual-norm and softcap cross-entropy kernels, for
// parity pinning and timing only. Compiled together with the unmodified reference sources
// (src/nanochat/model/fp8/fp8_kernel.cu, src/nanochat/model/ops/residual_norm_kernel.cu and
// src/nanochat/model/ops/softcap_ce_kernel.cu, which pull in mx_kernel.cuh) taken from the reference tree at
// build time; nothing of them is copied here.
// Test infrastructure: the product never loads this library.
#include <cstdint>

#include <cuda_runtime_api.h>

#include "nanochat/model/fp8/fp8_kernel.h"
#include "nanochat/model/ops/residual_norm_kernel.h"
#include "nanochat/model/ops/softcap_ce_kernel.h"

extern "C" {

// nanochat::kernels::quantize_mx (src/nanochat/model/fp8/fp8_kernel.h:35-39) on the given stream.
// Null data pointers skip a layout. Returns the launch's cudaError_t.
int ref_quantize_mx(const void* x, int x_bf16, int64_t rows, int64_t cols, void* data, int64_t ld, void* scale,
                    int64_t scale_tiles, void* data_t, int64_t ld_t, void* scale_t, int64_t scale_tiles_t,
                    int relu_square, void* stream) {
  nanochat::kernels::MxOut out{data, ld, scale, scale_tiles}, out_t{data_t, ld_t, scale_t, scale_tiles_t};
  nanochat::kernels::quantize_mx(x, x_bf16 != 0, rows, cols, out, out_t, relu_square != 0,
                                 static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}

// nanochat::kernels::quantize_mx_relu_square_bwd (src/nanochat/model/fp8/fp8_kernel.h:41-43)
int ref_quantize_mx_relu_square_bwd(const void* g, const void* h, int64_t rows, int64_t cols, void* data, int64_t ld,
                                    void* scale, int64_t scale_tiles, void* data_t, int64_t ld_t, void* scale_t,
                                    int64_t scale_tiles_t, void* stream) {
  nanochat::kernels::MxOut out{data, ld, scale, scale_tiles}, out_t{data_t, ld_t, scale_t, scale_tiles_t};
  nanochat::kernels::quantize_mx_relu_square_bwd(g, h, rows, cols, out, out_t, static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}

// nanochat::kernels::residual_norm_fwd (src/nanochat/model/ops/residual_norm_kernel.h:18-31): n written as bf16.
int ref_residual_norm_fwd(const void* x, const void* r, const void* x0, const float* lr, const float* l0, void* s,
                          void* res, void* n, float* rstd, int64_t rows, int cols, float eps, void* stream) {
  const nanochat::kernels::ResidualNormFwd a{x, r, x0, lr, l0, s, res, n, rstd, rows, cols, eps};
  nanochat::kernels::residual_norm_fwd(a, static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}

// nanochat::kernels::residual_norm_mx_fwd (src/nanochat/model/ops/residual_norm_kernel.h:33-44): n leaves
// MX-quantized in both layouts, its first n_cols columns also as bf16. Returns -1 for shapes the reference does not
// take (rows % 32, cols % 64, cols <= kResidualNormMxMaxCols).
int ref_residual_norm_mx_fwd(const void* x, const void* r, const void* x0, const float* lr, const float* l0, void* s,
                             void* res, void* n, float* rstd, int64_t rows, int cols, float eps, void* data,
                             int64_t ld, void* scale, int64_t scale_tiles, void* data_t, int64_t ld_t, void* scale_t,
                             int64_t scale_tiles_t, int n_cols, void* stream) {
  if (rows % 32 != 0 || cols % 64 != 0 || cols > nanochat::kernels::kResidualNormMxMaxCols)
    return -1;
  const nanochat::kernels::ResidualNormMxFwd a{{x, r, x0, lr, l0, s, res, n, rstd, rows, cols, eps},
                                               {data, ld, scale, scale_tiles},
                                               {data_t, ld_t, scale_t, scale_tiles_t},
                                               n_cols};
  nanochat::kernels::residual_norm_mx_fwd(a, static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}

// nanochat::kernels::softcap_ce (src/nanochat/model/ops/softcap_ce_kernel.h:13-22). With grad != 0 the logits are
// overwritten by their gradient.
int ref_softcap_ce(void* logits, int64_t rows, int64_t ld, const int64_t* targets, int vocab, int padded, float softcap,
                   float* loss, const float* grad_scale, int64_t grad_scale_stride, const int64_t* num_valid, int grad,
                   float* lse, void* stream) {
  nanochat::kernels::softcap_ce(logits, rows, ld, targets, vocab, padded, softcap, loss, grad_scale, grad_scale_stride,
                                num_valid, grad != 0, nullptr, lse, static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}

// nanochat::kernels::softcap_ce_grad_mx (src/nanochat/model/ops/softcap_ce_kernel.h:24-29)
int ref_softcap_ce_grad_mx(const void* logits, int64_t rows, int64_t ld, const int64_t* targets, const float* lse,
                           int vocab, int padded, float softcap, const float* grad_scale, int64_t grad_scale_stride,
                           const int64_t* num_valid, void* data, int64_t ld_out, void* scale, int64_t scale_tiles,
                           void* data_t, int64_t ld_t, void* scale_t, int64_t scale_tiles_t, void* stream) {
  nanochat::kernels::softcap_ce_grad_mx(logits, rows, ld, targets, lse, vocab, padded, softcap, grad_scale,
                                        grad_scale_stride, num_valid, {data, ld_out, scale, scale_tiles},
                                        {data_t, ld_t, scale_t, scale_tiles_t}, static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
