// TEST INFRASTRUCTURE. The one file of nanochat-cpp's MX path that is replaced when its host engine is built against
// libmxb200.so: definitions of the four entry points declared in the reference's
// src/nanochat/model/fp8/mx_gemm_kernel.h:13-32 (there implemented by mx_gemm_kernel.cu with CUTLASS for sm_120),
// each forwarding to the C ABI of include/mxb200.h. Everything above this seam (fp8.cpp, mx_gemm.cpp,
// ops/softcap_ce.cpp, ops/residual_norm.cpp) is compiled from the reference tree unmodified; selecting
// MxGemmBackend::Cutlass there then runs the B200 kernels. Error convention of the seam: a static message or null.
#include "nanochat/model/fp8/mx_gemm_kernel.h"

#include "mxb200.h"

namespace nanochat::kernels {

namespace {
const char* message(int status) {
  return status == MXB200_OK ? nullptr : mxb200_strerror(status);
}
}  // namespace

const char* cutlass_mx_gemm_bf16(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d, int64_t M,
                                 int64_t N, int64_t K, cudaStream_t stream) {
  return message(mxb200_gemm_bf16(a, a_scale, b, b_scale, d, nullptr, M, N, K, stream));
}

const char* cutlass_mx_gemm_f32(const void* a, const void* a_scale, const void* b, const void* b_scale, float* d, int64_t M,
                                int64_t N, int64_t K, const float* alpha, bool accumulate, cudaStream_t stream) {
  return message(mxb200_gemm_f32(a, a_scale, b, b_scale, d, M, N, K, alpha, accumulate ? 1 : 0, stream));
}

const char* cutlass_mx_gemm_relu_square(const void* a, const void* a_scale, const void* b, const void* b_scale, void* h,
                                        void* q, void* q_scale, void* q_t, void* q_t_scale, int64_t M, int64_t N,
                                        int64_t K, cudaStream_t stream) {
  return message(mxb200_gemm_relu_square(a, a_scale, b, b_scale, h, q, q_scale, q_t, q_t_scale, M, N, K, stream));
}

const char* cutlass_mx_gemm_relu_square_bwd(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                            const void* h, void* dh, void* dh_scale, void* dh_t, void* dh_t_scale,
                                            int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
  return message(mxb200_gemm_relu_square_bwd(a, a_scale, b, b_scale, h, dh, dh_scale, dh_t, dh_t_scale, M, N, K, stream));
}

}  // namespace nanochat::kernels
