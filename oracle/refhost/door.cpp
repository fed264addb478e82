// TEST INFRASTRUCTURE. A Python door into nanochat-cpp's own host engine (its fp8.cpp, mx_gemm.cpp, ops/softcap_ce.cpp
// and ops/residual_norm.cpp, compiled unmodified from the reference tree) so that the parity tests can call the
// reference's autograd functions with torch tensors, under either of its MX GEMM backends:
//   "cublas"  - cuBLASLt, the reference's default (src/nanochat/model/fp8/mx_gemm.cpp:158, 214-319): the reference
//               itself, as far as it can run on a B200;
//   "cutlass" - the kernel seam of mx_gemm_kernel.h, which in this build is b200_seam.cpp, i.e. libmxb200.so.
// Nothing here computes: every function forwards to the reference's public functions (fp8.h, mx_gemm.h,
// ops/softcap_ce.h, ops/residual_norm.h).
#include <torch/extension.h>

#include "nanochat/model/fp8/fp8.h"
#include "nanochat/model/fp8/mx_gemm.h"
#include "nanochat/model/ops/residual_norm.h"
#include "nanochat/model/ops/softcap_ce.h"

namespace nc = nanochat;

namespace {

void set_backend(const std::string& name) {
  TORCH_CHECK(name == "cublas" || name == "cutlass", "backend: cublas or cutlass");
  nc::set_mx_gemm_backend(name == "cutlass" ? nc::MxGemmBackend::Cutlass : nc::MxGemmBackend::Cublas);
}

std::string backend() {
  return nc::mx_gemm_backend() == nc::MxGemmBackend::Cutlass ? "cutlass" : "cublas";
}

std::vector<torch::Tensor> quantize_mx(const torch::Tensor& x, bool rows, bool cols, bool relu_square) {
  const nc::Fp8Tensor q = nc::quantize_mx(x, rows, cols, relu_square);
  return {q.data, q.inv_scale, q.data_t, q.inv_scale_t};
}

torch::Tensor fp8_matmul(const torch::Tensor& x, const torch::Tensor& w) {
  return nc::fp8_matmul(x, w, nullptr, nc::Fp8Recipe::Mx);
}

std::vector<torch::Tensor> fp8_qkv(const torch::Tensor& x, const torch::Tensor& wq, const torch::Tensor& wk,
                                   const torch::Tensor& wv, int64_t gate_cols) {
  return nc::fp8_qkv(x, wq, wk, wv, gate_cols, nullptr, nc::Fp8Recipe::Mx);
}

torch::Tensor fp8_relu_square_mlp(const torch::Tensor& x, const torch::Tensor& w_fc, const torch::Tensor& w_proj) {
  return nc::fp8_relu_square_mlp(x, w_fc, w_proj, nullptr, nullptr, nc::Fp8Recipe::Mx);
}

torch::Tensor softcap_cross_entropy(const torch::Tensor& x, const torch::Tensor& weight, const torch::Tensor& targets,
                                    int64_t vocab_size, double softcap, int64_t chunk_rows, const std::string& reduction) {
  const nc::LossReduction r = reduction == "mean" ? nc::LossReduction::Mean
                                                  : (reduction == "sum" ? nc::LossReduction::Sum : nc::LossReduction::None);
  return nc::softcap_cross_entropy(x, weight, targets, vocab_size, softcap, chunk_rows, r, true, nullptr, nc::Fp8Recipe::Mx);
}

torch::Tensor mx_gemm(const torch::Tensor& a, const torch::Tensor& a_scale, const torch::Tensor& b,
                      const torch::Tensor& b_scale, bool f32) {
  return nc::mx_gemm(a, a_scale, b, b_scale, f32 ? torch::kFloat32 : torch::kBFloat16);
}

void mx_gemm_f32(const torch::Tensor& a, const torch::Tensor& a_scale, const torch::Tensor& b, const torch::Tensor& b_scale,
                 const torch::Tensor& out, bool accumulate, const c10::optional<torch::Tensor>& alpha) {
  nc::mx_gemm_f32(a, a_scale, b, b_scale, out, accumulate, alpha.has_value() ? *alpha : torch::Tensor{});
}

std::vector<torch::Tensor> residual_norm_mx(const torch::Tensor& x, const c10::optional<torch::Tensor>& r,
                                            const c10::optional<torch::Tensor>& x0,
                                            const c10::optional<torch::Tensor>& resid_lambdas,
                                            const c10::optional<torch::Tensor>& x0_lambdas, int64_t layer,
                                            int64_t gate_cols) {
  auto t = [](const c10::optional<torch::Tensor>& o) { return o.has_value() ? *o : torch::Tensor{}; };
  const nc::ResidualNormMx out = nc::residual_norm_mx(x, t(r), t(x0), t(resid_lambdas), t(x0_lambdas), layer, {}, gate_cols);
  return {out.res, out.n, out.n_mx.data, out.n_mx.inv_scale, out.n_mx.data_t, out.n_mx.inv_scale_t};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("set_backend", &set_backend);
  m.def("backend", &backend);
  m.def("quantize_mx", &quantize_mx);
  m.def("fp8_matmul", &fp8_matmul);
  m.def("fp8_qkv", &fp8_qkv);
  m.def("fp8_relu_square_mlp", &fp8_relu_square_mlp);
  m.def("softcap_cross_entropy", &softcap_cross_entropy);
  m.def("mx_gemm", &mx_gemm);
  m.def("mx_gemm_f32", &mx_gemm_f32);
  m.def("residual_norm_mx", &residual_norm_mx);
  m.def("residual_norm_mx_fits", &nc::residual_norm_mx_fits);
}
