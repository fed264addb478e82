"""CPU: the C++ face of the library at nanochat-cpp's kernel seam (include/nanochat_b200_kernels.hpp) compiles as
C++20 with nothing but the CUDA runtime headers, links against libmxb200.so, and reports the C ABI's errors in the
reference's conventions (const char* messages; no CPU fallback)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include <cstdio>
#include <cstring>
#include "nanochat_b200_kernels.hpp"
namespace k = nanochat::kernels;
int main() {
  // the reference's signatures, argument for argument (fp8_kernel.h:35-43, mx_gemm_kernel.h:13-22)
  void (*q)(const void*, bool, int64_t, int64_t, k::MxOut, k::MxOut, bool, cudaStream_t) = &k::quantize_mx;
  void (*qb)(const void*, const void*, int64_t, int64_t, k::MxOut, k::MxOut, cudaStream_t) = &k::quantize_mx_relu_square_bwd;
  const char* (*g16)(const void*, const void*, const void*, const void*, void*, int64_t, int64_t, int64_t, cudaStream_t) = &k::b200_mx_gemm_bf16;
  const char* (*g32)(const void*, const void*, const void*, const void*, float*, int64_t, int64_t, int64_t, const float*, bool, cudaStream_t) = &k::b200_mx_gemm_f32;
  const char* (*gr)(const void*, const void*, const void*, const void*, void*, void*, void*, void*, void*, int64_t, int64_t, int64_t, cudaStream_t) = &k::b200_mx_gemm_relu_square;
  const char* (*grb)(const void*, const void*, const void*, const void*, const void*, void*, void*, void*, void*, int64_t, int64_t, int64_t, cudaStream_t) = &k::b200_mx_gemm_relu_square_bwd;
  void (*rn)(const k::ResidualNormMxFwd&, cudaStream_t) = &k::residual_norm_mx_fwd;
  void (*ce)(void*, int64_t, int64_t, const int64_t*, int, int, float, float*, const float*, int64_t, const int64_t*, bool, float*, float*, cudaStream_t) = &k::softcap_ce;
  void (*cg)(const void*, int64_t, int64_t, const int64_t*, const float*, int, int, float, const float*, int64_t, const int64_t*, k::MxOut, k::MxOut, cudaStream_t) = &k::softcap_ce_grad_mx;
  (void)q; (void)qb; (void)g16; (void)g32; (void)gr; (void)grb; (void)rn; (void)ce; (void)cg;
  k::ResidualNormMxFwd norm{};
  norm.base.rows = 128, norm.base.cols = 128;
  k::residual_norm_mx_fwd(norm, nullptr);
  if (k::last_status() == MXB200_OK) return 2;
  // without an sm_100 device every call refuses with a message instead of computing on the host
  const char* msg = k::b200_mx_gemm_bf16(nullptr, nullptr, nullptr, nullptr, nullptr, 128, 128, 128, nullptr);
  k::MxOut none{nullptr, 0, nullptr, 0};
  k::quantize_mx(nullptr, true, 128, 128, none, none, false, nullptr);
  std::printf("%s|%d\n", msg ? msg : "null", k::last_status());
  return 0;
}
"""


def test_header_compiles_links_and_reports_errors(tmp_path):
    cuda_inc = "/usr/local/cuda/include"
    if not os.path.exists(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("CUDA runtime headers not found")
    import nanochat_cpp_b200  # builds the library if needed  # noqa: F401
    lib_dir = os.path.join(ROOT, "nanochat_cpp_b200")
    src = tmp_path / "seam.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "seam"
    subprocess.check_call(["g++", "-std=c++20", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc,
                           str(src), "-o", str(exe), "-L", lib_dir, "-lmxb200", f"-Wl,-rpath,{lib_dir}"])
    out = subprocess.check_output([str(exe)], text=True).strip()
    msg, status = out.rsplit("|", 1)
    import torch
    if not torch.cuda.is_available():
        assert "no CPU fallback" in msg
        assert int(status) == 6  # MXB200_ERR_DEVICE
    else:
        assert msg != "null"  # null pointers are refused either way
