// C-callable door into the reference's own MX quantizer, for parity pinning and timing only.
// Compiled together with the unmodified reference source (src/nanochat/model/fp8/fp8_kernel.cu, which
// pulls in mx_kernel.cuh) taken from the reference tree at build time; nothing of it is copied here.
// Test infrastructure: the product never loads this library.
#include <cstdint>

#include <cuda_runtime_api.h>

#include "nanochat/model/fp8/fp8_kernel.h"

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

}  // extern "C"
