// MX block-scale arithmetic shared by the quantizer and the host side. Semantics of nanochat-cpp's
// src/nanochat/model/fp8/mx_kernel.cuh:29-44 (exponent, multiplier, swizzled scale index), restated.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

namespace mxb200 {

constexpr int kMxBlock = 32;          // values per scale
constexpr int kScaleTileBytes = 512;  // 128 rows x 4 blocks

// Biased E8M0 exponent of the block scale for a block maximum, integer math on the float's bits.
// Reference rule: smallest power of two with amax * 2^-e <= 448 = 1.75 * 2^8, i.e. exponent(amax) - 8, plus one
// when the mantissa exceeds 1.75. Floor rule: exponent(amax) - 8. Clamped to [0, 253]; amax == 0 gives 0.
__host__ __device__ __forceinline__ int mx_exponent(uint32_t amax_bits, bool floor_rule) {
  int e = static_cast<int>(amax_bits >> 23) - 8;
  if (!floor_rule && (amax_bits & 0x7fffffu) > 0x600000u)
    e += 1;
  return e < 0 ? 0 : (e > 253 ? 253 : e);
}

// Bits of 2^(127 - e): exact reciprocal of the scale.
__host__ __device__ __forceinline__ uint32_t mx_multiplier_bits(int e) {
  return static_cast<uint32_t>(254 - e) << 23;
}

// Byte offset inside one 512-byte scale tile of (row within 128, block within 4).
__host__ __device__ __forceinline__ int mx_scale_tile_offset(int row, int block) {
  return (row & 31) * 16 + ((row >> 5) & 3) * 4 + (block & 3);
}

}  // namespace mxb200
