// Packed bf16x2 arithmetic for the MX quantization steps that are fused into other kernels. Device-only.
//
// Why packed math gives the reference's bits, whose kernels unpack to fp32, operate and round back to bf16:
//   * the product of two bf16 values is exact in fp32 (8 x 8 significant bits), so bf16(fp32 a * b) is the single
//     rounding mul.rn.bf16x2 performs;
//   * the fp32 sum of two bf16 values is either exact or differs from the exact sum far below a bf16 rounding
//     boundary, so bf16(fp32 a + b) is the single rounding add.rn.bf16x2 performs;
//   * a multiply by a power of two is exact in bf16 wherever the result is a normal number, and anything smaller
//     is zero in e4m3 either way.
// NaN results are the canonical 0x7fff in both forms; subnormals are kept (no flush) in both forms.
#pragma once

#include <cstdint>

namespace mxb200 {

__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// x <= 0 ? +0 : x per half, NaN kept (the reference's relu: `v <= 0.f ? 0.f : v`)
__device__ __forceinline__ uint32_t relu_keep_nan_bf16x2(uint32_t a) {
  uint32_t d;
  asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(0u));
  return d;
}

// 0xffff per half where !(h <= 0), i.e. h > 0 or h is NaN; 0 elsewhere
__device__ __forceinline__ uint32_t positive_or_nan_mask_bf16x2(uint32_t h) {
  uint32_t d;
  asm("set.gtu.u32.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(h), "r"(0u));
  return d;
}

__device__ __forceinline__ float lo_f32(uint32_t w) {
  return __uint_as_float(w << 16);
}

__device__ __forceinline__ float hi_f32(uint32_t w) {
  return __uint_as_float(w & 0xffff0000u);
}

// {lo, hi} rounded to nearest even
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

__device__ __forceinline__ uint32_t e4m3x4_from_f32(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// e4m3 of four bf16 values (two packed words) times a power of two given as packed bf16
__device__ __forceinline__ uint32_t e4m3x4_scaled(uint32_t w0, uint32_t w1, uint32_t mul2) {
  const uint32_t a = mul_bf16x2(w0, mul2), b = mul_bf16x2(w1, mul2);
  return e4m3x4_from_f32(lo_f32(a), hi_f32(a), lo_f32(b), hi_f32(b));
}

// Running maximum of |x| over packed bf16 that skips NaN as fmaxf does (a NaN operand returns the other one), one
// instruction per word. The result's sign bits carry no meaning (xor of the operands' signs): mask them off at the end.
__device__ __forceinline__ uint32_t max_abs_skip_nan_bf16x2(uint32_t m, uint32_t w) {
  uint32_t d;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(m), "r"(w));
  return d;
}

}  // namespace mxb200
