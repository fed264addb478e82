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

// The same through the mixed-precision multiply-add (fp32 = bf16 * bf16 + fp32): the halves feed the multiplier
// as 16-bit operands, so no instruction is spent widening them. mlo and mhi are the bf16 bits of the multipliers of
// the low and the high halves. The addend is -0, which keeps the sign of a zero product.
__device__ __forceinline__ uint32_t e4m3x4_scaled_fma(uint32_t w0, uint32_t w1, uint16_t mlo, uint16_t mhi) {
  uint32_t d;
  asm("{\n\t.reg .b16 a0, a1, b0, b1, lo, hi;\n\t.reg .f32 f0, f1, f2, f3;\n\t"
      "mov.b32 {a0, a1}, %1;\n\tmov.b32 {b0, b1}, %2;\n\t"
      "fma.rn.f32.bf16 f0, a0, %3, 0f80000000;\n\tfma.rn.f32.bf16 f1, a1, %4, 0f80000000;\n\t"
      "fma.rn.f32.bf16 f2, b0, %3, 0f80000000;\n\tfma.rn.f32.bf16 f3, b1, %4, 0f80000000;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, f1, f0;\n\tcvt.rn.satfinite.e4m3x2.f32 hi, f3, f2;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}\n"
      : "=r"(d)
      : "r"(w0), "r"(w1), "h"(mlo), "h"(mhi));
  return d;
}

// Four packed words holding two interleaved series (low halves, high halves): the e4m3 of the four low halves times
// mlo and of the four high halves times mhi, each as one word.
__device__ __forceinline__ void e4m3x4_scaled_fma_split(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint16_t mlo,
                                                        uint16_t mhi, uint32_t& out_lo, uint32_t& out_hi) {
  asm("{\n\t.reg .b16 a0, a1, b0, b1, c0, c1, d0, d1, p, q;\n\t.reg .f32 f0, f1, f2, f3;\n\t"
      "mov.b32 {a0, a1}, %2;\n\tmov.b32 {b0, b1}, %3;\n\tmov.b32 {c0, c1}, %4;\n\tmov.b32 {d0, d1}, %5;\n\t"
      "fma.rn.f32.bf16 f0, a0, %6, 0f80000000;\n\tfma.rn.f32.bf16 f1, b0, %6, 0f80000000;\n\t"
      "fma.rn.f32.bf16 f2, c0, %6, 0f80000000;\n\tfma.rn.f32.bf16 f3, d0, %6, 0f80000000;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 p, f1, f0;\n\tcvt.rn.satfinite.e4m3x2.f32 q, f3, f2;\n\t"
      "mov.b32 %0, {p, q};\n\t"
      "fma.rn.f32.bf16 f0, a1, %7, 0f80000000;\n\tfma.rn.f32.bf16 f1, b1, %7, 0f80000000;\n\t"
      "fma.rn.f32.bf16 f2, c1, %7, 0f80000000;\n\tfma.rn.f32.bf16 f3, d1, %7, 0f80000000;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 p, f1, f0;\n\tcvt.rn.satfinite.e4m3x2.f32 q, f3, f2;\n\t"
      "mov.b32 %1, {p, q};\n\t}\n"
      : "=&r"(out_lo), "=&r"(out_hi)
      : "r"(w0), "r"(w1), "r"(w2), "r"(w3), "h"(mlo), "h"(mhi));
}

// Running maximum of |x| over packed bf16 that skips NaN as fmaxf does (a NaN operand returns the other one), one
// instruction per word. The result's sign bits carry no meaning (xor of the operands' signs): mask them off at the end.
__device__ __forceinline__ uint32_t max_abs_skip_nan_bf16x2(uint32_t m, uint32_t w) {
  uint32_t d;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(m), "r"(w));
  return d;
}

}  // namespace mxb200
