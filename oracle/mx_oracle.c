/* CPU oracle for the MXFP8 Linear path, plain C: test infrastructure, never the product.
 *
 * A scalar restatement of nanochat-cpp's MX quantizer and block-scaled GEMM semantics,
 * independent of the numpy one in mx_oracle.py so the two can check each other. Only tests,
 * the smoke check and the benchmark's CPU-baseline leg may load this library.
 * Citations are file:line within the nanochat-cpp repository.
 *
 * Parity pin: see mx_oracle.py's header (torch-op formulation on CPU + bytes written by the
 * reference's own CUDA quantizer on a B200, stored under tests/golden/).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> bf16 -> fp32, round to nearest even (src/nanochat/model/fp8/fp8_kernel.cu:44-50) */
float mxo_round_bf16(float x) {
  uint32_t b = f2u(x);
  if (isnan(x)) return u2f(0x7FFF0000u);
  b = (b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u;
  return u2f(b);
}

/* biased e8m0 byte: src/nanochat/model/fp8/mx_kernel.cuh:29-34 (rule 0); rule 1 = floor(log2 amax) - 8 */
int mxo_exponent(float amax, int rule) {
  const uint32_t bits = f2u(amax);
  int e = (int)(bits >> 23) - 8;
  if (rule == 0 && (bits & 0x7FFFFFu) > 0x600000u) e += 1;
  return e < 0 ? 0 : (e > 253 ? 253 : e);
}

/* 2^(127 - e): src/nanochat/model/fp8/mx_kernel.cuh:37-39 */
float mxo_multiplier(int e) { return u2f((uint32_t)(254 - e) << 23); }

/* fp32 -> e4m3, RNE, saturate to +-448, NaN -> 0x7f (src/nanochat/model/fp8/mx_kernel.cuh:61) */
uint8_t mxo_e4m3(float x) {
  if (isnan(x)) return 0x7F;
  const uint8_t sign = (uint8_t)((f2u(x) >> 31) << 7);
  double a = fabs((double)x);
  if (a > 448.0) a = 448.0;
  if (a == 0.0) return sign;
  int ex;
  frexp(a, &ex); /* a = m * 2^ex, m in [0.5, 1) */
  double q = a < 0.015625 ? 0.001953125 : ldexp(1.0, ex - 1 - 3);
  double r = nearbyint(a / q) * q; /* default rounding mode: ties to even */
  if (r > 448.0) r = 448.0;
  if (r == 0.0) return sign;
  if (r < 0.015625) return (uint8_t)(sign | (uint8_t)nearbyint(r / 0.001953125));
  frexp(r, &ex);
  const int fl = ex - 1;
  const int mant = (int)nearbyint((r / ldexp(1.0, fl) - 1.0) * 8.0);
  return (uint8_t)(sign | ((fl + 7) << 3) | mant);
}

float mxo_e4m3_to_f32(uint8_t v) {
  const float s = (v & 0x80) ? -1.f : 1.f;
  const int ef = (v >> 3) & 0xF, m = v & 7;
  if (ef == 0xF && m == 7) return NAN;
  if (ef == 0) return s * (float)m * 0.001953125f;
  return s * (1.f + (float)m / 8.f) * ldexpf(1.f, ef - 7);
}

/* src/nanochat/model/fp8/mx_kernel.cuh:42-44 */
int64_t mxo_scale_index(int64_t row, int64_t block, int64_t tiles) {
  return ((row >> 7) * tiles + (block >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (block & 3);
}

/* prologue: 0 none, 1 relu^2 (fp8_kernel.cu:44-50), 2 relu^2 backward from g = x, h (fp8_kernel.cu:154-168) */
static float prologue_value(float v, float h, int prologue) {
  if (prologue == 1) {
    const float r = v <= 0.f ? 0.f : v;
    return mxo_round_bf16(r * r);
  }
  if (prologue == 2) return mxo_round_bf16(h <= 0.f ? 0.f : v * (2.f * h));
  return v;
}

/* Quantize one direction. x (rows, cols) fp32 values; when transposed != 0 the stored matrix is x^T
 * (cols, rows) with blocks along x's rows. data has row stride ld; scale is swizzled with `tiles` tiles per
 * 128 stored rows. src/nanochat/model/fp8/mx_kernel.cuh:72-107. */
void mxo_quantize(const float* x, const float* h, int64_t rows, int64_t cols, int transposed, int prologue, int rule,
                  uint8_t* data, int64_t ld, uint8_t* scale, int64_t tiles) {
  const int64_t R = transposed ? cols : rows, C = transposed ? rows : cols;
  for (int64_t r = 0; r < R; ++r)
    for (int64_t b = 0; b < C / 32; ++b) {
      float v[32], amax = 0.f;
      for (int k = 0; k < 32; ++k) {
        const int64_t c = b * 32 + k;
        const int64_t i = transposed ? c * cols + r : r * cols + c;
        v[k] = prologue_value(x[i], h ? h[i] : 0.f, prologue);
        amax = fmaxf(amax, fabsf(v[k])); /* fmaxf skips NaN */
      }
      const int e = mxo_exponent(amax, rule);
      const float mul = mxo_multiplier(e);
      for (int k = 0; k < 32; ++k) data[r * ld + b * 32 + k] = mxo_e4m3(v[k] * mul);
      scale[mxo_scale_index(r, b, tiles)] = (uint8_t)e;
    }
}

/* (R, C) bytes + swizzled scales -> fp32 (tests/test_fp8.cpp:43-49) */
void mxo_dequantize(const uint8_t* data, const uint8_t* scale, int64_t R, int64_t C, float* out) {
  const int64_t tiles = C / 128;
  for (int64_t r = 0; r < R; ++r)
    for (int64_t c = 0; c < C; ++c) {
      const int e = scale[mxo_scale_index(r, c / 32, tiles)];
      out[r * C + c] = (float)((double)mxo_e4m3_to_f32(data[r * C + c]) * ldexp(1.0, e - 127));
    }
}

/* D[M,N] = alpha * deq(A)[M,K] . deq(B)[N,K]^T (+ D when accumulate), fp32
 * (src/nanochat/model/fp8/mx_gemm.h:18-22, 44-50). Accumulates in double: an order-free reference. */
void mxo_gemm_f32(const uint8_t* a, const uint8_t* a_scale, const uint8_t* b, const uint8_t* b_scale, float* d,
                  int64_t M, int64_t N, int64_t K, float alpha, int accumulate) {
  float* fa = (float*)malloc(sizeof(float) * M * K);
  float* fb = (float*)malloc(sizeof(float) * N * K);
  mxo_dequantize(a, a_scale, M, K, fa);
  mxo_dequantize(b, b_scale, N, K, fb);
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int64_t k = 0; k < K; ++k) acc += (double)fa[m * K + k] * (double)fb[n * K + k];
      const float v = alpha * (float)acc;
      d[m * N + n] = accumulate ? d[m * N + n] + v : v;
    }
  free(fa);
  free(fb);
}

/* bf16 output rounding of an fp32 accumulator, optional residual: bf16(float(bf16(acc)) + resid)
 * (src/nanochat/model/ops/residual_norm_kernel.cu:96-104) */
float mxo_bf16_out(float acc, int has_resid, float resid) {
  float o = mxo_round_bf16(acc);
  if (has_resid) o = mxo_round_bf16(o + resid);
  return o;
}

/* Fused residual add + lambda blend + RMS norm, one row at a time
 * (src/nanochat/model/ops/residual_norm_kernel.cu:80-128). Inputs and outputs are fp32 arrays holding bf16 values:
 *   s = r ? bf16(x + r) : x;  res = x0 ? bf16(bf16(lr_b * s) + bf16(l0_b * x0)) : s   (lr_b, l0_b = bf16 of the lambdas)
 *   rstd = 1 / sqrt(sum(res^2) / cols + eps);  n = bf16(res * rstd)
 * The sum of squares follows the kernel's order: 32 lanes, lane l accumulating columns (it * 32 + l) * 8 .. + 7 for
 * it = 0, 1, ... in fp32 (a bf16 square is exact in fp32, so fused and unfused multiply-add agree), then the
 * xor 16-8-4-2-1 butterfly, after which every lane holds the same total. The device's rsqrt is approximate, so a
 * caller that wants n bit for bit passes the device's rstd in rstd_in (null: computed here in double).
 * r, x0, s, n may be null. */
void mxo_residual_norm(const float* x, const float* r, const float* x0, float lr, float l0, int64_t rows, int cols,
                       float eps, const float* rstd_in, float* s, float* res, float* rstd, float* n) {
  const float lr_b = mxo_round_bf16(lr), l0_b = mxo_round_bf16(l0);
  for (int64_t row = 0; row < rows; ++row) {
    float lane_sum[32];
    for (int l = 0; l < 32; ++l) lane_sum[l] = 0.f;
    for (int it = 0; it * 256 < cols; ++it)
      for (int l = 0; l < 32; ++l) {
        const int col = (it * 32 + l) * 8;
        if (col >= cols) break;
        for (int k = 0; k < 8; ++k) {
          const int64_t i = row * cols + col + k;
          float v = x[i];
          if (r) {
            v = mxo_round_bf16(v + r[i]);
            if (s) s[i] = v;
          }
          if (x0) v = mxo_round_bf16(mxo_round_bf16(lr_b * v) + mxo_round_bf16(l0_b * x0[i]));
          res[i] = v;
          lane_sum[l] = v * v + lane_sum[l];
        }
      }
    for (int o = 16; o > 0; o >>= 1) {
      float next[32];
      for (int l = 0; l < 32; ++l) next[l] = lane_sum[l] + lane_sum[l ^ o];
      for (int l = 0; l < 32; ++l) lane_sum[l] = next[l];
    }
    const float mean = lane_sum[0] / (float)cols + eps;
    const float rs = rstd_in ? rstd_in[row] : (float)(1.0 / sqrt((double)mean));
    rstd[row] = rs;
    if (n)
      for (int c = 0; c < cols; ++c) n[row * cols + c] = mxo_round_bf16(res[row * cols + c] * rs);
  }
}

/* Loss pass of the chunked lm_head (src/nanochat/model/ops/softcap_ce_kernel.cu:62-103): per row of bf16 logits held as
 * fp32, lse = softcap + log(sum exp(softcap * tanh(z / softcap) - softcap)) over the first `vocab` columns and
 * loss = lse - capped[target]; target < 0: loss 0, lse untouched. Summed in the kernel's order (256 threads, thread t
 * takes columns t * 8 + 2048 * i + k, a butterfly per warp, then a butterfly over the 8 warp sums) with the host's
 * tanhf / expf / logf, which differ from the device's by a few ulp: this pins the structure, the tolerance is in the
 * tests. loss and lse may be null. */
void mxo_softcap_ce_loss(const float* logits, int64_t rows, int64_t ld, const int64_t* targets, int vocab, int padded,
                         float softcap, float* loss, float* lse) {
  for (int64_t row = 0; row < rows; ++row) {
    const float* z = logits + row * ld;
    const int64_t t = targets[row];
    if (t < 0) {
      if (loss) loss[row] = 0.f;
      continue;
    }
    float part[256];
    for (int th = 0; th < 256; ++th) {
      float s = 0.f;
      for (int j = th * 8; j < padded; j += 2048)
        for (int k = 0; k < 8; ++k)
          if (j + k < vocab) s += expf(softcap * tanhf(z[j + k] / softcap) - softcap);
      part[th] = s;
    }
    float warp[32];
    for (int w = 0; w < 32; ++w) warp[w] = 0.f;
    for (int w = 0; w < 8; ++w) {
      float lane[32];
      for (int l = 0; l < 32; ++l) lane[l] = part[w * 32 + l];
      for (int o = 16; o > 0; o >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ o];
        memcpy(lane, next, sizeof(lane));
      }
      warp[w] = lane[0];
    }
    for (int o = 16; o > 0; o >>= 1) {
      float next[32];
      for (int l = 0; l < 32; ++l) next[l] = warp[l] + warp[l ^ o];
      memcpy(warp, next, sizeof(warp));
    }
    const float l = softcap + logf(warp[0]);
    if (loss) loss[row] = l - softcap * tanhf(z[t] / softcap);
    if (lse) lse[row] = l;
  }
}

/* The gradient the quantizer's softcap prologue quantizes (softcap_ce_kernel.cu:49-54, 118-145), as bf16 values in
 * fp32: g = bf16((p - onehot) * (1 - th * th) * scale), th = tanh(z / softcap), p = exp(softcap * th - lse[row]);
 * scale = grad_scale ? grad_scale[row * stride] : 1, divided by num_valid when that is positive; rows with
 * target < 0 and columns >= vocab give 0. */
void mxo_softcap_ce_grad(const float* logits, int64_t rows, int64_t ld, const int64_t* targets, const float* lse,
                         int vocab, int padded, float softcap, const float* grad_scale, int64_t stride,
                         int64_t num_valid, float* g) {
  for (int64_t row = 0; row < rows; ++row) {
    const int64_t t = targets[row];
    float scale = grad_scale ? grad_scale[row * stride] : 1.f;
    if (num_valid > 0) scale /= (float)num_valid;
    for (int c = 0; c < padded; ++c) {
      float v = 0.f;
      if (t >= 0 && c < vocab) {
        const float th = tanhf(logits[row * ld + c] / softcap);
        const float p = expf(softcap * th - lse[row]);
        v = (p - (c == t ? 1.f : 0.f)) * (1.f - th * th) * scale;
      }
      g[row * padded + c] = mxo_round_bf16(v);
    }
  }
}
