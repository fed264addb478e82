// MX quantizer for sm_100a: bf16/fp32 -> E4M3 with one E8M0 scale per 32 values, row-wise and column-wise
// (transposed) in one pass over the input. Replaces nanochat-cpp's nanochat_mx_quantize_* kernels
// (src/nanochat/model/fp8/fp8_kernel.cu:197-210, body mx_kernel.cuh:72-107); same bytes, different schedule.
//
// One CTA owns a 128 x 128 tile, which is exactly one 512-byte swizzled scale tile in each layout.
//   row pass:    each thread loads 16 consecutive values with 256-bit loads (one for bf16, two for fp32), fully
//                coalesced; the block maximum of 32 values is a 2-lane shuffle (for plain bf16 input the
//                per-thread maximum and the multiply by the power-of-two scale stay packed bf16x2); 16 E4M3 bytes leave with one
//                128-bit store (a warp writes 512 contiguous bytes). The loaded values are parked in shared
//                memory in their input type (prologue values are bf16-exact).
//   column pass: each thread owns two adjacent columns x 32 rows, read from shared memory as packed pairs
//                (a warp reads 128 contiguous bytes per row, conflict-free), needs no shuffle, and writes
//                32 contiguous bytes of each transposed row with one 256-bit store (a full DRAM sector).
//   scales:      staged in shared memory in swizzled order and written as 16-byte vectors, 512 bytes per tile.
// HBM traffic is the algorithmic minimum: every input byte read once, every output byte written once.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "bf16x2_sm100.cuh"
#include "internal.h"
#include "mx_common.cuh"

namespace mxb200 {

namespace {

constexpr int kTile = 128;
constexpr int kThreads = 256;

enum Prologue : int { kNone = 0, kReluSquare = 1, kReluSquareBwd = 2, kSoftcapGrad = 3 };

// The softcap cross-entropy gradient prologue's inputs (src/nanochat/model/ops/softcap_ce_kernel.cu:118-145): x holds
// the chunk's logits, and per row a target, the log-sum-exp of its capped logits and an upstream scale.
struct SoftcapGrad {
  const int64_t* targets;
  const float* lse;
  const float* grad_scale;
  int64_t grad_scale_stride;
  const int64_t* num_valid;
  int vocab;
  float softcap;
};

struct QuantParams {
  const void* x;
  const void* h;  // relu^2 backward only
  int64_t cols;   // row stride of x (and h), elements
  mxb200_mx_out out, out_t;
  int tiles_c;
  bool floor_rule;
  bool wide_in;     // x is 32-byte aligned
  bool wide_out_t;  // out_t.data and its ld are 32-byte aligned
  SoftcapGrad ce;   // softcap gradient prologue only
};

// d loss_row / d z of one logit, before rounding: p = softmax of the capped logits, th = tanh(z / softcap). The
// expressions are the reference's (softcap_ce_kernel.cu:49-54), so the compiler contracts them the same way.
__device__ __forceinline__ float softcap_ce_grad(float z, bool is_target, float lse, float softcap, float scale) {
  const float th = tanhf(z / softcap);
  const float p = expf(softcap * th - lse);
  return (p - (is_target ? 1.f : 0.f)) * (1.f - th * th) * scale;
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16(v));
}

template <int kPro>
__device__ __forceinline__ float prologue(float v, float h) {
  if constexpr (kPro == kReluSquare) {
    const float r = v <= 0.f ? 0.f : v;
    return bf16_round(r * r);
  } else if constexpr (kPro == kReluSquareBwd) {
    return bf16_round(h <= 0.f ? 0.f : v * (2.f * h));
  } else {
    return v;
  }
}

__device__ __forceinline__ uint4 load_u4_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void store_u32x8(void* p, const uint32_t (&w)[8], bool wide) {
  if (wide) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  } else {
    reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// two floats -> two E4M3 bytes (RNE, saturating), lo in bits 0-7
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  return cvt_e4m3x2(a, b) | (cvt_e4m3x2(c, d) << 16);
}

__device__ __forceinline__ void load_u32x8_stream(const void* p, uint32_t (&w)[8], bool wide) {
  if (wide) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
  } else {
    const uint4 a = load_u4_stream(p), b = load_u4_stream(static_cast<const unsigned char*>(p) + 16);
    w[0] = a.x, w[1] = a.y, w[2] = a.z, w[3] = a.w, w[4] = b.x, w[5] = b.y, w[6] = b.z, w[7] = b.w;
  }
}

// kIn32: fp32 input (parked as float), else bf16 (parked as bf16).
// Row pass: a thread owns 16 consecutive values of a row (one 256-bit load of bf16), two lanes share a 32-value
// block (one shuffle), 16 E4M3 bytes leave with one 128-bit store (512 contiguous bytes per warp).
// One CTA's work: tile number `tile_index` (row-major over the tensor's 128 x 128 tiles) of the tensor p describes.
template <bool kIn32, int kPro>
__device__ __forceinline__ void quantize_tile(const QuantParams& p, int tile_index) {
  using Park = typename std::conditional<kIn32, float, __nv_bfloat16>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Park* tile = reinterpret_cast<Park*>(smem_raw);                               // [128][128]
  unsigned char* sc_rows = smem_raw + sizeof(Park) * kTile * kTile;             // 512 B, swizzled
  unsigned char* sc_cols = sc_rows + kScaleTileBytes;                           // 512 B, swizzled

  const int t = static_cast<int>(threadIdx.x);
  const int tile_r = tile_index / p.tiles_c, tile_c = tile_index % p.tiles_c;
  const int64_t row0 = static_cast<int64_t>(tile_r) * kTile, col0 = static_cast<int64_t>(tile_c) * kTile;
  const bool want_rows = p.out.data != nullptr, want_cols = p.out_t.data != nullptr;

  // ---- row pass: 128 rows x 8 vectors of 16 values = 1024 vectors, 4 per thread
  constexpr int kIters = kTile * (kTile / 16) / kThreads;
  constexpr int kWords = kIn32 ? 16 : 8;  // 32-bit words of input per 16 values
  uint32_t raw[kIters][kWords];
  uint32_t rawh[kPro == kReluSquareBwd ? kIters : 1][8];
  // all loads first: 4 (bf16) or 8 (fp32) independent 32-byte requests per thread in flight
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int q = it * kThreads + t, r = q >> 3, c = (q & 7) * 16;
    const int64_t i = (row0 + r) * p.cols + col0 + c;
    if constexpr (kIn32) {
      uint32_t lo[8], hi[8];
      load_u32x8_stream(static_cast<const float*>(p.x) + i, lo, p.wide_in);
      load_u32x8_stream(static_cast<const float*>(p.x) + i + 8, hi, p.wide_in);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        raw[it][k] = lo[k], raw[it][8 + k] = hi[k];
    } else {
      load_u32x8_stream(static_cast<const __nv_bfloat16*>(p.x) + i, raw[it], p.wide_in);
      if constexpr (kPro == kReluSquareBwd)
        load_u32x8_stream(static_cast<const __nv_bfloat16*>(p.h) + i, rawh[it], p.wide_in);
    }
  }
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int q = it * kThreads + t, r = q >> 3, c = (q & 7) * 16;
    float v[16];
    uint32_t m_bits;  // bits of this thread's max |v|
    if constexpr (kIn32) {
      float m = 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        v[k] = __uint_as_float(raw[it][k]);
        m = fmaxf(m, fabsf(v[k]));  // fmaxf drops NaN, as the reference's amax
      }
      m_bits = __float_as_uint(m);
      if (want_cols) {
        float4* dst = reinterpret_cast<float4*>(tile + r * kTile + c);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          dst[k] = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
      }
    } else {
      if constexpr (kPro != kNone) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[2 * k] = __uint_as_float(raw[it][k] << 16);
          v[2 * k + 1] = __uint_as_float(raw[it][k] & 0xffff0000u);
        }
      }
      if constexpr (kPro == kNone) {
        // the packed maximum skips NaN operands, as the reference's fmaxf does
        uint32_t m = 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          m = max_abs_skip_nan_bf16x2(m, raw[it][k]);
        m &= 0x7fff7fffu;
        m_bits = max(m & 0xffffu, m >> 16) << 16;
        if (want_cols) {
          uint4* dst = reinterpret_cast<uint4*>(tile + r * kTile + c);
          dst[0] = make_uint4(raw[it][0], raw[it][1], raw[it][2], raw[it][3]);
          dst[1] = make_uint4(raw[it][4], raw[it][5], raw[it][6], raw[it][7]);
        }
      } else {
        float m = 0.f;
        uint32_t pk[8];
        if constexpr (kPro == kSoftcapGrad) {
          // the gradient as the reference's grad kernel would have written it in bf16: 0 for ignored rows and for
          // the padding columns
          const int64_t grow = row0 + r;
          const int64_t target = p.ce.targets[grow];
          if (target < 0) {
#pragma unroll
            for (int k = 0; k < 16; ++k)
              v[k] = 0.f;
          } else {
            const float lse = p.ce.lse[grow];
            float scale = p.ce.grad_scale != nullptr ? p.ce.grad_scale[grow * p.ce.grad_scale_stride] : 1.f;
            if (p.ce.num_valid != nullptr)
              scale /= static_cast<float>(*p.ce.num_valid);
            const int64_t gcol = col0 + c;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const float g = gcol + k < p.ce.vocab ? softcap_ce_grad(v[k], gcol + k == target, lse, p.ce.softcap, scale) : 0.f;
              v[k] = bf16_round(g);
              m = fmaxf(m, fabsf(v[k]));
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            float hv = 0.f;
            if constexpr (kPro == kReluSquareBwd)
              hv = (k & 1) ? __uint_as_float(rawh[it][k >> 1] & 0xffff0000u) : __uint_as_float(rawh[it][k >> 1] << 16);
            v[k] = prologue<kPro>(v[k], hv);
            m = fmaxf(m, fabsf(v[k]));
          }
        }
        m_bits = __float_as_uint(m);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // prologue values are bf16-exact: repack by truncation
          pk[k] = (__float_as_uint(v[2 * k]) >> 16) | (__float_as_uint(v[2 * k + 1]) & 0xffff0000u);
        if (want_cols) {
          uint4* dst = reinterpret_cast<uint4*>(tile + r * kTile + c);
          dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
    }
    if (want_rows) {
      // non-negative float bits order as integers
      m_bits = max(m_bits, __shfl_xor_sync(0xffffffffu, m_bits, 1));
      const int e = mx_exponent(m_bits, p.floor_rule);
      uint4 o;
      if constexpr (!kIn32 && kPro == kNone) {
        // the multiplier is a power of two: the packed bf16 product is exact wherever e4m3 can tell
        const uint32_t mul2 = (mx_multiplier_bits(e) >> 16) * 0x10001u;
        o.x = e4m3x4_scaled(raw[it][0], raw[it][1], mul2);
        o.y = e4m3x4_scaled(raw[it][2], raw[it][3], mul2);
        o.z = e4m3x4_scaled(raw[it][4], raw[it][5], mul2);
        o.w = e4m3x4_scaled(raw[it][6], raw[it][7], mul2);
      } else {
        const float mul = __uint_as_float(mx_multiplier_bits(e));
        o.x = cvt_e4m3x4(v[0] * mul, v[1] * mul, v[2] * mul, v[3] * mul);
        o.y = cvt_e4m3x4(v[4] * mul, v[5] * mul, v[6] * mul, v[7] * mul);
        o.z = cvt_e4m3x4(v[8] * mul, v[9] * mul, v[10] * mul, v[11] * mul);
        o.w = cvt_e4m3x4(v[12] * mul, v[13] * mul, v[14] * mul, v[15] * mul);
      }
      *reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out.data) + (row0 + r) * p.out.ld + col0 + c) = o;
      if ((t & 1) == 0)
        sc_rows[mx_scale_tile_offset(r, c >> 5)] = static_cast<unsigned char>(e);
    }
  }
  __syncthreads();

  // ---- column pass: thread = (column pair, 32-row block)
  if (want_cols) {
    const int cp = t & 63, rb = t >> 6;
    uint32_t wlo[8], whi[8];
    int elo, ehi;
    if constexpr (kIn32) {
      float lo[32], hi[32];
      float mlo = 0.f, mhi = 0.f;
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const float2 f = *reinterpret_cast<const float2*>(tile + (rb * 32 + k) * kTile + 2 * cp);
        lo[k] = f.x, hi[k] = f.y;
        mlo = fmaxf(mlo, fabsf(lo[k]));
        mhi = fmaxf(mhi, fabsf(hi[k]));
      }
      elo = mx_exponent(__float_as_uint(mlo), p.floor_rule), ehi = mx_exponent(__float_as_uint(mhi), p.floor_rule);
      const float mullo = __uint_as_float(mx_multiplier_bits(elo)), mulhi = __uint_as_float(mx_multiplier_bits(ehi));
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        wlo[k] = cvt_e4m3x4(lo[4 * k] * mullo, lo[4 * k + 1] * mullo, lo[4 * k + 2] * mullo, lo[4 * k + 3] * mullo);
        whi[k] = cvt_e4m3x4(hi[4 * k] * mulhi, hi[4 * k + 1] * mulhi, hi[4 * k + 2] * mulhi, hi[4 * k + 3] * mulhi);
      }
    } else {
      // the two columns stay packed as bf16 pairs: 32 registers instead of 64, absmax on the 16-bit patterns
      uint32_t w[32];
#pragma unroll
      for (int k = 0; k < 32; ++k)
        w[k] = *reinterpret_cast<const uint32_t*>(tile + (rb * 32 + k) * kTile + 2 * cp);
      uint32_t m = 0u;
#pragma unroll
      for (int k = 0; k < 32; ++k)
        m = max_abs_skip_nan_bf16x2(m, w[k]);
      m &= 0x7fff7fffu;
      elo = mx_exponent((m & 0xffffu) << 16, p.floor_rule), ehi = mx_exponent(m & 0xffff0000u, p.floor_rule);
      // both columns scaled at once: powers of two, so the packed bf16 products are exact wherever e4m3 can tell
      const uint32_t mul2 = (mx_multiplier_bits(elo) >> 16) | (mx_multiplier_bits(ehi) & 0xffff0000u);
#pragma unroll
      for (int k = 0; k < 32; ++k)
        w[k] = mul_bf16x2(w[k], mul2);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        wlo[k] = cvt_e4m3x4(lo_f32(w[4 * k]), lo_f32(w[4 * k + 1]), lo_f32(w[4 * k + 2]), lo_f32(w[4 * k + 3]));
        whi[k] = cvt_e4m3x4(hi_f32(w[4 * k]), hi_f32(w[4 * k + 1]), hi_f32(w[4 * k + 2]), hi_f32(w[4 * k + 3]));
      }
    }
    unsigned char* dst = static_cast<unsigned char*>(p.out_t.data) + (col0 + 2 * cp) * p.out_t.ld + row0 + rb * 32;
    store_u32x8(dst, wlo, p.wide_out_t);
    store_u32x8(dst + p.out_t.ld, whi, p.wide_out_t);
    sc_cols[mx_scale_tile_offset(2 * cp, rb)] = static_cast<unsigned char>(elo);
    sc_cols[mx_scale_tile_offset(2 * cp + 1, rb)] = static_cast<unsigned char>(ehi);
    __syncthreads();
  }

  // ---- scales: one 512-byte tile per layout, 16 bytes per thread
  if (t < 32) {
    if (want_rows)
      reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out.scale) +
                               (static_cast<int64_t>(tile_r) * p.out.scale_tiles + tile_c) * kScaleTileBytes)[t] =
            reinterpret_cast<const uint4*>(sc_rows)[t];
  } else if (t < 64) {
    if (want_cols)
      reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out_t.scale) +
                               (static_cast<int64_t>(tile_c) * p.out_t.scale_tiles + tile_r) * kScaleTileBytes)[t - 32] =
            reinterpret_cast<const uint4*>(sc_cols)[t - 32];
  }
}

// Several tensors in one launch: a weight matrix of a d12-d26 model is 36 to 700 tiles, under one or two waves of
// the machine, so a launch per weight is bound by its own ramp-up and tail (12 us for 14 MB). The tiles of up to
// kMaxBatch tensors are numbered through; a CTA finds its tensor by its first tile.
constexpr int kMaxBatch = 32;

struct BatchJob {
  const void* x;
  int64_t ld;
  mxb200_mx_out out, out_t;
  int tiles_c;
  int first_tile;
  bool wide_in, wide_out_t;
};

struct BatchParams {
  BatchJob jobs[kMaxBatch];
  int n;
  bool floor_rule;
};

// One CTA of the batched launch: finds its tensor by its first tile.
template <bool kIn32>
__device__ __forceinline__ void quantize_batch_tile(const BatchParams& bp) {
  int j = 0;
  const int tile = static_cast<int>(blockIdx.x);
  while (j + 1 < bp.n && tile >= bp.jobs[j + 1].first_tile)
    ++j;
  const BatchJob& job = bp.jobs[j];
  QuantParams p{job.x,      nullptr,         job.ld, job.out, job.out_t, job.tiles_c, bp.floor_rule,
                job.wide_in, job.wide_out_t, SoftcapGrad{}};
  quantize_tile<kIn32, kNone>(p, tile - job.first_tile);
}

}  // namespace
}  // namespace mxb200

// Kernels: global, non-template, plain mxb200_* names, as nanochat-cpp names its own
// (src/nanochat/model/fp8/fp8_kernel.cu:174-175, 197-210). CTAs per SM: four for bf16 input, fewer where a prologue or
// fp32 input needs more registers or shared memory per CTA.
#define MXB200_QUANTIZE_KERNEL(name, IN32, PRO, CTAS)                                                                  \
  __global__ void __launch_bounds__(mxb200::kThreads, CTAS) name(const mxb200::QuantParams p) {                        \
    mxb200::quantize_tile<IN32, PRO>(p, static_cast<int>(blockIdx.x));                                                 \
  }
#define MXB200_QUANTIZE_BATCH_KERNEL(name, IN32, CTAS)                                                                 \
  __global__ void __launch_bounds__(mxb200::kThreads, CTAS) name(const __grid_constant__ mxb200::BatchParams bp) {     \
    mxb200::quantize_batch_tile<IN32>(bp);                                                                             \
  }

MXB200_QUANTIZE_KERNEL(mxb200_quantize_bf16, false, mxb200::kNone, 4)
MXB200_QUANTIZE_KERNEL(mxb200_quantize_f32, true, mxb200::kNone, 2)
MXB200_QUANTIZE_KERNEL(mxb200_quantize_relu_square, false, mxb200::kReluSquare, 4)
MXB200_QUANTIZE_KERNEL(mxb200_quantize_relu_square_bwd, false, mxb200::kReluSquareBwd, 3)
MXB200_QUANTIZE_KERNEL(mxb200_quantize_softcap_grad, false, mxb200::kSoftcapGrad, 2)
MXB200_QUANTIZE_BATCH_KERNEL(mxb200_quantize_batch_bf16, false, 4)
MXB200_QUANTIZE_BATCH_KERNEL(mxb200_quantize_batch_f32, true, 2)

namespace mxb200 {
namespace {

using QuantKernel = void (*)(QuantParams);
using QuantBatchKernel = void (*)(BatchParams);

template <bool kIn32, int kPro>
constexpr QuantKernel quantize_kernel() {
  if constexpr (kIn32)
    return mxb200_quantize_f32;
  else if constexpr (kPro == kReluSquare)
    return mxb200_quantize_relu_square;
  else if constexpr (kPro == kReluSquareBwd)
    return mxb200_quantize_relu_square_bwd;
  else if constexpr (kPro == kSoftcapGrad)
    return mxb200_quantize_softcap_grad;
  else
    return mxb200_quantize_bf16;
}

template <bool kIn32>
constexpr QuantBatchKernel quantize_batch_kernel() {
  return kIn32 ? mxb200_quantize_batch_f32 : mxb200_quantize_batch_bf16;
}

int check_out(const mxb200_mx_out& o, int64_t ld_min) {
  if (o.data == nullptr)
    return MXB200_OK;
  if (o.scale == nullptr)
    return MXB200_ERR_NULL;
  if (o.ld < ld_min || o.scale_tiles < ld_min / 128)
    return MXB200_ERR_SHAPE;
  if (!aligned16(o.data) || !aligned16(o.scale) || o.ld % 16 != 0)
    return MXB200_ERR_ALIGNMENT;
  return MXB200_OK;
}

template <bool kIn32, int kPro>
int launch(const QuantParams& p, int64_t tiles, cudaStream_t stream) {
  constexpr size_t smem = (kIn32 ? 4 : 2) * kTile * kTile + 2 * kScaleTileBytes;
  static std::atomic<int> configured_for{-1};
  int device = 0;
  cudaGetDevice(&device);
  if (smem > 48 * 1024 && configured_for.load() != device) {
    if (cudaFuncSetAttribute(quantize_kernel<kIn32, kPro>(), cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
    configured_for.store(device);
  }
  quantize_kernel<kIn32, kPro>()<<<static_cast<unsigned>(tiles), kThreads, smem, stream>>>(p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}

int quantize(const void* x, const void* h, bool x_bf16, int64_t rows, int64_t cols, mxb200_mx_out out,
             mxb200_mx_out out_t, int pro, int scale_rule, void* stream, const SoftcapGrad* ce = nullptr,
             int64_t ld = 0) {
  DeviceInfo dev;
  if (int s = current_device(&dev); s != MXB200_OK)
    return s;
  if (x == nullptr || (pro == kReluSquareBwd && h == nullptr))
    return MXB200_ERR_NULL;
  if (rows <= 0 || cols <= 0 || rows % kTile != 0 || cols % kTile != 0 || rows * cols / (kTile * kTile) > 0x7fffffffLL)
    return MXB200_ERR_SHAPE;
  if (scale_rule != MXB200_SCALE_REFERENCE && scale_rule != MXB200_SCALE_OCP_FLOOR)
    return MXB200_ERR_ARGUMENT;
  if (pro != kNone && !x_bf16)
    return MXB200_ERR_ARGUMENT;  // prologues read bf16 only, as the reference
  if (!aligned16(x) || (h != nullptr && !aligned16(h)))
    return MXB200_ERR_ALIGNMENT;
  if (int s = check_out(out, cols); s != MXB200_OK)
    return s;
  if (int s = check_out(out_t, rows); s != MXB200_OK)
    return s;
  if (out.data == nullptr && out_t.data == nullptr)
    return MXB200_OK;
  if (ld == 0)
    ld = cols;
  if (ld < cols || ld % 8 != 0)
    return MXB200_ERR_SHAPE;
  QuantParams p{x, h, ld, out, out_t, static_cast<int>(cols / kTile), scale_rule == MXB200_SCALE_OCP_FLOOR,
                (reinterpret_cast<uintptr_t>(x) & 31u) == 0 && ld % 16 == 0,
                (reinterpret_cast<uintptr_t>(out_t.data) & 31u) == 0 && out_t.ld % 32 == 0, SoftcapGrad{}};
  if (ce != nullptr)
    p.ce = *ce;
  const int64_t tiles = (rows / kTile) * (cols / kTile);
  auto* s = static_cast<cudaStream_t>(stream);
  if (!x_bf16)
    return launch<true, kNone>(p, tiles, s);
  switch (pro) {
    case kNone:
      return launch<false, kNone>(p, tiles, s);
    case kReluSquare:
      return launch<false, kReluSquare>(p, tiles, s);
    case kReluSquareBwd:
      return launch<false, kReluSquareBwd>(p, tiles, s);
    case kSoftcapGrad:
      return ce != nullptr ? launch<false, kSoftcapGrad>(p, tiles, s) : MXB200_ERR_NULL;
    default:
      return MXB200_ERR_ARGUMENT;
  }
}

template <bool kIn32>
int launch_batch(const BatchParams& bp, int tiles, cudaStream_t stream) {
  constexpr size_t smem = (kIn32 ? 4 : 2) * kTile * kTile + 2 * kScaleTileBytes;
  static std::atomic<int> configured_for{-1};
  int device = 0;
  cudaGetDevice(&device);
  if (smem > 48 * 1024 && configured_for.load() != device) {
    if (cudaFuncSetAttribute(quantize_batch_kernel<kIn32>(), cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
    configured_for.store(device);
  }
  quantize_batch_kernel<kIn32>()<<<static_cast<unsigned>(tiles), kThreads, smem, stream>>>(bp);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}

int quantize_batch(const mxb200_quantize_job* jobs, int n_jobs, bool x_bf16, int scale_rule, void* stream) {
  DeviceInfo dev;
  if (int s = current_device(&dev); s != MXB200_OK)
    return s;
  if (n_jobs < 0 || (n_jobs > 0 && jobs == nullptr))
    return MXB200_ERR_NULL;
  if (scale_rule != MXB200_SCALE_REFERENCE && scale_rule != MXB200_SCALE_OCP_FLOOR)
    return MXB200_ERR_ARGUMENT;
  // every job is checked before anything is launched
  for (int i = 0; i < n_jobs; ++i) {
    const mxb200_quantize_job& j = jobs[i];
    if (j.x == nullptr)
      return MXB200_ERR_NULL;
    if (j.rows <= 0 || j.cols <= 0 || j.rows % kTile != 0 || j.cols % kTile != 0 ||
        j.rows * j.cols / (kTile * kTile) > 0x3fffffffLL)
      return MXB200_ERR_SHAPE;
    if (!aligned16(j.x))
      return MXB200_ERR_ALIGNMENT;
    if (int s = check_out(j.out, j.cols); s != MXB200_OK)
      return s;
    if (int s = check_out(j.out_t, j.rows); s != MXB200_OK)
      return s;
  }
  auto* s = static_cast<cudaStream_t>(stream);
  int i = 0;
  while (i < n_jobs) {
    BatchParams bp{};
    bp.floor_rule = scale_rule == MXB200_SCALE_OCP_FLOOR;
    int64_t tiles = 0;
    while (i < n_jobs && bp.n < kMaxBatch) {
      const mxb200_quantize_job& j = jobs[i];
      const int64_t mine = (j.rows / kTile) * (j.cols / kTile);
      if (j.out.data == nullptr && j.out_t.data == nullptr) {  // nothing asked of this one
        ++i;
        continue;
      }
      if (tiles + mine > 0x7fffffffLL)
        break;
      bp.jobs[bp.n++] = BatchJob{j.x, j.cols, j.out, j.out_t, static_cast<int>(j.cols / kTile), static_cast<int>(tiles),
                                 (reinterpret_cast<uintptr_t>(j.x) & 31u) == 0,
                                 (reinterpret_cast<uintptr_t>(j.out_t.data) & 31u) == 0 && j.out_t.ld % 32 == 0};
      tiles += mine;
      ++i;
    }
    if (bp.n == 0)
      continue;
    const int st = x_bf16 ? launch_batch<false>(bp, static_cast<int>(tiles), s) : launch_batch<true>(bp, static_cast<int>(tiles), s);
    if (st != MXB200_OK)
      return st;
  }
  return MXB200_OK;
}

}  // namespace

}  // namespace mxb200

extern "C" int mxb200_quantize_mx_batch(const mxb200_quantize_job* jobs, int n_jobs, int x_bf16, int scale_rule,
                                        void* stream) {
  return mxb200::quantize_batch(jobs, n_jobs, x_bf16 != 0, scale_rule, stream);
}

extern "C" int mxb200_quantize_mx(const void* x, int x_bf16, int64_t rows, int64_t cols, mxb200_mx_out out,
                                  mxb200_mx_out out_t, int prologue, int scale_rule, void* stream) {
  if (prologue != MXB200_PROLOGUE_NONE && prologue != MXB200_PROLOGUE_RELU_SQUARE)
    return MXB200_ERR_ARGUMENT;
  return mxb200::quantize(x, nullptr, x_bf16 != 0, rows, cols, out, out_t, prologue, scale_rule, stream);
}

extern "C" int mxb200_quantize_mx_relu_square_bwd(const void* g, const void* h, int64_t rows, int64_t cols,
                                                  mxb200_mx_out out, mxb200_mx_out out_t, int scale_rule,
                                                  void* stream) {
  return mxb200::quantize(g, h, true, rows, cols, out, out_t, mxb200::kReluSquareBwd, scale_rule, stream);
}

extern "C" int mxb200_softcap_ce_grad_mx(const void* logits, int64_t rows, int64_t ld, const int64_t* targets,
                                         const float* lse, int vocab, int padded, float softcap,
                                         const float* grad_scale, int64_t grad_scale_stride, const int64_t* num_valid,
                                         mxb200_mx_out out, mxb200_mx_out out_t, int scale_rule, void* stream) {
  if (targets == nullptr || lse == nullptr)
    return MXB200_ERR_NULL;
  if (vocab <= 0 || vocab > padded || !(softcap > 0.f))
    return MXB200_ERR_ARGUMENT;
  const mxb200::SoftcapGrad ce{targets, lse, grad_scale, grad_scale_stride, num_valid, vocab, softcap};
  return mxb200::quantize(logits, nullptr, true, rows, padded, out, out_t, mxb200::kSoftcapGrad, scale_rule, stream,
                          &ce, ld);
}
