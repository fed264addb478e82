// MX quantizer for sm_100a: bf16/fp32 -> E4M3 with one E8M0 scale per 32 values, row-wise and column-wise
// (transposed) in one pass over the input. Replaces nanochat-cpp's nanochat_mx_quantize_* kernels
// (src/nanochat/model/fp8/fp8_kernel.cu:197-210, body mx_kernel.cuh:72-107); same bytes, different schedule.
//
// The unit of work is a 128 x 128 tile, which is exactly one 512-byte swizzled scale tile in each layout.
//   row pass:    each thread takes 16 consecutive values (256-bit loads, one for bf16, two for fp32, fully
//                coalesced); the block maximum of 32 values is a 2-lane shuffle (for plain bf16 input the per-thread
//                maximum stays packed bf16x2 and the multiply by the power-of-two scale is the mixed-precision
//                fp32 = bf16 * bf16 multiply-add, which takes the 16-bit halves as they are); 16 E4M3 bytes leave
//                with one 128-bit store (a warp writes 512 contiguous bytes). The loaded values are parked in
//                shared memory in their input type (prologue values are bf16-exact).
//   column pass: each thread owns two adjacent columns x 32 rows, read from shared memory as packed pairs
//                (a warp reads 128 contiguous bytes per row, conflict-free), needs no shuffle, and writes
//                32 contiguous bytes of each transposed row with one 256-bit store (a full DRAM sector).
//   scales:      staged in shared memory in swizzled order and written as 16-byte vectors, 512 bytes per tile.
// Two schedules: one CTA per tile (every input type and prologue; tensors of up to one wave), and for plain bf16
// tensors of more than one wave persistent CTAs that draw tiles from a counter and bring them in by TMA a tile ahead.
// HBM traffic is the algorithmic minimum: every input byte read once, every output byte written once.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "bf16x2_sm100.cuh"
#include "internal.h"
#include "mx_common.cuh"
#include "ptx_sm100.cuh"

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

// Column pass over a parked 128 x 128 tile: thread = (column pair, 32-row block); reads packed pairs (a warp reads 128
// contiguous bytes per row), writes 32 contiguous bytes of each transposed row and stages the two scale bytes.
template <bool kIn32>
__device__ __forceinline__ void column_pass(const typename std::conditional<kIn32, float, __nv_bfloat16>::type* tile,
                                            const QuantParams& p, int64_t row0, int64_t col0, unsigned char* sc_cols,
                                            int t) {
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
    // four running maxima, so that the chain of dependent instructions is 8 + 2 long instead of 32
    uint32_t m4[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int k = 0; k < 32; ++k)
      m4[k & 3] = max_abs_skip_nan_bf16x2(m4[k & 3], w[k]);
    uint32_t m = max_abs_skip_nan_bf16x2(max_abs_skip_nan_bf16x2(m4[0], m4[1]), max_abs_skip_nan_bf16x2(m4[2], m4[3]));
    m &= 0x7fff7fffu;
    elo = mx_exponent((m & 0xffffu) << 16, p.floor_rule), ehi = mx_exponent(m & 0xffff0000u, p.floor_rule);
    const uint16_t mlo = static_cast<uint16_t>(mx_multiplier_bits(elo) >> 16), mhi = static_cast<uint16_t>(mx_multiplier_bits(ehi) >> 16);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      e4m3x4_scaled_fma_split(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3], mlo, mhi, wlo[k], whi[k]);
  }
  unsigned char* dst = static_cast<unsigned char*>(p.out_t.data) + (col0 + 2 * cp) * p.out_t.ld + row0 + rb * 32;
  store_u32x8(dst, wlo, p.wide_out_t);
  store_u32x8(dst + p.out_t.ld, whi, p.wide_out_t);
  sc_cols[mx_scale_tile_offset(2 * cp, rb)] = static_cast<unsigned char>(elo);
  sc_cols[mx_scale_tile_offset(2 * cp + 1, rb)] = static_cast<unsigned char>(ehi);
}

// One 512-byte scale tile per layout leaves shared memory as 16-byte vectors (threads 0-31 rows, 32-63 columns).
__device__ __forceinline__ void write_scale_tiles(const QuantParams& p, int tile_r, int tile_c, const unsigned char* sc_rows,
                                                  const unsigned char* sc_cols, int t) {
  const bool want_rows = p.out.data != nullptr, want_cols = p.out_t.data != nullptr;
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

// kIn32: fp32 input (parked as float), else bf16 (parked as bf16).
// Row pass: a thread owns 16 consecutive values of a row (one 256-bit load of bf16), two lanes share a 32-value
// block (one shuffle), 16 E4M3 bytes leave with one 128-bit store (512 contiguous bytes per warp).
// One CTA's work: tile number `tile_index` (row-major over the tensor's 128 x 128 tiles) of the tensor p describes.
template <bool kIn32, int kPro>
__device__ __forceinline__ void quantize_tile(const QuantParams& p, int tile_index) {
  using Park = typename std::conditional<kIn32, float, __nv_bfloat16>::type;
  extern __shared__ __align__(128) unsigned char smem_raw[];
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
        const uint16_t mb = static_cast<uint16_t>(mx_multiplier_bits(e) >> 16);
        o.x = e4m3x4_scaled_fma(raw[it][0], raw[it][1], mb, mb);
        o.y = e4m3x4_scaled_fma(raw[it][2], raw[it][3], mb, mb);
        o.z = e4m3x4_scaled_fma(raw[it][4], raw[it][5], mb, mb);
        o.w = e4m3x4_scaled_fma(raw[it][6], raw[it][7], mb, mb);
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

  // ---- column pass, then the scales
  if (want_cols) {
    column_pass<kIn32>(tile, p, row0, col0, sc_cols, t);
    __syncthreads();
  }
  write_scale_tiles(p, tile_r, tile_c, sc_rows, sc_cols, t);
}

// ---- streaming form for plain bf16 input: persistent CTAs, tiles drawn from a counter and brought in by TMA
//
// The one-shot kernel above holds a tile's loads in registers, so a CTA reads, computes and writes in turn and only
// the other CTAs of its SM overlap with it. Here three CTAs per SM each keep two 32 KB tile buffers: while all threads
// work on one tile out of shared memory (no load or store instruction is spent on the input), the tiled TMA load of
// the next is in flight, marked evict-first in L2 because the input is read once. Tiles are handed out by a counter
// and not by a fixed stride: the CTAs of one SM advance at very different rates (with a fixed stride the first CTA of
// a 6144-tile tensor was done after 32 us and the last after 81), so a fixed share per CTA leaves most of the machine
// waiting for the slowest. Inside the benchmark step this form takes 27.5 us for a 16384 x 1536 activation and 61 us
// for the 16384 x 4608 gradient of the merged QKV, against 28.3 and 66.7 us for the one-shot kernel.
constexpr int kStreamStages = 2;
#define MXB200_STREAM_CTAS_PER_SM 3  // also the kernel's launch bound
constexpr int kStreamCtasPerSm = MXB200_STREAM_CTAS_PER_SM;
constexpr uint32_t kStreamTileBytes = kTile * kTile * 2;
constexpr uint64_t kStreamWaitLimitNs = 2000000000ull;
constexpr uint64_t kStreamDrainLimitNs = 50000000ull;

struct StreamBarriers {
  uint64_t full[kStreamStages];
  int tile_of[kStreamStages];  // the tile whose load completes full[s]; -1 is the stop sign
  uint32_t abort_flag;
};

// One pair of words per launch in flight, taken round-robin: the next tile to hand out and the CTAs that have left.
constexpr int kStreamSchedSlots = 256;

constexpr size_t kStreamSmemBytes = kStreamStages * kStreamTileBytes + 4 * kScaleTileBytes + sizeof(StreamBarriers);

}  // namespace

// Non-zero after a bounded wait of the streaming quantizer ran out: 0x40000000 | CTA << 8 | tile in the CTA's walk.
__device__ uint32_t g_quantize_watchdog_word;
__device__ uint32_t g_quantize_sched[2 * kStreamSchedSlots];

namespace {

__device__ __forceinline__ bool stream_wait(uint64_t* bar, uint32_t parity, StreamBarriers* bars, uint64_t limit_ns,
                                            uint32_t site) {
  if (mbar_try_wait(bar, parity))
    return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0) {
      if (*reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) != 0)
        return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) = 1;
        atomicCAS(&g_quantize_watchdog_word, 0u, 0x40000000u | (blockIdx.x << 8) | (site & 0xffu));
        return false;
      }
    }
  }
  return true;
}

// Row pass from a tile in shared memory. A thread owns 16 consecutive values (32 bytes) and reads them as two 16-byte
// vectors; lanes 4-7 of every eight take the upper vector first, so the eight lanes of a request cover all 32 banks.
__device__ __forceinline__ void stream_row_pass(const __nv_bfloat16* tile, const QuantParams& p, int64_t row0,
                                                int64_t col0, unsigned char* sc_rows, int t) {
  constexpr int kIters = kTile * (kTile / 16) / kThreads;
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int q = it * kThreads + t, r = q >> 3, piece = q & 7, c = piece * 16;
    const int swap = piece >> 2;
    const uint4* src = reinterpret_cast<const uint4*>(tile + r * kTile + c);
    const uint4 a = src[swap], b = src[swap ^ 1];
    uint32_t m = max_abs_skip_nan_bf16x2(
          max_abs_skip_nan_bf16x2(max_abs_skip_nan_bf16x2(a.x, a.y), max_abs_skip_nan_bf16x2(a.z, a.w)),
          max_abs_skip_nan_bf16x2(max_abs_skip_nan_bf16x2(b.x, b.y), max_abs_skip_nan_bf16x2(b.z, b.w)));
    m = max_abs_skip_nan_bf16x2(m, 0u);  // a lone NaN operand gives way to the zero, as in a running maximum from 0
    m &= 0x7fff7fffu;
    uint32_t m_bits = max(m & 0xffffu, m >> 16) << 16;
    m_bits = max(m_bits, __shfl_xor_sync(0xffffffffu, m_bits, 1));
    const int e = mx_exponent(m_bits, p.floor_rule);
    const uint16_t mb = static_cast<uint16_t>(mx_multiplier_bits(e) >> 16);
    const uint32_t a0 = e4m3x4_scaled_fma(a.x, a.y, mb, mb), a1 = e4m3x4_scaled_fma(a.z, a.w, mb, mb);
    const uint32_t b0 = e4m3x4_scaled_fma(b.x, b.y, mb, mb), b1 = e4m3x4_scaled_fma(b.z, b.w, mb, mb);
    const uint4 o = swap ? make_uint4(b0, b1, a0, a1) : make_uint4(a0, a1, b0, b1);
    *reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out.data) + (row0 + r) * p.out.ld + col0 + c) = o;
    if ((t & 1) == 0)
      sc_rows[mx_scale_tile_offset(r, c >> 5)] = static_cast<unsigned char>(e);
  }
}

struct StreamParams {
  QuantParams q;
  int tiles;
  int slot;
};

__device__ __forceinline__ void quantize_stream(const CUtensorMap* map_x, const StreamParams& sp) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* sc = smem_raw + kStreamStages * kStreamTileBytes;  // [2 tiles in turn][rows, columns][512]
  StreamBarriers* bars = reinterpret_cast<StreamBarriers*>(sc + 4 * kScaleTileBytes);
  const QuantParams& p = sp.q;
  const int t = static_cast<int>(threadIdx.x);
  const bool want_rows = p.out.data != nullptr, want_cols = p.out_t.data != nullptr;
  uint32_t* sched = g_quantize_sched + 2 * sp.slot;  // [0] next tile to hand out, [1] CTAs that have left

  if (t == 0) {
    for (int s = 0; s < kStreamStages; ++s)
      mbar_init(&bars->full[s], 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  // Thread 0 posts this CTA's i-th tile and starts its load into buffer i % stages. A number past the last tile is the
  // stop sign: posted once (a bare arrival completes the phase), after which nothing more is drawn or posted.
  // A CTA's first tile is its own number, so its first load does not wait for an atomic; every later tile comes from
  // the launch's counter, which starts at gridDim.x, and each draw is issued a whole tile before its number is needed
  // (the second tile's at the very start, behind the first load). Only one tile is fixed because a CTA may start late:
  // when another kernel (a collective on a side stream) holds SMs, the CTAs that do not fit wait until others have run
  // out of tiles, and whatever is fixed to them is then worked on after everything else.
  bool drawing = true;
  auto post = [&](int i, int tile) {
    const int s = i % kStreamStages;
    if (tile >= sp.tiles) {
      bars->tile_of[s] = -1;
      mbar_arrive(&bars->full[s]);
      drawing = false;
      return;
    }
    bars->tile_of[s] = tile;
    mbar_arrive_expect_tx(1u, &bars->full[s], kStreamTileBytes);
    tma_load_2d_hint(1u, smem_raw + s * kStreamTileBytes, map_x, &bars->full[s], (tile % p.tiles_c) * kTile,
                     (tile / p.tiles_c) * kTile, l2_policy_evict_first());
  };
  if (t == 0) {
    post(0, static_cast<int>(blockIdx.x));
    for (int i = 1; i < kStreamStages && drawing; ++i)
      post(i, static_cast<int>(gridDim.x + atomicAdd(&sched[0], 1u)));
  }

  int i = 0;
  for (;; ++i) {
    const int s = i % kStreamStages;
    int drawn = 0;  // thread 0: the tile of iteration i + stages, asked for now and posted after this tile
    if (t == 0 && drawing)
      drawn = static_cast<int>(gridDim.x + atomicAdd(&sched[0], 1u));
    const bool landed = stream_wait(&bars->full[s], static_cast<uint32_t>(i / kStreamStages) & 1u, bars,
                                    kStreamWaitLimitNs, static_cast<uint32_t>(i));
    const int tile = landed ? *reinterpret_cast<volatile int*>(&bars->tile_of[s]) : -1;
    const int tile_r = tile / p.tiles_c, tile_c = tile % p.tiles_c;
    const int64_t row0 = static_cast<int64_t>(tile_r) * kTile, col0 = static_cast<int64_t>(tile_c) * kTile;
    const __nv_bfloat16* buf = reinterpret_cast<const __nv_bfloat16*>(smem_raw + s * kStreamTileBytes);
    unsigned char* sc_rows = sc + (i & 1) * 2 * kScaleTileBytes;
    unsigned char* sc_cols = sc_rows + kScaleTileBytes;
    if (tile >= 0) {
      if (want_rows)
        stream_row_pass(buf, p, row0, col0, sc_rows, t);
      if (want_cols)
        column_pass<false>(buf, p, row0, col0, sc_cols, t);
    }
    // every thread is done with the buffer and the scale bytes are staged; the stop sign, or a wait that gave up,
    // ends the walk for all threads together
    if (__syncthreads_and(tile >= 0) == 0)
      break;
    if (t == 0 && drawing)
      post(i + kStreamStages, drawn);
    // the next tile stages its scale bytes in the other half, and the one after that comes after another barrier
    write_scale_tiles(p, tile_r, tile_c, sc_rows, sc_cols, t);
  }
  if (t == 0) {
    if (*reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) != 0) {
      // loads drawn and not taken may still land in this CTA's shared memory: give them a bounded time before leaving
      for (int j = i; j < i + kStreamStages; ++j) {
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(&bars->full[j % kStreamStages], static_cast<uint32_t>(j / kStreamStages) & 1u))
          if (global_timer_ns() - t0 > kStreamDrainLimitNs)
            break;
      }
    }
    // the last CTA to leave hands the slot back zeroed
    __threadfence();
    if (atomicAdd(&sched[1], 1u) == gridDim.x - 1) {
      sched[0] = 0u;
      sched[1] = 0u;
      __threadfence();
    }
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
// Streaming form: persistent, three CTAs per SM, each with two 32 KB tile buffers.
__global__ void __launch_bounds__(mxb200::kThreads, MXB200_STREAM_CTAS_PER_SM)
    mxb200_quantize_bf16_stream(const __grid_constant__ CUtensorMap map_x, const mxb200::StreamParams sp) {
  mxb200::quantize_stream(&map_x, sp);
}
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

// The streaming kernel on a plain bf16 tensor: (rows, ld) row-major behind a tiled map with a 128 x 128 box.
int launch_stream(const QuantParams& p, int64_t rows, int64_t cols, int64_t tiles, int sms, cudaStream_t stream) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr)
    return MXB200_ERR_DRIVER;
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.cols) * 2};
  const cuuint32_t box[2] = {kTile, kTile};
  const cuuint32_t estr[2] = {1, 1};
  if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p.x), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return MXB200_ERR_DRIVER;
  static std::atomic<int> configured_for{-1};
  int device = 0;
  cudaGetDevice(&device);
  if (configured_for.load() != device) {
    if (cudaFuncSetAttribute(mxb200_quantize_bf16_stream, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kStreamSmemBytes)) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
    configured_for.store(device);
  }
  static std::atomic<uint32_t> next_slot{0};
  const StreamParams sp{p, static_cast<int>(tiles), static_cast<int>(next_slot.fetch_add(1) % kStreamSchedSlots)};
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(tiles, kStreamCtasPerSm * static_cast<int64_t>(sms)));
  mxb200_quantize_bf16_stream<<<grid, kThreads, kStreamSmemBytes, stream>>>(map, sp);
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
      // more tiles than the one-shot kernel holds at once (4 CTAs per SM): stream them through persistent CTAs
      if (tiles > 4 * static_cast<int64_t>(dev.sms))
        return launch_stream(p, rows, cols, tiles, dev.sms, s);
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

namespace mxb200 {
uint32_t take_quantize_watchdog_word() {
  uint32_t w = 0;
  if (cudaMemcpyFromSymbol(&w, g_quantize_watchdog_word, sizeof(w)) != cudaSuccess)
    return 0;
  if (w != 0) {
    const uint32_t zero = 0;
    cudaMemcpyToSymbol(g_quantize_watchdog_word, &zero, sizeof(zero));
    static const uint32_t zeros[2 * kStreamSchedSlots] = {};
    cudaMemcpyToSymbol(g_quantize_sched, zeros, sizeof(zeros));
  }
  return w;
}
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
