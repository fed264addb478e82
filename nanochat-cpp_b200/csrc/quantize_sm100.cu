// MX quantizer for sm_100a: bf16/fp32 -> E4M3 with one E8M0 scale per 32 values, row-wise and column-wise
// (transposed) in one pass over the input. Replaces nanochat-cpp's nanochat_mx_quantize_* kernels
// (src/nanochat/model/fp8/fp8_kernel.cu:197-210, body mx_kernel.cuh:72-107); same bytes, different schedule.
//
// One CTA owns a 128 x 128 tile, which is exactly one 512-byte swizzled scale tile in each layout.
//   row pass:    each thread loads 8 consecutive values with one 128-bit (bf16) or 256-bit (fp32) load, fully
//                coalesced; the block maximum of 32 values is a 4-lane shuffle reduction; 8 E4M3 bytes leave
//                with one 64-bit store (a warp writes 256 contiguous bytes). The loaded values are parked in
//                shared memory in their input type (prologue values are bf16-exact).
//   column pass: each thread owns two adjacent columns x 32 rows, read from shared memory as packed pairs
//                (a warp reads 128 contiguous bytes per row, conflict-free), needs no shuffle, and writes
//                32 contiguous bytes of each transposed row with one 256-bit store (a full DRAM sector).
//   scales:      staged in shared memory in swizzled order and written as 16-byte vectors, 512 bytes per tile.
// HBM traffic is the algorithmic minimum: every input byte read once, every output byte written once.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "internal.h"
#include "mx_common.cuh"

namespace mxb200 {

namespace {

constexpr int kTile = 128;
constexpr int kThreads = 256;

enum Prologue : int { kNone = 0, kReluSquare = 1, kReluSquareBwd = 2 };

struct QuantParams {
  const void* x;
  const void* h;  // relu^2 backward only
  int64_t cols;   // row stride of x (and h), elements
  mxb200_mx_out out, out_t;
  int tiles_c;
  bool floor_rule;
  bool wide_in;     // x is 32-byte aligned
  bool wide_out_t;  // out_t.data and its ld are 32-byte aligned
};

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

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = __uint_as_float(w[k] << 16);
    v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
  }
}

// wide: the address is 32-byte aligned (one 256-bit access); the interface only promises 16 bytes
__device__ __forceinline__ void load_f32x8(const float* p, float (&v)[8], bool wide) {
  if (wide) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(p));
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
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

// kIn32: fp32 input (parked as float), else bf16 (parked as bf16).
template <bool kIn32, int kPro>
__global__ void __launch_bounds__(kThreads) mxb200_quantize_kernel(const QuantParams p) {
  using Park = typename std::conditional<kIn32, float, __nv_bfloat16>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Park* tile = reinterpret_cast<Park*>(smem_raw);                               // [128][128]
  unsigned char* sc_rows = smem_raw + sizeof(Park) * kTile * kTile;             // 512 B, swizzled
  unsigned char* sc_cols = sc_rows + kScaleTileBytes;                           // 512 B, swizzled

  const int t = static_cast<int>(threadIdx.x);
  const int tile_r = static_cast<int>(blockIdx.x) / p.tiles_c, tile_c = static_cast<int>(blockIdx.x) % p.tiles_c;
  const int64_t row0 = static_cast<int64_t>(tile_r) * kTile, col0 = static_cast<int64_t>(tile_c) * kTile;
  const bool want_rows = p.out.data != nullptr, want_cols = p.out_t.data != nullptr;

  // ---- row pass: 128 rows x 16 vectors of 8 values = 2048 vectors, 8 per thread
  constexpr int kIters = kTile * (kTile / 8) / kThreads;
  float v[kIters][8];
  {
    // all loads first: 8 independent 16/32-byte requests per thread in flight
    uint4 raw[kIn32 ? 1 : kIters], rawh[kPro == kReluSquareBwd ? kIters : 1];
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int q = it * kThreads + t, r = q >> 4, c = (q & 15) * 8;
      const int64_t i = (row0 + r) * p.cols + col0 + c;
      if constexpr (kIn32) {
        load_f32x8(static_cast<const float*>(p.x) + i, v[it], p.wide_in);
      } else {
        raw[it] = load_u4_stream(static_cast<const __nv_bfloat16*>(p.x) + i);
        if constexpr (kPro == kReluSquareBwd)
          rawh[it] = load_u4_stream(static_cast<const __nv_bfloat16*>(p.h) + i);
      }
    }
    if constexpr (!kIn32) {
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        unpack_bf16x8(raw[it], v[it]);
        if constexpr (kPro == kReluSquareBwd) {
          float hv[8];
          unpack_bf16x8(rawh[it], hv);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            v[it][k] = prologue<kPro>(v[it][k], hv[k]);
        } else if constexpr (kPro != kNone) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            v[it][k] = prologue<kPro>(v[it][k], 0.f);
        }
      }
    }
  }
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int q = it * kThreads + t, r = q >> 4, c = (q & 15) * 8;
    if (want_cols) {
      if constexpr (kIn32) {
        float4* dst = reinterpret_cast<float4*>(tile + r * kTile + c);
        dst[0] = make_float4(v[it][0], v[it][1], v[it][2], v[it][3]);
        dst[1] = make_float4(v[it][4], v[it][5], v[it][6], v[it][7]);
      } else {
        uint4 pk;
        pk.x = (__float_as_uint(v[it][0]) >> 16) | (__float_as_uint(v[it][1]) & 0xffff0000u);
        pk.y = (__float_as_uint(v[it][2]) >> 16) | (__float_as_uint(v[it][3]) & 0xffff0000u);
        pk.z = (__float_as_uint(v[it][4]) >> 16) | (__float_as_uint(v[it][5]) & 0xffff0000u);
        pk.w = (__float_as_uint(v[it][6]) >> 16) | (__float_as_uint(v[it][7]) & 0xffff0000u);
        *reinterpret_cast<uint4*>(tile + r * kTile + c) = pk;
      }
    }
    if (want_rows) {
      float m = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        m = fmaxf(m, fabsf(v[it][k]));  // fmaxf drops NaN, as the reference's amax
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const int e = mx_exponent(__float_as_uint(m), p.floor_rule);
      const float mul = __uint_as_float(mx_multiplier_bits(e));
      uint2 o;
      o.x = cvt_e4m3x4(v[it][0] * mul, v[it][1] * mul, v[it][2] * mul, v[it][3] * mul);
      o.y = cvt_e4m3x4(v[it][4] * mul, v[it][5] * mul, v[it][6] * mul, v[it][7] * mul);
      *reinterpret_cast<uint2*>(static_cast<unsigned char*>(p.out.data) + (row0 + r) * p.out.ld + col0 + c) = o;
      if ((t & 3) == 0)
        sc_rows[mx_scale_tile_offset(r, c >> 5)] = static_cast<unsigned char>(e);
    }
  }
  __syncthreads();

  // ---- column pass: thread = (column pair, 32-row block)
  if (want_cols) {
    const int cp = t & 63, rb = t >> 6;
    float lo[32], hi[32];
    float mlo = 0.f, mhi = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const Park* src = tile + (rb * 32 + k) * kTile + 2 * cp;
      if constexpr (kIn32) {
        const float2 f = *reinterpret_cast<const float2*>(src);
        lo[k] = f.x, hi[k] = f.y;
      } else {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(src);
        lo[k] = __uint_as_float(w << 16), hi[k] = __uint_as_float(w & 0xffff0000u);
      }
      mlo = fmaxf(mlo, fabsf(lo[k]));
      mhi = fmaxf(mhi, fabsf(hi[k]));
    }
    const int elo = mx_exponent(__float_as_uint(mlo), p.floor_rule), ehi = mx_exponent(__float_as_uint(mhi), p.floor_rule);
    const float mullo = __uint_as_float(mx_multiplier_bits(elo)), mulhi = __uint_as_float(mx_multiplier_bits(ehi));
    uint32_t wlo[8], whi[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      wlo[k] = cvt_e4m3x4(lo[4 * k] * mullo, lo[4 * k + 1] * mullo, lo[4 * k + 2] * mullo, lo[4 * k + 3] * mullo);
      whi[k] = cvt_e4m3x4(hi[4 * k] * mulhi, hi[4 * k + 1] * mulhi, hi[4 * k + 2] * mulhi, hi[4 * k + 3] * mulhi);
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
    if (cudaFuncSetAttribute(mxb200_quantize_kernel<kIn32, kPro>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
    configured_for.store(device);
  }
  mxb200_quantize_kernel<kIn32, kPro><<<static_cast<unsigned>(tiles), kThreads, smem, stream>>>(p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}

int quantize(const void* x, const void* h, bool x_bf16, int64_t rows, int64_t cols, mxb200_mx_out out,
             mxb200_mx_out out_t, int pro, int scale_rule, void* stream) {
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
  QuantParams p{x, h, cols, out, out_t, static_cast<int>(cols / kTile), scale_rule == MXB200_SCALE_OCP_FLOOR,
                (reinterpret_cast<uintptr_t>(x) & 31u) == 0,
                (reinterpret_cast<uintptr_t>(out_t.data) & 31u) == 0 && out_t.ld % 32 == 0};
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
    default:
      return MXB200_ERR_ARGUMENT;
  }
}

}  // namespace

}  // namespace mxb200

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
