// Fused residual add + lambda blend + RMS norm whose normalized output leaves MX-quantized in both layouts: the
// producer of the quantized input of the QKV and MLP-fc GEMMs. Replaces nanochat-cpp's
// nanochat_residual_norm_mx_fwd_c* (src/nanochat/model/ops/residual_norm_kernel.cu:153-214, launcher :330-349),
// same bits. Per row of `cols` bf16 values:
//   s = r ? bf16(x + r) : x;  res = x0 ? bf16(bf16(lr * s) + bf16(l0 * x0)) : s   (lr, l0 rounded to bf16 first)
//   rstd = rsqrt(sum(res^2) / cols + eps);  n = bf16(res * rstd);  MX(n) row-wise and column-wise
// The roundings are the reference's (residual_norm_kernel.cu:80-128). rstd is bit-exact only if the sum of squares
// is taken in the reference's order, so that part is fixed: a warp owns a row, lane l owns columns
// (it * 32 + l) * 8 .. + 7 for it = 0, 1, ..., accumulates them in order with fused multiply-adds, and the warp
// combines with the xor-16-8-4-2-1 butterfly. Everything around it is laid out for HBM: every global access is a
// 16- or 32-byte vector in a fully coalesced warp pattern, each input byte is read once and each output byte
// written once (x, r, x0: 2 B each; res, s: 2 B each; MX: 2 x (1 + 1/32) B per element).
//
// One CTA owns a tile of 32 rows (one scale block of the column-wise layout) x all columns, 8 warps x 4 rows each;
// the bf16 n values are parked in shared memory for the column pass, in which a thread owns two adjacent columns
// (packed 32-bit reads, conflict-free) and writes 32 contiguous bytes per transposed row.
#include <cuda_bf16.h>

#include "internal.h"
#include "mx_common.cuh"

namespace mxb200 {

namespace {

constexpr int kRows = 32;       // rows per tile
constexpr int kThreads = 256;     // two CTAs per SM: one tile's column pass overlaps the other's row loads
constexpr int kWarps = kThreads / 32;
constexpr int kVec = 8;         // bf16 per 16-byte load
constexpr int kMaxCols = 2048;

struct NormParams {
  mxb200_residual_norm_mx a;
  bool wide_out_t;
};

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16(v));
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[2 * k] = __uint_as_float(w[k] << 16);
    v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 raw;
  uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    w[k] = *reinterpret_cast<const uint32_t*>(&b);
  }
  return raw;
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ uint4 load16(const void* base, int64_t element) {
  return __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + element));
}

template <int kIters>
__global__ void __launch_bounds__(kThreads, 2) mxb200_residual_norm_mx_kernel(const NormParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const mxb200_residual_norm_mx& a = p.a;
  const int cols = a.cols;
  const int pitch = cols + kVec;  // bf16 elements per parked row: 16 bytes of padding keep row starts on distinct banks
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem);
  const int lane = static_cast<int>(threadIdx.x) & 31, warp = static_cast<int>(threadIdx.x) >> 5;
  const bool add = a.r != nullptr, blend = a.x0 != nullptr;
  const float lr = blend ? round_bf16(*a.lr) : 0.f, l0 = blend ? round_bf16(*a.l0) : 0.f;
  auto* out = static_cast<unsigned char*>(a.out.data);
  auto* out_scale = static_cast<unsigned char*>(a.out.scale);
  auto* out_t = static_cast<unsigned char*>(a.out_t.data);
  auto* out_t_scale = static_cast<unsigned char*>(a.out_t.scale);

  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRows; row0 < a.rows; row0 += static_cast<int64_t>(gridDim.x) * kRows) {
    // ---- rows: a warp per row, four rows per warp
    for (int r = warp; r < kRows; r += kWarps) {
      const int64_t row = row0 + r;
      float ss = 0.f;
      uint4 nv[kIters];
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        const int col = (it * 32 + lane) * kVec;
        if (col < cols) {
          const int64_t i = row * cols + col;
          // loads are issued per 256-column step; the compiler hoists as many as the register budget allows and
          // the SM's 16 warps cover the rest of the latency
          const uint4 xs = load16(a.x, i);
          uint4 rs = make_uint4(0, 0, 0, 0), x0s = make_uint4(0, 0, 0, 0);
          if (add)
            rs = load16(a.r, i);
          if (blend)
            x0s = load16(a.x0, i);
          float v[8];
          unpack8(xs, v);
          if (add) {
            float rv[8];
            unpack8(rs, rv);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              v[k] = round_bf16(v[k] + rv[k]);
            if (a.s != nullptr)
              reinterpret_cast<uint4*>(a.s)[i / kVec] = pack8(v);
          }
          if (blend) {
            float x0v[8];
            unpack8(x0s, x0v);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              v[k] = round_bf16(round_bf16(lr * v[k]) + round_bf16(l0 * x0v[k]));
          }
#pragma unroll
          for (int k = 0; k < 8; ++k)
            ss = fmaf(v[k], v[k], ss);
          nv[it] = pack8(v);
          reinterpret_cast<uint4*>(a.res)[i / kVec] = nv[it];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss / static_cast<float>(cols) + a.eps);
      if (lane == 0)
        a.rstd[row] = rstd;
      // n = bf16(res * rstd): parked for the column pass, quantized row-wise from registers (4 lanes per block)
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        const int col = (it * 32 + lane) * kVec;
        const bool active = col < cols;  // whole 4-lane groups: cols % 32 == 0
        float v[8] = {};
        float m = 0.f;
        uint4 packed = make_uint4(0, 0, 0, 0);
        if (active) {
          unpack8(nv[it], v);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            v[k] *= rstd;
          packed = pack8(v);
          unpack8(packed, v);
          *reinterpret_cast<uint4*>(tile + r * pitch + col) = packed;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            m = fmaxf(m, fabsf(v[k]));
        }
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        if (active) {
          const int e = mx_exponent(__float_as_uint(m), false);
          const float mul = __uint_as_float(mx_multiplier_bits(e));
          uint2 o;
          o.x = cvt_e4m3x4(v[0] * mul, v[1] * mul, v[2] * mul, v[3] * mul);
          o.y = cvt_e4m3x4(v[4] * mul, v[5] * mul, v[6] * mul, v[7] * mul);
          *reinterpret_cast<uint2*>(out + row * a.out.ld + col) = o;
          if ((lane & 3) == 0) {
            const int b = col >> 5;
            out_scale[(static_cast<int64_t>(row >> 7) * a.out.scale_tiles + (b >> 2)) * kScaleTileBytes +
                      mx_scale_tile_offset(static_cast<int>(row & 127), b)] = static_cast<unsigned char>(e);
          }
          if (col < a.n_cols)
            reinterpret_cast<uint4*>(a.n)[(row * cols + col) / kVec] = packed;
        }
      }
    }
    __syncthreads();

    // ---- columns: a thread owns two adjacent columns over the tile's 32 rows
    for (int cp = static_cast<int>(threadIdx.x); cp < cols / 2; cp += kThreads) {
      uint32_t w[kRows];
#pragma unroll
      for (int k = 0; k < kRows; ++k)
        w[k] = *reinterpret_cast<const uint32_t*>(tile + k * pitch + 2 * cp);
      float mlo = 0.f, mhi = 0.f;
#pragma unroll
      for (int k = 0; k < kRows; ++k) {
        mlo = fmaxf(mlo, fabsf(__uint_as_float(w[k] << 16)));
        mhi = fmaxf(mhi, fabsf(__uint_as_float(w[k] & 0xffff0000u)));
      }
      const int elo = mx_exponent(__float_as_uint(mlo), false), ehi = mx_exponent(__float_as_uint(mhi), false);
      const float mullo = __uint_as_float(mx_multiplier_bits(elo)), mulhi = __uint_as_float(mx_multiplier_bits(ehi));
      uint32_t qlo[8], qhi[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        qlo[k] = cvt_e4m3x4(__uint_as_float(w[4 * k] << 16) * mullo, __uint_as_float(w[4 * k + 1] << 16) * mullo,
                            __uint_as_float(w[4 * k + 2] << 16) * mullo, __uint_as_float(w[4 * k + 3] << 16) * mullo);
        qhi[k] = cvt_e4m3x4(__uint_as_float(w[4 * k] & 0xffff0000u) * mulhi,
                            __uint_as_float(w[4 * k + 1] & 0xffff0000u) * mulhi,
                            __uint_as_float(w[4 * k + 2] & 0xffff0000u) * mulhi,
                            __uint_as_float(w[4 * k + 3] & 0xffff0000u) * mulhi);
      }
      unsigned char* dst = out_t + static_cast<int64_t>(2 * cp) * a.out_t.ld + row0;
      if (p.wide_out_t) {
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(qlo[0]), "r"(qlo[1]), "r"(qlo[2]),
                     "r"(qlo[3]), "r"(qlo[4]), "r"(qlo[5]), "r"(qlo[6]), "r"(qlo[7])
                     : "memory");
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + a.out_t.ld), "r"(qhi[0]),
                     "r"(qhi[1]), "r"(qhi[2]), "r"(qhi[3]), "r"(qhi[4]), "r"(qhi[5]), "r"(qhi[6]), "r"(qhi[7])
                     : "memory");
      } else {
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(qlo[0], qlo[1], qlo[2], qlo[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(qlo[4], qlo[5], qlo[6], qlo[7]);
        reinterpret_cast<uint4*>(dst + a.out_t.ld)[0] = make_uint4(qhi[0], qhi[1], qhi[2], qhi[3]);
        reinterpret_cast<uint4*>(dst + a.out_t.ld)[1] = make_uint4(qhi[4], qhi[5], qhi[6], qhi[7]);
      }
      const int b = static_cast<int>(row0 >> 5);
      const int c0 = 2 * cp, c1 = 2 * cp + 1;
      out_t_scale[(static_cast<int64_t>(c0 >> 7) * a.out_t.scale_tiles + (b >> 2)) * kScaleTileBytes +
                  mx_scale_tile_offset(c0 & 127, b)] = static_cast<unsigned char>(elo);
      out_t_scale[(static_cast<int64_t>(c1 >> 7) * a.out_t.scale_tiles + (b >> 2)) * kScaleTileBytes +
                  mx_scale_tile_offset(c1 & 127, b)] = static_cast<unsigned char>(ehi);
    }
    __syncthreads();  // before the next tile overwrites the parked rows
  }
}

template <int kIters>
int launch(const NormParams& p, int sms, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(kRows) * (kIters * 256 + kVec) * sizeof(__nv_bfloat16);
  static std::atomic<int> configured_for{-1};
  int device = 0;
  cudaGetDevice(&device);
  if (smem > 48 * 1024 && configured_for.load() != device) {
    if (cudaFuncSetAttribute(mxb200_residual_norm_mx_kernel<kIters>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
    configured_for.store(device);
  }
  const int64_t tiles = p.a.rows / kRows;
  const int grid = static_cast<int>(std::min<int64_t>(tiles, 2 * static_cast<int64_t>(sms)));
  mxb200_residual_norm_mx_kernel<kIters><<<grid, kThreads, smem, stream>>>(p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}

}  // namespace

}  // namespace mxb200

extern "C" int mxb200_residual_norm_mx_fwd(const mxb200_residual_norm_mx* args, void* stream) {
  using namespace mxb200;
  DeviceInfo dev;
  if (int s = current_device(&dev); s != MXB200_OK)
    return s;
  if (args == nullptr)
    return MXB200_ERR_NULL;
  const mxb200_residual_norm_mx& a = *args;
  if (a.x == nullptr || a.res == nullptr || a.rstd == nullptr || a.out.data == nullptr || a.out.scale == nullptr ||
      a.out_t.data == nullptr || a.out_t.scale == nullptr || (a.x0 != nullptr && (a.lr == nullptr || a.l0 == nullptr)) ||
      (a.n_cols > 0 && a.n == nullptr))
    return MXB200_ERR_NULL;
  if (a.rows <= 0 || a.cols <= 0 || a.rows % 128 != 0 || a.cols % 128 != 0 || a.cols > kMaxCols || a.n_cols < 0 ||
      a.n_cols > a.cols || a.out.ld < a.cols || a.out_t.ld < a.rows ||
      a.out.scale_tiles < a.cols / 128 || a.out_t.scale_tiles < a.rows / 128)
    return MXB200_ERR_SHAPE;
  for (const void* ptr : {a.x, a.r, a.x0, static_cast<const void*>(a.s), static_cast<const void*>(a.res),
                          static_cast<const void*>(a.n), static_cast<const void*>(a.out.data),
                          static_cast<const void*>(a.out.scale), static_cast<const void*>(a.out_t.data),
                          static_cast<const void*>(a.out_t.scale)})
    if (ptr != nullptr && !aligned16(ptr))
      return MXB200_ERR_ALIGNMENT;
  if (a.out.ld % 16 != 0 || a.out_t.ld % 16 != 0)
    return MXB200_ERR_ALIGNMENT;
  NormParams p{a, (reinterpret_cast<uintptr_t>(a.out_t.data) & 31u) == 0 && a.out_t.ld % 32 == 0};
  auto* s = static_cast<cudaStream_t>(stream);
  switch ((a.cols + 255) / 256) {
    case 1: return launch<1>(p, dev.sms, s);
    case 2: return launch<2>(p, dev.sms, s);
    case 3: return launch<3>(p, dev.sms, s);
    case 4: return launch<4>(p, dev.sms, s);
    case 5: return launch<5>(p, dev.sms, s);
    case 6: return launch<6>(p, dev.sms, s);
    case 7: return launch<7>(p, dev.sms, s);
    default: return launch<8>(p, dev.sms, s);
  }
}
