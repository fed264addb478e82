// Block-scaled MXFP8 GEMM for sm_100a: D[M,N] = A[M,K] . B[N,K]^T, E4M3 operands with one E8M0 scale per 32
// values along K (cuBLAS-swizzled scale tiles), fp32 accumulation in tensor memory.
// Replaces nanochat-cpp's CUTLASS Sm120 kernels (src/nanochat/model/fp8/mx_gemm_kernel.cu:341-351) behind the
// same contract (mx_gemm_kernel.h:13-22); forward, dgrad and wgrad all use this one K-major x K-major layout.
//
// Structure (one CTA per SM, persistent over output tiles, 192 threads):
//   warp 0      producer: TMA loads of a 128 x 128-byte A tile and a BN x 128-byte B tile (128-byte swizzle)
//               plus untiled bulk copies of the 512-byte scale tiles, into a ring of shared-memory stages
//               guarded by full/empty mbarriers. Every load lands in the CTA that issued it.
//   warp 1      MMA issuer (one thread): per stage, tcgen05.cp moves the scale tiles into TMEM (4 columns per
//               128 rows, byte = K block), then four tcgen05.mma kind::mxf8f6f4.block_scale steps of K = 32;
//               tcgen05.commit releases the stage and, after the last K step, publishes the accumulator.
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulator (each warp its own 32-lane quarter), then bf16
//               (optional residual add with the reference's two roundings) or fp32 (=, +=, device alpha)
//               stores of 32 bytes per thread.
// Two accumulator buffers let the epilogue of tile i overlap the main loop of tile i+1. With BN = 256 they
// overlap by 32 TMEM columns ([0,256) and [224,480), scales at [480,492)); the epilogue drains the shared
// columns first and signals that separately, so the next main loop starts after one 32-column read.
// Split-K (weight gradients, K = tokens): partial tiles go to a caller-provided workspace and the CTA that
// finishes a tile last sums the slices in fixed order, so results are deterministic.
// Every wait is bounded: after kWaitLimitNs a wait records its site in a device word, raises a CTA-wide abort
// flag that all other waits poll, and the kernel drains and returns.
#include <algorithm>
#include <cmath>
#include <mutex>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "bf16x2_sm100.cuh"
#include "internal.h"
#include "mx_common.cuh"
#include "ptx_sm100.cuh"

namespace mxb200 {

// one watchdog word per device context (module-scope device variable: no allocation)
__device__ uint32_t g_watchdog_word;

// Split-K scratch for mxb200_gemm_splitk_static: lives in the library's own device image, so every GPU that
// loads the library holds these bytes until the process exits. In host code this name is only a handle for
// cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_splitk_scratch[MXB200_STATIC_SCRATCH_BYTES];

// Work counters of the CTA-pair kernel's tile scheduler: {next unit, pairs done} per launch slot, zero between
// launches (the last pair to leave a launch zeroes its slot, whether or not a bounded wait gave up on the way).
// Launches take slots round-robin, so kernels that overlap on one device (different streams) do not share one as
// long as fewer than kSchedLaunchSlots pair launches are in flight on the device at once.
constexpr int kSchedLaunchSlots = 1024;
__device__ uint32_t g_sched_words[2 * kSchedLaunchSlots];


namespace {

constexpr int kBM = 128;
constexpr int kBK = 128;  // bytes == elements; one 128-byte swizzle atom wide
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr uint32_t kTmemCols = 512;
constexpr uint64_t kWaitLimitNs = 2000000000ull;

enum OutKind : int { kOutBf16 = 0, kOutF32 = 1 };
// What the epilogue does besides (or instead of) writing the bf16 output.
enum Fuse : int {
  kFuseNone = 0,
  kFuseReluSquare = 1,     // h = bf16(acc) written; MX(bf16(relu(h)^2)) in both layouts written
  kFuseReluSquareBwd = 2,  // ga = bf16(acc) not written; MX(bf16(h > 0 ? ga * 2h : 0)) in both layouts written
};


// where a wait gave up (stored in the watchdog word's low byte)
enum WaitSite : uint32_t {
  kSiteProducerEmpty = 1,
  kSiteMmaFull = 2,
  kSiteMmaTmemEmpty = 3,
  kSiteMmaOverlap = 4,
  kSiteEpilogueFull = 5,
  kSiteEpilogueSync = 6,
  kSiteSchedEmpty = 7,
  kSiteSchedFull = 8,
};

template <int BN>
struct Config {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kSfbTiles = BN / 128;
  static constexpr uint32_t kABytes = kBM * kBK;
  static constexpr uint32_t kBBytes = BN * kBK;
  static constexpr uint32_t kSfBytes = kScaleTileBytes * (1 + kSfbTiles);
  // TMEM columns: two accumulator buffers, then scales of A (4 columns) and B (4 per 128 rows)
  static constexpr bool kOverlap = BN == 256;
  static constexpr uint32_t kAcc0 = 0;
  static constexpr uint32_t kAcc1 = kOverlap ? 224 : BN;
  static constexpr uint32_t kSfaCol = kOverlap ? 480 : 2 * BN;
  static constexpr uint32_t kSfbCol = kSfaCol + 4;
  static constexpr size_t kSmemBytes =
        1024 /* alignment slack */ + static_cast<size_t>(kStages) * (kABytes + kBBytes + kSfBytes) + 512 /* barriers */;
};

struct GemmParams {
  const uint8_t* a_scale;
  const uint8_t* b_scale;
  void* d;
  const void* resid;
  const float* alpha;
  float* partials;     // split-K: [tile][split][128 * BN] fp32
  uint32_t* counters;  // split-K: [tile], zero on entry, zero on exit
  int M, N, K;
  int tiles_m, tiles_n;
  int k_tiles_total;   // K / 128
  int k_tiles_split;   // K tiles per split
  int splits;
  int panel;           // n-tiles per raster panel
  int out_kind;
  int accumulate;
  bool wide;  // d and resid are 32-byte aligned: 256-bit global accesses
  // fused MX quantization of the output (CTA-pair kernel): scales of q (rows of the output) and of q_t (its
  // columns), each at its buffer's first tile, with the tiles-per-128-rows of each buffer; h_in: relu^2 backward
  uint8_t* q_scale;
  uint8_t* qt_scale;
  int q_scale_tiles, qt_scale_tiles;
  const void* h_in;
  bool floor_rule;
  int sched_slot;  // CTA-pair kernel: this launch's pair of words in g_sched_words
};

struct Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t overlap_free;
  uint64_t epi_sync;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t last_flag;
  uint32_t scale_done[2];  // fused quantizer, 256-wide tile: epilogue warps done with the tile in accumulator buffer 0 / 1
  // CTA-pair kernel, tile scheduler: the leader CTA's producer draws unit indices from a global counter and posts each
  // to both CTAs (sched_unit, sched_full); every other role of the pair reads it and reports to the leader's sched_empty
  uint64_t sched_full[4];
  uint64_t sched_empty[4];
  uint32_t sched_unit[4];
};
constexpr int kSchedSlots = 4;

__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, Barriers* bars, uint32_t site) {
  if (mbar_try_wait(bar, parity))
    return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0) {
      if (*reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) != 0)
        return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) = 1;
        atomicCAS(&g_watchdog_word, 0u, 0x80000000u | (blockIdx.x << 8) | site);
        return false;
      }
    }
  }
  return true;
}

// The same wait for a converged warp: every lane polls, the warp agrees on the outcome.
__device__ __forceinline__ bool wait_bounded_warp(uint64_t* bar, uint32_t parity, Barriers* bars, uint32_t site) {
  return __all_sync(0xffffffffu, wait_bounded(bar, parity, bars, site)) != 0;
}

// ... and with the barrier given as a shared-memory address
__device__ __forceinline__ bool wait_bounded_warp(uint32_t bar_addr, uint32_t parity, Barriers* bars, uint32_t site) {
  bool ok = true;
  if (!mbar_try_wait(bar_addr, parity)) {
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar_addr, parity)) {
      if ((++spins & 63u) == 0) {
        if (*reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) != 0) {
          ok = false;
          break;
        }
        if (global_timer_ns() - t0 > kWaitLimitNs) {
          *reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) = 1;
          atomicCAS(&g_watchdog_word, 0u, 0x80000000u | (blockIdx.x << 8) | site);
          ok = false;
          break;
        }
      }
    }
  }
  return __all_sync(0xffffffffu, ok) != 0;
}

struct TileCoord {
  int m, n, split, tile;
};

__device__ __forceinline__ TileCoord decode_unit(const GemmParams& p, int unit) {
  TileCoord c;
  c.tile = unit / p.splits;
  c.split = unit - c.tile * p.splits;
  const int panel_tiles = p.panel * p.tiles_m;
  const int pi = c.tile / panel_tiles, rem = c.tile - pi * panel_tiles;
  const int width = min(p.panel, p.tiles_n - pi * p.panel);
  c.m = rem / width;
  c.n = pi * p.panel + (rem - c.m * width);
  return c;
}

// 32 bytes to / from global memory: one 256-bit access when the address allows, else two 128-bit ones
// (the interface only promises 16-byte alignment).
__device__ __forceinline__ void store_u32x8(void* p, const uint32_t* w, bool wide) {
  if (wide) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  } else {
    reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

__device__ __forceinline__ void load_u32x8(const void* p, uint32_t* w, bool wide) {
  if (wide) {
    asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p)
                 : "memory");
  } else {
    const uint4 a = reinterpret_cast<const uint4*>(p)[0], b = reinterpret_cast<const uint4*>(p)[1];
    w[0] = a.x, w[1] = a.y, w[2] = a.z, w[3] = a.w, w[4] = b.x, w[5] = b.y, w[6] = b.z, w[7] = b.w;
  }
}

// L2-coherent read (partials written by other SMs)
__device__ __forceinline__ void load_u32x8_cg(const void* p, uint32_t* w) {
  asm volatile("ld.global.cg.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(p)
               : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// The output words of 32 consecutive columns of one row from fp32 values acc[32]: 16 words of packed bf16
// (optionally plus the residual, rounded twice as the reference's separate add) or 32 fp32 words (alpha, +=).
// `valid` guards the reads of resid / the old output.
__device__ __forceinline__ void compute_chunk(const GemmParams& p, float alpha, int64_t row, int col, const float* acc,
                                              bool valid, uint32_t* o) {
  const int64_t idx = row * p.N + col;
  if (p.out_kind == kOutBf16) {
    if (p.resid != nullptr && valid) {
      uint32_t rw[16];
      const auto* rp = static_cast<const __nv_bfloat16*>(p.resid) + idx;
      load_u32x8(rp, rw, p.wide);
      load_u32x8(rp + 16, rw + 8, p.wide);
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        // the reference's separate add: the GEMM's bf16 output, then bf16(x + r)
        const float y0 = __bfloat162float(__float2bfloat16(acc[2 * k]));
        const float y1 = __bfloat162float(__float2bfloat16(acc[2 * k + 1]));
        o[k] = pack_bf16x2(y0 + __uint_as_float(rw[k] << 16), y1 + __uint_as_float(rw[k] & 0xffff0000u));
      }
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k)
        o[k] = pack_bf16x2(acc[2 * k], acc[2 * k + 1]);
    }
  } else {
    const float* dp = static_cast<const float*>(p.d) + idx;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (p.accumulate && valid) {
        uint32_t old[8];
        load_u32x8(dp + 8 * g, old, p.wide);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          o[8 * g + k] = __float_as_uint(fmaf(alpha, acc[8 * g + k], __uint_as_float(old[k])));
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          o[8 * g + k] = __float_as_uint(alpha * acc[8 * g + k]);
      }
    }
  }
}

// compute_chunk, then 32-byte stores straight from the thread that owns the row.
__device__ __forceinline__ void write_chunk(const GemmParams& p, float alpha, int64_t row, int col, const float* acc) {
  const int64_t idx = row * p.N + col;
  uint32_t o[32];
  compute_chunk(p, alpha, row, col, acc, true, o);
  if (p.out_kind == kOutBf16) {
    auto* dp = static_cast<__nv_bfloat16*>(p.d) + idx;
    store_u32x8(dp, o, p.wide);
    store_u32x8(dp + 16, o + 8, p.wide);
  } else {
    float* dp = static_cast<float*>(p.d) + idx;
#pragma unroll
    for (int g = 0; g < 4; ++g)
      store_u32x8(dp + 8 * g, o + 8 * g, p.wide);
  }
}

// Final write of 8 consecutive output columns of one row (the split-K reduction's unit of work).
__device__ __forceinline__ void write_octet(const GemmParams& p, float alpha, int64_t row, int col, const float* acc) {
  const int64_t idx = row * p.N + col;
  if (p.out_kind == kOutBf16) {
    uint4 o;
    if (p.resid != nullptr) {
      const uint4 rw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.resid) + idx);
      const uint32_t r[4] = {rw.x, rw.y, rw.z, rw.w};
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float y0 = __bfloat162float(__float2bfloat16(acc[2 * k]));
        const float y1 = __bfloat162float(__float2bfloat16(acc[2 * k + 1]));
        w[k] = pack_bf16x2(y0 + __uint_as_float(r[k] << 16), y1 + __uint_as_float(r[k] & 0xffff0000u));
      }
      o = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                     pack_bf16x2(acc[6], acc[7]));
    }
    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.d) + idx) = o;
  } else {
    float* dp = static_cast<float*>(p.d) + idx;
    float o[8];
    if (p.accumulate) {
      const float4 a = reinterpret_cast<const float4*>(dp)[0], b = reinterpret_cast<const float4*>(dp)[1];
      const float old[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int k = 0; k < 8; ++k)
        o[k] = fmaf(alpha, acc[k], old[k]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        o[k] = alpha * acc[k];
    }
    reinterpret_cast<float4*>(dp)[0] = make_float4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<float4*>(dp)[1] = make_float4(o[4], o[5], o[6], o[7]);
  }
}

// A warp's 32 rows x 64 bytes leave through shared memory and one TMA store: each lane parks its row's 64 bytes
// (16-byte pieces placed by the 64-byte swizzle the tensor map expects, which also spreads the lanes over the
// banks), the warp syncs, one lane issues the store. The TMA engine writes whole contiguous row segments,
// where per-thread stores of one row each reach L2 as 32 scattered sectors per instruction and back up the SM's
// store path. `issue` false: rows or columns past the matrix, nothing to write.
__device__ __forceinline__ void store_rows_tma(const CUtensorMap* map_d, unsigned char* stage, int lane,
                                               const uint32_t* w, int x, int y, bool issue) {
  if (lane == 0)
    tma_store_wait_read<0>();  // the previous store from this buffer has been read out
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(stage + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
          make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && issue) {
    // the output is not read again by this kernel: it should leave L2 before the operands do
    tma_store_2d_hint(map_d, stage, x, y, l2_policy_evict_first());
    tma_store_commit();
  }
}

template <int BN>
__device__ __forceinline__ void one_cta_kernel_body(const CUtensorMap* map_a, const CUtensorMap* map_b,
                                                    const GemmParams& p) {
  using C = Config<BN>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* s_a = smem;
  unsigned char* s_b = s_a + C::kStages * C::kABytes;
  unsigned char* s_sf = s_b + C::kStages * C::kBBytes;  // per stage: A's tile, then B's tiles
  Barriers* bars = reinterpret_cast<Barriers*>(s_sf + C::kStages * C::kSfBytes);

  const int warp = static_cast<int>(threadIdx.x) >> 5, lane = static_cast<int>(threadIdx.x) & 31;
  const int total_units = p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], kEpilogueThreads);
    }
    mbar_init(&bars->overlap_free, kEpilogueThreads);
    mbar_init(&bars->epi_sync, kEpilogueThreads);
    bars->abort_flag = 0;
    bars->last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(map_a);
    prefetch_tensormap(map_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp, one lane issues)
    {
      const uint32_t el = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
        const TileCoord tc = decode_unit(p, unit);
        const int n_rows_left = p.N - tc.n * BN;
        const int sfb_tiles = n_rows_left >= BN ? C::kSfbTiles : n_rows_left / 128;
        const uint32_t tx = C::kABytes + C::kBBytes + kScaleTileBytes * (1 + sfb_tiles);
        const int k_begin = tc.split * p.k_tiles_split;
        const int k_end = min(k_begin + p.k_tiles_split, p.k_tiles_total);
        const uint8_t* sfa_src = p.a_scale + static_cast<int64_t>(tc.m) * p.k_tiles_total * kScaleTileBytes;
        const uint8_t* sfb_src = p.b_scale + static_cast<int64_t>(tc.n) * C::kSfbTiles * p.k_tiles_total * kScaleTileBytes;
        for (int kt = k_begin; kt < k_end; ++kt) {
          if (!wait_bounded_warp(&bars->empty[stage], phase ^ 1u, bars, kSiteProducerEmpty)) {
            ok = false;
            break;
          }
          uint64_t* full = &bars->full[stage];
          mbar_arrive_expect_tx(el, full, tx);
          tma_load_2d(el, s_a + stage * C::kABytes, map_a, full, kt * kBK, tc.m * kBM);
          tma_load_2d(el, s_b + stage * C::kBBytes, map_b, full, kt * kBK, tc.n * BN);
          unsigned char* sf = s_sf + stage * C::kSfBytes;
          bulk_load(el, sf, sfa_src + static_cast<int64_t>(kt) * kScaleTileBytes, kScaleTileBytes, full);
          for (int j = 0; j < sfb_tiles; ++j)
            bulk_load(el, sf + (1 + j) * kScaleTileBytes,
                      sfb_src + (static_cast<int64_t>(j) * p.k_tiles_total + kt) * kScaleTileBytes, kScaleTileBytes,
                      full);
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
    {
      const uint32_t el = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t local = 0;  // tiles this CTA has started
      bool ok = true;
      const uint32_t sfa_t = tmem_base + C::kSfaCol, sfb_t = tmem_base + C::kSfbCol;
      for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x, ++local) {
        const TileCoord tc = decode_unit(p, unit);
        const int n_rows_left = p.N - tc.n * BN;
        const int n_valid = n_rows_left >= BN ? BN : n_rows_left;
        const int sfb_tiles = n_valid / 128;
        const uint32_t idesc = make_idesc_mxf8(kBM, static_cast<uint32_t>(n_valid));
        const uint32_t buf = local & 1u, use = local >> 1;
        // the buffer's previous tile (two tiles ago) must be drained ...
        if (!wait_bounded_warp(&bars->tmem_empty[buf], (use & 1u) ^ 1u, bars, kSiteMmaTmemEmpty)) {
          ok = false;
          break;
        }
        // ... and, with overlapping buffers, the previous tile must have given up the shared columns
        if (C::kOverlap && local > 0) {
          if (!wait_bounded_warp(&bars->overlap_free, (local - 1) & 1u, bars, kSiteMmaOverlap)) {
            ok = false;
            break;
          }
        }
        tcgen05_fence_after_sync();
        const uint32_t acc_t = tmem_base + (buf ? C::kAcc1 : C::kAcc0);
        const int k_begin = tc.split * p.k_tiles_split;
        const int k_end = min(k_begin + p.k_tiles_split, p.k_tiles_total);
        for (int kt = k_begin; kt < k_end; ++kt) {
          if (!wait_bounded_warp(&bars->full[stage], phase, bars, kSiteMmaFull)) {
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint32_t sf_addr = smem_u32(s_sf + stage * C::kSfBytes);
          // scale tiles: 32 rows x 16 bytes, 8-row groups 128 bytes apart, no swizzle
          tcgen05_cp_32x128b_warpx4(el, sfa_t, make_smem_desc(sf_addr, 0, 128, 0));
          for (int j = 0; j < sfb_tiles; ++j)
            tcgen05_cp_32x128b_warpx4(el, sfb_t + 4 * j, make_smem_desc(sf_addr + (1 + j) * kScaleTileBytes, 0, 128, 0));
          // operand tiles: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
          const uint64_t a_desc = make_smem_desc(smem_u32(s_a + stage * C::kABytes), 16, 1024, 2);
          const uint64_t b_desc = make_smem_desc(smem_u32(s_b + stage * C::kBBytes), 16, 1024, 2);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) {
            // K = 32 per step: 32 bytes further into the swizzle atom; scale byte k of the 32-bit column
            tcgen05_mma_mxf8(el, acc_t, a_desc + 2 * k, b_desc + 2 * k, idesc_with_sf(idesc, k, k), sfa_t, sfb_t,
                             (kt > k_begin || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(el, &bars->empty[stage]);
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok)
          tcgen05_commit(el, &bars->tmem_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: 32 * (warp id % 4) ...
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float alpha = (p.out_kind == kOutF32 && p.alpha != nullptr) ? *p.alpha : 1.f;
    uint32_t local = 0, sync_phase = 0;
    bool ok = true;
    constexpr int kChunks = BN / 32;
    for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x, ++local) {
      const TileCoord tc = decode_unit(p, unit);
      const uint32_t buf = local & 1u, use = local >> 1;
      if (!wait_bounded(&bars->tmem_full[buf], use & 1u, bars, kSiteEpilogueFull)) {
        ok = false;
        break;
      }
      tcgen05_fence_after_sync();
      const uint32_t acc_t = tmem_base + lane_base + (buf ? C::kAcc1 : C::kAcc0);
      const int64_t row = static_cast<int64_t>(tc.m) * kBM + quarter * 32 + lane;
      const int col0 = tc.n * BN;
      float* part = p.splits > 1
                          ? p.partials + (static_cast<int64_t>(tc.tile) * p.splits + tc.split) * (kBM * BN) +
                                  static_cast<int64_t>(quarter * 32 + lane) * BN
                          : nullptr;
#pragma unroll 1
      for (int i = 0; i < kChunks; ++i) {
        // overlapping buffers: buffer 0 shares its last 32 columns, buffer 1 its first 32; drain those first
        const int c = (C::kOverlap && buf == 0) ? (i == 0 ? kChunks - 1 : i - 1) : i;
        uint32_t r[32];
        tmem_ld_32x32b_x32(acc_t + c * 32, r);
        tmem_ld_wait();
        if (C::kOverlap && i == 0) {
          tcgen05_fence_before_sync();
          mbar_arrive(&bars->overlap_free);
        }
        if (col0 + c * 32 < p.N) {
          if (part != nullptr) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
              store_u32x8(part + c * 32 + 8 * g, r + 8 * g, true);
          } else {
            write_chunk(p, alpha, row, col0 + c * 32, reinterpret_cast<const float*>(r));
          }
        }
      }
      tcgen05_fence_before_sync();
      mbar_arrive(&bars->tmem_empty[buf]);

      if (part != nullptr) {
        // split-K: publish this slice, then the last CTA to arrive for the tile sums all slices in order
        __threadfence();
        mbar_arrive(&bars->epi_sync);
        if (!wait_bounded(&bars->epi_sync, sync_phase, bars, kSiteEpilogueSync)) {
          ok = false;
          break;
        }
        sync_phase ^= 1u;
        if (threadIdx.x == 64) {
          const uint32_t prev = atomicAdd(&p.counters[tc.tile], 1u);
          const bool last = prev + 1 == static_cast<uint32_t>(p.splits);
          if (last)
            p.counters[tc.tile] = 0;  // ready for the next call
          *reinterpret_cast<volatile uint32_t*>(&bars->last_flag) = last ? 1u : 0u;
        }
        mbar_arrive(&bars->epi_sync);
        if (!wait_bounded(&bars->epi_sync, sync_phase, bars, kSiteEpilogueSync)) {
          ok = false;
          break;
        }
        sync_phase ^= 1u;
        const bool last = *reinterpret_cast<volatile uint32_t*>(&bars->last_flag) != 0;
        if (last) {
          __threadfence();
          const float* tile_part = p.partials + static_cast<int64_t>(tc.tile) * p.splits * (kBM * BN) +
                                   static_cast<int64_t>(quarter * 32 + lane) * BN;
#pragma unroll 1
          for (int c = 0; c < kChunks; ++c) {
            if (col0 + c * 32 >= p.N)
              break;
            float acc[32];
#pragma unroll
            for (int k = 0; k < 32; ++k)
              acc[k] = 0.f;
            for (int s = 0; s < p.splits; ++s) {
              const float* src = tile_part + static_cast<int64_t>(s) * (kBM * BN) + c * 32;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint32_t w[8];
                load_u32x8_cg(src + 8 * g, w);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                  acc[8 * g + k] += __uint_as_float(w[k]);
              }
            }
            write_chunk(p, alpha, row, col0 + c * 32, acc);
          }
        }
        // the flag is rewritten only after every thread has read it
        mbar_arrive(&bars->epi_sync);
        if (!wait_bounded(&bars->epi_sync, sync_phase, bars, kSiteEpilogueSync)) {
          ok = false;
          break;
        }
        sync_phase ^= 1u;
      }
    }
  }

  // teardown: on an abort give copies and MMAs in flight time to land before shared and tensor memory go away
  if (*reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}


// ------------------------------------------------------------------------------------------------ fused quantizer
//
// The MX quantizer run on a 32 x 32 block of the accumulator while it is still in registers, for the two GEMMs of
// the relu^2 MLP whose output only exists to be quantized (nanochat-cpp fuses the same two:
// cutlass_mx_gemm_relu_square / cutlass_mx_gemm_relu_square_bwd, src/nanochat/model/fp8/mx_gemm_kernel.cu:353-389,
// used at fp8.cpp:279-284, 318-323). Same bytes as the GEMM followed by mxb200_quantize_mx.
//   rows:    a thread holds its row's 32 columns = one scale block: no communication.
//   columns: the block goes through shared memory (bf16, the 64-byte-swizzled 2 KB tile the output store uses),
//            lane j then reads column j's 32 rows = one scale block of the transposed layout.
// Both results are parked as 32 rows x 32 bytes (16-byte halves placed by the 32-byte swizzle their tensor maps
// expect, which keeps the 16-byte stores of a quarter warp on distinct banks) and leave by TMA store; scale bytes go
// straight to their swizzled positions. The values stay packed bf16x2 throughout (bf16x2_sm100.cuh says why that
// gives the bits of the fp32-then-round form). Layout of `stage` (6 KB per warp): [0,2K) output rows, [2K,4K)
// transpose tile, [4K,5K) q, [5K,6K) q_t.

// The relu^2 backward form's second input: this lane's four 16-byte pieces of the 32 x 32 bf16 block of h at
// (warp_row0, col). Zeros outside the matrix.
__device__ __forceinline__ void load_h_pieces(const GemmParams& p, int lane, int warp_row0, int col, uint4* pieces) {
  const bool inside = warp_row0 < p.M && col < p.N;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = j * 8 + (lane >> 2), piece = lane & 3;
    pieces[j] = inside ? __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.h_in) +
                                                              (static_cast<int64_t>(warp_row0) + r) * p.N + col + piece * 8))
                       : make_uint4(0, 0, 0, 0);
  }
}

// Quantizes one scale block held as 16 packed words (32 bf16 in block order) into 32 e4m3 bytes w[8]; returns the
// block's biased exponent.
__device__ __forceinline__ int quantize_block(const uint32_t* v, int floor_rule, uint32_t* w) {
  // NaN operands are skipped, as by the quantizer's fmaxf; four running maxima keep the dependent chain short
  uint32_t m4[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int k = 0; k < 16; ++k)
    m4[k & 3] = max_abs_skip_nan_bf16x2(m4[k & 3], v[k]);
  uint32_t m = max_abs_skip_nan_bf16x2(max_abs_skip_nan_bf16x2(m4[0], m4[1]), max_abs_skip_nan_bf16x2(m4[2], m4[3]));
  m &= 0x7fff7fffu;
  const int e = mx_exponent(max(m & 0xffffu, m >> 16) << 16, floor_rule);
  const uint16_t mb = static_cast<uint16_t>(mx_multiplier_bits(e) >> 16);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    w[k] = e4m3x4_scaled_fma(v[2 * k], v[2 * k + 1], mb, mb);
  return e;
}

// Parks a block's 32 bytes as row `lane` of a 32 x 32-byte staging tile in the 32-byte swizzle (the 16-byte half
// index is xor-ed with bit 7 of the offset).
__device__ __forceinline__ void park_block(const uint32_t* w, unsigned char* st, int lane) {
  const int flip = ((lane >> 2) & 1) << 4;
  *reinterpret_cast<uint4*>(st + lane * 32 + flip) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4*>(st + lane * 32 + (flip ^ 16)) = make_uint4(w[4], w[5], w[6], w[7]);
}

template <int kFuse>
__device__ __forceinline__ void fused_quantize_chunk(const GemmParams& p, const CUtensorMap* map_d,
                                                     const CUtensorMap* map_q, const CUtensorMap* map_qt,
                                                     unsigned char* stage, int lane, const float* acc, int64_t row,
                                                     int col, int warp_row0, bool valid, uint4* h_pieces, int next_col,
                                                     unsigned char* scale_stage, int chunk) {
  unsigned char* st_out = stage;         // TMA source (forward form); h hand-over buffer (backward form, never a source)
  unsigned char* st_tr = stage + 2048;   // transpose tile, only ever touched by this warp's threads
  unsigned char* st_q = stage + 4096;    // TMA source
  unsigned char* st_qt = stage + 5120;   // TMA source
  // The previous chunk's TMA stores may still be reading st_out / st_q / st_qt: everything up to the point where those
  // are written again (all of the arithmetic) runs first, and only then does the warp wait for the reads to finish.

  // ---- the values to quantize: this thread's row of the block, 32 bf16 as 16 packed words
  uint32_t v[16];
  uint32_t o[kFuse == kFuseReluSquare ? 16 : 1];
  if constexpr (kFuse == kFuseReluSquare) {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      o[k] = pack_bf16x2_rn(acc[2 * k], acc[2 * k + 1]);
      const uint32_t r = relu_keep_nan_bf16x2(o[k]);
      v[k] = mul_bf16x2(r, r);
    }
  } else {
    // h's 32 x 32 block was loaded coalesced (load_h_pieces: 4 lanes per 64-byte row segment, 8 rows per
    // instruction, issued a chunk ahead) and is handed to the row owners through the otherwise unused output buffer;
    // the pieces' registers then take the next chunk's block (next_col >= 0), which has this whole chunk to arrive
    uint32_t hw[16];
    if (warp_row0 < p.M && col < p.N) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = j * 8 + (lane >> 2), piece = lane & 3;
        *reinterpret_cast<uint4*>(st_out + r * 64 + ((piece ^ ((r >> 1) & 3)) << 4)) = h_pieces[j];
      }
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 t = *reinterpret_cast<const uint4*>(st_out + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4));
        hw[4 * j] = t.x, hw[4 * j + 1] = t.y, hw[4 * j + 2] = t.z, hw[4 * j + 3] = t.w;
      }
      __syncwarp();  // all rows read before the next chunk's pieces overwrite them
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k)
        hw[k] = 0;
    }
    if (next_col >= 0)
      load_h_pieces(p, lane, warp_row0, next_col, h_pieces);
#pragma unroll
    for (int k = 0; k < 16; ++k) {  // dh = bf16(h <= 0 ? 0 : bf16(ga) * 2h)
      const uint32_t g = pack_bf16x2_rn(acc[2 * k], acc[2 * k + 1]);
      v[k] = mul_bf16x2(g, add_bf16x2(hw[k], hw[k])) & positive_or_nan_mask_bf16x2(hw[k]);
    }
  }

  // ---- columns, first half: into the transpose tile, 64 bytes per column (its 32 rows as bf16). A store instruction
  // puts one column's 32 rows there (32 lanes x 2 bytes, conflict-free); the 16-byte pieces of column c sit at piece
  // index xor (c >> 1) & 3, so that lane c then reads its column as four 16-byte vectors without bank conflicts.
  {
    unsigned char* mine[4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
      mine[x] = st_tr + ((((lane >> 3) ^ x) << 4) | ((lane & 7) << 1));
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      *reinterpret_cast<uint16_t*>(mine[k & 3] + (2 * k) * 64) = static_cast<uint16_t>(v[k]);
      *reinterpret_cast<uint16_t*>(mine[k & 3] + (2 * k + 1) * 64) = static_cast<uint16_t>(v[k] >> 16);
    }
  }
  __syncwarp();

  // ---- rows: this thread's 32 values are one block
  uint32_t wq[8];
  const int e_row = quantize_block(v, p.floor_rule, wq);

  // ---- columns, second half: lane c owns column c
  uint32_t wqt[8];
  int e_col;
  {
    uint32_t c[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 t = *reinterpret_cast<const uint4*>(st_tr + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4));
      c[4 * j] = t.x, c[4 * j + 1] = t.y, c[4 * j + 2] = t.z, c[4 * j + 3] = t.w;
    }
    e_col = quantize_block(c, p.floor_rule, wqt);
  }

  // ---- results out: data through the staging tiles; scale bytes into the CTA's shared-memory copy of its four scale
  // tiles (written out whole once the half tile is done: a byte store to global memory costs a 32-byte sector of
  // the SM's path to L2, a third more write traffic for the kernel), or, without one, straight to their swizzled
  // positions
  const int n = col + lane;  // row of the transposed layout
  if (scale_stage != nullptr) {
    const int t = chunk >> 2;  // which of the tile's two 128-column groups
    scale_stage[t * kScaleTileBytes + mx_scale_tile_offset(static_cast<int>(row & 127), chunk)] = static_cast<uint8_t>(e_row);
    scale_stage[(2 + t) * kScaleTileBytes + mx_scale_tile_offset(n & 127, warp_row0 >> 5)] = static_cast<uint8_t>(e_col);
  } else {
    if (valid) {
      const int b = col >> 5;
      p.q_scale[(static_cast<int64_t>(row >> 7) * p.q_scale_tiles + (b >> 2)) * kScaleTileBytes +
                mx_scale_tile_offset(static_cast<int>(row & 127), b)] = static_cast<uint8_t>(e_row);
    }
    if (warp_row0 < p.M && n < p.N) {
      const int b = warp_row0 >> 5;
      p.qt_scale[(static_cast<int64_t>(n >> 7) * p.qt_scale_tiles + (b >> 2)) * kScaleTileBytes +
                 mx_scale_tile_offset(n & 127, b)] = static_cast<uint8_t>(e_col);
    }
  }
  if (lane == 0)
    tma_store_wait_read<0>();  // the previous chunk's stores have been read out of the staging tiles
  __syncwarp();
  if constexpr (kFuse == kFuseReluSquare) {
#pragma unroll
    for (int j = 0; j < 4; ++j)  // h itself leaves as the plain epilogue's output does
      *reinterpret_cast<uint4*>(st_out + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
            make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
  }
  park_block(wq, st_q, lane);
  park_block(wqt, st_qt, lane);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && warp_row0 < p.M && col < p.N) {
    if constexpr (kFuse == kFuseReluSquare)
      tma_store_2d(map_d, st_out, col, warp_row0);
    tma_store_2d(map_q, st_q, col, warp_row0);
    tma_store_2d(map_qt, st_qt, warp_row0, col);
    tma_store_commit();
  }
}

// ------------------------------------------------------------------------------------------------ CTA-pair kernel
//
// Tile scheduler. The persistent pairs do not stride through the unit list: the leader CTA's producer warp draws the
// next unit from a global counter (one unit ahead, so the atomic's latency hides behind a tile's loads) and posts it
// in a 4-slot ring in both CTAs' shared memory; the other roles (peer producer, MMA warp, all epilogue warps) read
// each posting in order. A pair that starts late, because its SMs were busy with another kernel (a collective's
// CTAs on a side stream, say), then simply takes fewer units instead of holding the whole launch back with a fixed
// share. A drawn index at or past the number of units is the stop sign; the last pair to see it zeroes the counters
// for the next launch.

// One reader's step: waits for posting number `seq`, returns its unit, and frees the slot for this reader. Called by a
// whole warp. `arm`: this warp arms the peer CTA's copy of the barrier for the remote store (peer producer only).
__device__ __forceinline__ bool sched_read(Barriers* bars, uint32_t seq, bool arm, uint32_t empty_leader0, int lane,
                                           int* unit) {
  const uint32_t slot = seq & (kSchedSlots - 1), parity = (seq / kSchedSlots) & 1u;
  if (arm) {
    mbar_arrive_expect_tx(lane == 0 ? 1u : 0u, &bars->sched_full[slot], 4);
    __syncwarp();
  }
  if (!wait_bounded_warp(&bars->sched_full[slot], parity, bars, kSiteSchedFull))
    return false;
  int u = static_cast<int>(*reinterpret_cast<volatile uint32_t*>(&bars->sched_unit[slot]));
  u = __shfl_sync(0xffffffffu, u, 0);  // lane 0's load has returned before its arrival below is issued
  if (lane == 0)
    mbar_arrive_cluster(empty_leader0 + slot * 8);
  *unit = u;
  return true;
}

//
// Two CTAs on the SMs of one TPC (a cluster of 2) share one 256 x 256 output tile: tcgen05.mma.cta_group::2 reads
// 128 rows of A and 128 rows of B from each CTA's shared memory and leaves each CTA its own 128 rows of the
// accumulator in its own TMEM. Per K step every CTA therefore loads 16 KB of A and 16 KB of B for 128 x 256 x 128
// multiply-adds: half the L2-to-SM traffic per flop of the one-CTA kernel, and a 34 KB stage, so 6 stages fit.
// Both CTAs run the same three roles. Each loads its own halves (tiled loads, the byte counts credited to the
// leader's full barrier); only the leader (cluster rank 0) issues tcgen05.cp / tcgen05.mma, and its commits
// arrive on both CTAs' empty / tmem_full barriers; each CTA's epilogue drains its own TMEM and reports to the
// leader's tmem_empty / overlap barriers. Scale tiles come through tensor maps too, so rows past the end of a
// matrix read as zero scales (2^-127) against zero data instead of touching memory out of range.

// TN = 256: the widest tile (least L2 traffic per flop); its two accumulator buffers overlap by 32 columns, so
// the next tile's first MMA waits until the previous tile's epilogue has read those columns: a bubble of about
// 1500 cycles per tile, negligible for long K. TN = 192: two disjoint buffers, no bubble, for shapes with a
// short main loop. Scale tiles of B are loaded as the two 128-row tiles covering the tile's columns; the tile's
// first column is ((n * TN) % 128) / 32 TMEM columns into the first of them. That offset must be even: a scale
// address at an odd column (a tile starting 32 or 96 rows into a scale tile, as a 224-wide tiling would) is a
// misaligned-address fault, so tile widths are multiples of 64.
constexpr int kEpiStageBytes = 2048;       // one epilogue warp's staging buffer for TMA stores
constexpr int kEpiFusedBytes = 6144;       // ... with a fused quantizer: output rows, transpose tile, q rows, q_t rows

// Threads: producer warp, MMA warp, then the epilogue warps, kParts per TMEM lane quarter, each taking a share of the
// tile's 32-column chunks. The plain epilogue keeps up with the main loop with two per quarter. The fused quantizers
// execute several hundred instructions per chunk and thread and are bound by instruction latency, not by a pipe: a
// third warp per quarter fills the idle issue slots (128 registers per thread hold both forms without spills worth
// the name; a fourth would leave under 100).

template <int TN, int kFuse = kFuseNone>
struct PairConfig {
  static_assert(TN == 192 || TN == 256, "tile width");
  static constexpr int kEpiBytes = kFuse == kFuseNone ? kEpiStageBytes : kEpiFusedBytes;
  static constexpr int kParts = kFuse == kFuseNone ? 2 : 3;
  static constexpr int kEpiWarps = 4 * kParts;
  static constexpr int kEpiThreads = 32 * kEpiWarps;
  static constexpr int kThreads = 64 + kEpiThreads;
  static constexpr int kTileM = 256, kTileN = TN;
  static constexpr int kBRows = TN / 2;                // this CTA's rows of B
  static constexpr int kSfbTiles = 2;
  static constexpr uint32_t kABytes = 128 * kBK;       // this CTA's 128 rows of A
  static constexpr uint32_t kBBytes = kBRows * kBK;
  static constexpr uint32_t kSfBytes = kScaleTileBytes * (1 + kSfbTiles);  // A: own 128 rows; B: all its tiles
  static constexpr uint32_t kTxPerCta = kABytes + kBBytes + kSfBytes;
  static constexpr int kStages = (TN == 192 ? 7 : 6) - (kFuse == kFuseNone ? 0 : 2);
  static constexpr bool kOverlap = TN == 256;
  static constexpr uint32_t kAcc0 = 0, kAcc1 = kOverlap ? 224 : TN;
  static constexpr uint32_t kSfaCol = kOverlap ? 480 : 2 * TN, kSfbCol = kSfaCol + 4;
  // fused quantizer on the 256-wide tile: a CTA's 128 x 256 half tile is exactly two scale tiles of q and two of q_t
  // (512 bytes each), assembled in shared memory (one set per accumulator buffer) and written out whole
  static constexpr bool kStageScales = kFuse != kFuseNone && TN == 256;
  static constexpr int kScaleStageBytes = kStageScales ? 2 * 4 * kScaleTileBytes : 0;
  static constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * (kABytes + kBBytes + kSfBytes) +
                                       kEpiWarps * kEpiBytes + kScaleStageBytes + 512;
  static_assert(kSmemBytes <= 232448, "shared memory per CTA");
  static_assert(sizeof(Barriers) <= 512, "barrier block");
};

// The kernel body; the kernels themselves are the non-template functions at the end of this file (plain global
// names read the same in every profiler). The tensor maps stay in the kernels' parameter space and come by address.
template <int TN, int kFuse>
__device__ __forceinline__ void pair_kernel_body(const CUtensorMap* map_a, const CUtensorMap* map_b,
                                                 const CUtensorMap* map_sfa, const CUtensorMap* map_sfb,
                                                 const CUtensorMap* map_d, const CUtensorMap* map_part,
                                                 const CUtensorMap* map_q, const CUtensorMap* map_qt,
                                                 const GemmParams& p) {
  using C = PairConfig<TN, kFuse>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* s_a = smem;
  unsigned char* s_b = s_a + C::kStages * C::kABytes;
  unsigned char* s_epi = s_b + C::kStages * C::kBBytes;  // 2 KB per epilogue warp: 32 rows x 64 bytes
  unsigned char* s_sf = s_epi + C::kEpiWarps * C::kEpiBytes;  // per stage: A's tile, B's two tiles
  unsigned char* s_scales = s_sf + C::kStages * C::kSfBytes;  // fused quantizer: [buffer][q tile 0, 1, q_t tile 0, 1][512]
  Barriers* bars = reinterpret_cast<Barriers*>(s_scales + C::kScaleStageBytes);

  const int warp = static_cast<int>(threadIdx.x) >> 5, lane = static_cast<int>(threadIdx.x) & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_pairs = static_cast<int>(gridDim.x) >> 1;
  const int total_units = p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 2 * C::kEpiWarps);  // one arrival per epilogue warp of either CTA (leader's copy is used)
    }
    mbar_init(&bars->overlap_free, 8);  // the four warps per CTA that own the shared columns
    mbar_init(&bars->epi_sync, C::kEpiThreads);
    for (int i = 0; i < kSchedSlots; ++i) {
      mbar_init(&bars->sched_full[i], 1);
      // readers of a posted unit: the MMA warp, the peer's producer, and both CTAs' epilogue warps (leader's copy)
      mbar_init(&bars->sched_empty[i], 2 * C::kEpiWarps + 2);
    }
    bars->abort_flag = 0;
    bars->last_flag = 0;
    bars->scale_done[0] = bars->scale_done[1] = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(map_a);
    prefetch_tensormap(map_b);
    prefetch_tensormap(map_sfa);
    prefetch_tensormap(map_sfb);
    prefetch_tensormap(map_d);
    if (p.splits > 1)
      prefetch_tensormap(map_part);
    if (kFuse != kFuseNone) {
      prefetch_tensormap(map_q);
      prefetch_tensormap(map_qt);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_arrive();  // the peer's barriers exist before anything is credited to them
  cluster_wait();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs; one lane issues)
    // Shared-memory and barrier addresses advance by a constant per stage and wrap with the ring: the issuing
    // warp's per-stage instruction count is what bounds the pipeline once the MMA stream is saturated.
    {
      const uint32_t el = elect_one() ? 1u : 0u;
      const uint32_t el_leader = leader ? el : 0u;
      const uint32_t a0 = smem_u32(s_a), b0 = smem_u32(s_b), sf0 = smem_u32(s_sf);
      const uint32_t empty0 = smem_u32(&bars->empty[0]), full0 = smem_u32(&bars->full[0]);
      const uint32_t full_leader0 = map_to_cta(full0, 0);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      uint32_t* const sched = g_sched_words + 2 * p.sched_slot;
      const uint32_t sched_empty_leader0 = map_to_cta(smem_u32(&bars->sched_empty[0]), 0);
      const uint32_t sched_full_peer0 = map_to_cta(smem_u32(&bars->sched_full[0]), 1);
      const uint32_t sched_unit_peer0 = map_to_cta(smem_u32(&bars->sched_unit[0]), 1);
      int drawn = 0;  // leader: the unit drawn for the next posting
      if (leader) {
        if (lane == 0)
          drawn = static_cast<int>(atomicAdd(&sched[0], 1u));
        drawn = __shfl_sync(0xffffffffu, drawn, 0);
      }
      for (uint32_t seq = 0; ok; ++seq) {
        int unit;
        if (leader) {
          // post the drawn unit to both CTAs once every reader is done with the slot's previous posting
          const uint32_t slot = seq & (kSchedSlots - 1), parity = (seq / kSchedSlots) & 1u;
          if (!wait_bounded_warp(&bars->sched_empty[slot], parity ^ 1u, bars, kSiteSchedEmpty)) {
            ok = false;
            break;
          }
          unit = drawn;
          if (lane == 0) {
            *reinterpret_cast<volatile uint32_t*>(&bars->sched_unit[slot]) = static_cast<uint32_t>(unit);
            mbar_arrive(&bars->sched_full[slot]);  // release: the store above is visible to this CTA's readers
            st_async_u32(sched_unit_peer0 + slot * 4, static_cast<uint32_t>(unit), sched_full_peer0 + slot * 8);
            if (unit < total_units)  // draw one ahead: the round trip overlaps this unit's loads
              drawn = static_cast<int>(atomicAdd(&sched[0], 1u));
          }
          __syncwarp();
        } else if (!sched_read(bars, seq, true, sched_empty_leader0, lane, &unit)) {
          ok = false;
          break;
        }
        if (unit >= total_units)
          break;
        const TileCoord tc = decode_unit(p, unit);
        const int k_begin = tc.split * p.k_tiles_split;
        const int k_end = min(k_begin + p.k_tiles_split, p.k_tiles_total);
        const int row_a = tc.m * C::kTileM + static_cast<int>(rank) * 128;
        const int row_b = tc.n * C::kTileN + static_cast<int>(rank) * C::kBRows;
        const int sfa_tile = row_a >> 7, sfb_tile = (tc.n * C::kTileN) >> 7;
        for (int kt = k_begin; kt < k_end; ++kt) {
          if (!wait_bounded_warp(empty0 + stage * 8, phase ^ 1u, bars, kSiteProducerEmpty)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(el_leader, full0 + stage * 8, 2 * C::kTxPerCta);
          const uint32_t full = full_leader0 + stage * 8;
          const uint32_t sf = sf0 + stage * C::kSfBytes;
          tma_load_2d_pair(el, a0 + stage * C::kABytes, map_a, full, kt * kBK, row_a);
          tma_load_2d_pair(el, b0 + stage * C::kBBytes, map_b, full, kt * kBK, row_b);
          tma_load_4d_pair(el, sf, map_sfa, full, 0, 0, kt, sfa_tile);
          tma_load_4d_pair(el, sf + kScaleTileBytes, map_sfb, full, 0, 0, kt, sfb_tile);
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (leader)
          drawn = __shfl_sync(0xffffffffu, drawn, 0);
      }
      // the launch's last pair leaves the counters at zero for the next launch that takes this slot; every pair's
      // final draw (the one past the end) has happened before it counts itself done. A pair that gave up on a
      // bounded wait counts itself too: a slot must never stay part-way through a unit list.
      if (leader && lane == 0 && atomicAdd(&sched[1], 1u) == static_cast<uint32_t>(num_pairs) - 1u) {
        sched[0] = 0;
        sched[1] = 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader) {
      const uint32_t el = elect_one() ? 1u : 0u;
      uint32_t stage = 0, phase = 0;
      uint32_t local = 0;
      bool ok = true;
      const uint32_t sfa_t = tmem_base + C::kSfaCol, sfb_t = tmem_base + C::kSfbCol;
      const uint32_t idesc = make_idesc_mxf8(C::kTileM, C::kTileN);
      const uint32_t empty0 = smem_u32(&bars->empty[0]), full0 = smem_u32(&bars->full[0]);
      // operand tiles: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart; scale tiles: 32 rows x 16 bytes,
      // 8-row groups 128 bytes apart, no swizzle
      const uint64_t a_desc0 = make_smem_desc(smem_u32(s_a), 16, 1024, 2);
      const uint64_t b_desc0 = make_smem_desc(smem_u32(s_b), 16, 1024, 2);
      const uint64_t sf_desc0 = make_smem_desc(smem_u32(s_sf), 0, 128, 0);
      const uint32_t sched_empty_leader0 = map_to_cta(smem_u32(&bars->sched_empty[0]), 0);
      for (; ok; ++local) {
        int unit;
        if (!sched_read(bars, local, false, sched_empty_leader0, lane, &unit)) {
          ok = false;
          break;
        }
        if (unit >= total_units)
          break;
        const TileCoord tc = decode_unit(p, unit);
        const uint32_t buf = local & 1u, use = local >> 1;
        if (!wait_bounded_warp(&bars->tmem_empty[buf], (use & 1u) ^ 1u, bars, kSiteMmaTmemEmpty)) {
          ok = false;
          break;
        }
        if (C::kOverlap && local > 0 &&
            !wait_bounded_warp(&bars->overlap_free, (local - 1) & 1u, bars, kSiteMmaOverlap)) {
          ok = false;
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t acc_t = tmem_base + (buf ? C::kAcc1 : C::kAcc0);
        // the tile's first column is ((n * TN) % 128) / 32 scale columns into the first of B's two tiles
        const uint32_t sfb_mma = sfb_t + static_cast<uint32_t>(((tc.n * C::kTileN) & 127) >> 5);
        const int k_begin = tc.split * p.k_tiles_split;
        const int k_end = min(k_begin + p.k_tiles_split, p.k_tiles_total);
        for (int kt = k_begin; kt < k_end; ++kt) {
          if (!wait_bounded_warp(full0 + stage * 8, phase, bars, kSiteMmaFull)) {
            ok = false;
            break;
          }
          // descriptors of this stage: the ring's first stage plus a constant per stage (16-byte units)
          const uint64_t sf_desc = sf_desc0 + stage * (C::kSfBytes >> 4);
          tcgen05_cp_32x128b_warpx4_pair(el, sfa_t, sf_desc);
#pragma unroll
          for (int j = 0; j < C::kSfbTiles; ++j)
            tcgen05_cp_32x128b_warpx4_pair(el, sfb_t + 4 * j, sf_desc + (1 + j) * (kScaleTileBytes >> 4));
          const uint64_t a_desc = a_desc0 + stage * (C::kABytes >> 4);
          const uint64_t b_desc = b_desc0 + stage * (C::kBBytes >> 4);
          // K = 32 per step: 32 bytes (2 units) further into the swizzle atom; scale byte k of the 32-bit column
          tcgen05_mma_mxf8_pair(el, acc_t, a_desc, b_desc, idesc_with_sf(idesc, 0, 0), sfa_t, sfb_mma,
                                kt > k_begin ? 1u : 0u);
#pragma unroll
          for (uint32_t k = 1; k < 4; ++k)
            tcgen05_mma_mxf8_pair(el, acc_t, a_desc + 2 * k, b_desc + 2 * k, idesc_with_sf(idesc, k, k), sfa_t, sfb_mma,
                                  1u);
          tcgen05_commit_pair(el, empty0 + stage * 8, 3);  // frees this stage in both CTAs
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok)
          tcgen05_commit_pair(el, &bars->tmem_full[buf], 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2 and up, both CTAs)
    // A warp may read only the TMEM lanes of its quarter (warp id % 4); kParts warps share each quarter and take
    // a contiguous share of the tile's 32-column chunks each. TMEM loads are software-pipelined: the next 32
    // columns are in flight while the current 32 are converted and stored.
    const int quarter = warp & 3;
    const int col_part = (warp - 2) >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float alpha = (p.out_kind == kOutF32 && p.alpha != nullptr) ? *p.alpha : 1.f;
    uint32_t local = 0, sync_phase = 0;
    bool ok = true;
    constexpr int kChunks = C::kTileN / 32;
    constexpr int kMine = (kChunks + C::kParts - 1) / C::kParts;  // the most chunks any part takes
    constexpr int kHalf = 128 * C::kTileN;                        // elements of one CTA's half tile
    // part p takes chunks [first, first + n_mine): the remainder of kChunks / kParts goes to the leading parts
    const int n_mine = kChunks / C::kParts + (col_part < kChunks % C::kParts ? 1 : 0);
    const int first = col_part * (kChunks / C::kParts) + min(col_part, kChunks % C::kParts);
    constexpr int kLast = C::kParts - 1;
    const uint32_t empty_leader[2] = {map_to_cta(smem_u32(&bars->tmem_empty[0]), 0),
                                      map_to_cta(smem_u32(&bars->tmem_empty[1]), 0)};
    const uint32_t overlap_leader = map_to_cta(smem_u32(&bars->overlap_free), 0);
    unsigned char* stage = s_epi + (warp - 2) * C::kEpiBytes;
    const uint32_t sched_empty_leader0 = map_to_cta(smem_u32(&bars->sched_empty[0]), 0);
    for (; ok; ++local) {
      int unit;
      if (!sched_read(bars, local, false, sched_empty_leader0, lane, &unit)) {
        ok = false;
        break;
      }
      if (unit >= total_units)
        break;
      const TileCoord tc = decode_unit(p, unit);
      const uint32_t buf = local & 1u, use = local >> 1;
      // the relu^2 backward form reads h: the first chunk's block is requested before the accumulator is waited for
      uint4 h_pieces[4];
      if constexpr (kFuse == kFuseReluSquareBwd) {
        const int c0 = (C::kOverlap && buf == 0 && col_part == kLast) ? kChunks - 1 : first;
        load_h_pieces(p, lane, tc.m * C::kTileM + static_cast<int>(rank) * 128 + quarter * 32, tc.n * C::kTileN + c0 * 32,
                      h_pieces);
      }
      if (!wait_bounded(&bars->tmem_full[buf], use & 1u, bars, kSiteEpilogueFull)) {
        ok = false;
        break;
      }
      tcgen05_fence_after_sync();
      const uint32_t acc_t = tmem_base + lane_base + (buf ? C::kAcc1 : C::kAcc0);
      const int64_t row = static_cast<int64_t>(tc.m) * C::kTileM + rank * 128 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const int warp_row0 = tc.m * C::kTileM + static_cast<int>(rank) * 128 + quarter * 32;
      const int col0 = tc.n * C::kTileN;
      const int64_t half_index = (static_cast<int64_t>(tc.tile) * p.splits + tc.split) * 2 + rank;
      float* part = p.splits > 1 ? p.partials + half_index * kHalf + static_cast<int64_t>(quarter * 32 + lane) * C::kTileN
                                 : nullptr;
      // Overlapping buffers: buffer 0 shares its last 32 columns (owned by the last part), buffer 1 its first 32
      // (part 0). The owning warps read those first and hand them over before anything else.
      const bool owns_shared = C::kOverlap && (buf == 0 ? col_part == kLast : col_part == 0);
      auto chunk_of = [&](int i) {
        if (C::kOverlap && buf == 0 && col_part == kLast)
          return i == 0 ? kChunks - 1 : first + i - 1;
        return first + i;
      };
      uint32_t r[2][32];
      tmem_ld_32x32b_x32(acc_t + chunk_of(0) * 32, r[0]);
#pragma unroll
      for (int i = 0; i < kMine; ++i) {
        if (i >= n_mine)
          break;
        const int c = chunk_of(i);
        tmem_ld_wait();
        if (i + 1 < n_mine) {
          tmem_ld_32x32b_x32(acc_t + chunk_of(i + 1) * 32, r[(i + 1) & 1]);
        }
        if (i == 0 && owns_shared) {
          tcgen05_fence_before_sync();
          __syncwarp();
          if (lane == 0)
            mbar_arrive_cluster(overlap_leader);
        }
        const int col = col0 + c * 32;
        if (part != nullptr) {
          // split-K partials take the same TMA store path: the workspace is a (half tiles x 128 rows, TN) matrix
          const int part_row0 = static_cast<int>(half_index) * 128 + quarter * 32;
          store_rows_tma(map_part, stage, lane, r[i & 1], c * 32, part_row0, true);
          store_rows_tma(map_part, stage, lane, r[i & 1] + 16, c * 32 + 16, part_row0, true);
        } else if constexpr (kFuse != kFuseNone) {
          fused_quantize_chunk<kFuse>(p, map_d, map_q, map_qt, stage, lane, reinterpret_cast<const float*>(r[i & 1]),
                                      row, col, warp_row0, row_ok && col < p.N, h_pieces,
                                      i + 1 < n_mine ? col0 + chunk_of(i + 1) * 32 : -1,
                                      C::kStageScales ? s_scales + buf * (4 * kScaleTileBytes) : nullptr, c);
        } else {
          const bool valid = row_ok && col < p.N;
          const bool issue = warp_row0 < p.M && col < p.N;
          uint32_t o[32];
          compute_chunk(p, alpha, row, col, reinterpret_cast<const float*>(r[i & 1]), valid, o);
          store_rows_tma(map_d, stage, lane, o, col, warp_row0, issue);
          if (p.out_kind == kOutF32)
            store_rows_tma(map_d, stage, lane, o + 16, col + 16, warp_row0, issue);
        }
      }
      if constexpr (C::kStageScales) {
        // the warp that finishes the half tile last writes its four assembled scale tiles out, 16 bytes per lane and
        // step; the accumulator buffer (and with it this set of staged tiles) is handed back only after that
        __syncwarp();
        uint32_t prev = 0;
        if (lane == 0) {
          __threadfence_block();
          prev = atomicAdd(&bars->scale_done[buf], 1u);
        }
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == static_cast<uint32_t>(C::kEpiWarps) - 1u) {
          __threadfence_block();
          const unsigned char* src = s_scales + buf * (4 * kScaleTileBytes);
          const int row0 = tc.m * C::kTileM + static_cast<int>(rank) * 128;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int group = (col0 >> 7) + (t & 1);  // 128-column group of the output
            if (row0 < p.M && group * 128 < p.N) {
              uint8_t* dst = t < 2 ? p.q_scale + (static_cast<int64_t>(row0 >> 7) * p.q_scale_tiles + group) * kScaleTileBytes
                                   : p.qt_scale + (static_cast<int64_t>(group) * p.qt_scale_tiles + (row0 >> 7)) * kScaleTileBytes;
              reinterpret_cast<uint4*>(dst)[lane] = reinterpret_cast<const uint4*>(src + t * kScaleTileBytes)[lane];
            }
          }
          __syncwarp();
          if (lane == 0)
            *reinterpret_cast<volatile uint32_t*>(&bars->scale_done[buf]) = 0;
        }
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive_cluster(empty_leader[buf]);

      if (part != nullptr) {
        // split-K, per half tile: the rows of this CTA are reduced by whichever CTA finishes them last
        if (lane == 0) {
          tma_store_wait_all<0>();                       // this warp's partial stores have completed ...
          asm volatile("fence.proxy.async;" ::: "memory");  // ... and are ordered before generic-proxy traffic
        }
        __threadfence();
        mbar_arrive(&bars->epi_sync);
        if (!wait_bounded(&bars->epi_sync, sync_phase, bars, kSiteEpilogueSync)) {
          ok = false;
          break;
        }
        sync_phase ^= 1u;
        if (threadIdx.x == 64) {
          uint32_t* counter = &p.counters[tc.tile * 2 + rank];
          const uint32_t prev = atomicAdd(counter, 1u);
          const bool last = prev + 1 == static_cast<uint32_t>(p.splits);
          if (last)
            *counter = 0;
          *reinterpret_cast<volatile uint32_t*>(&bars->last_flag) = last ? 1u : 0u;
        }
        mbar_arrive(&bars->epi_sync);
        if (!wait_bounded(&bars->epi_sync, sync_phase, bars, kSiteEpilogueSync)) {
          ok = false;
          break;
        }
        sync_phase ^= 1u;
        const bool last = *reinterpret_cast<volatile uint32_t*>(&bars->last_flag) != 0;
        if (last) {
          // The reduction reads only the workspace, so it need not follow the TMEM lane mapping: a warp takes whole
          // rows, a lane 8 consecutive columns, and every load and store is a contiguous run across the warp.
          __threadfence();
          const float* half_base = p.partials + (static_cast<int64_t>(tc.tile) * p.splits * 2 + rank) * kHalf;
          const int sub = lane * 8;
          if (sub < C::kTileN && col0 + sub < p.N) {
#pragma unroll 1
            for (int rr = warp - 2; rr < 128; rr += C::kEpiWarps) {
              const int64_t grow = static_cast<int64_t>(tc.m) * C::kTileM + rank * 128 + rr;
              if (grow >= p.M)
                break;
              float acc[8];
#pragma unroll
              for (int k = 0; k < 8; ++k)
                acc[k] = 0.f;
              for (int sl = 0; sl < p.splits; ++sl) {  // slice order: the sum does not depend on who arrived last
                uint32_t w[8];
                load_u32x8_cg(half_base + static_cast<int64_t>(sl) * 2 * kHalf + rr * C::kTileN + sub, w);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                  acc[k] += __uint_as_float(w[k]);
              }
              write_octet(p, alpha, grow, col0 + sub, acc);
            }
          }
        }
        mbar_arrive(&bars->epi_sync);
        if (!wait_bounded(&bars->epi_sync, sync_phase, bars, kSiteEpilogueSync)) {
          ok = false;
          break;
        }
        sync_phase ^= 1u;
      }
    }
  }

  if (*reinterpret_cast<volatile uint32_t*>(&bars->abort_flag) != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  if (warp >= 2 && lane == 0)
    tma_store_wait_all<0>();  // this warp's output stores have left shared memory and reached global memory
  // neither CTA may leave while the other can still read its shared memory or signal its barriers
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace
}  // namespace mxb200

// ------------------------------------------------------------------------------------------------ kernels
//
// Global, non-template kernels with plain mxb200_* names, as nanochat-cpp names its own
// (src/nanochat/model/fp8/fp8_kernel.cu:174-175): a launch list or a timeline shows which tile shape and which
// epilogue ran without decoding template arguments. <rows>x<columns> is the output tile; the CTA-pair kernels share
// it between the two SMs of a TPC.
#define MXB200_GEMM_KERNEL(name, BN)                                                                                   \
  __global__ void __launch_bounds__(mxb200::kThreads, 1) name(const __grid_constant__ CUtensorMap map_a,               \
                                                              const __grid_constant__ CUtensorMap map_b,               \
                                                              const mxb200::GemmParams p) {                            \
    mxb200::one_cta_kernel_body<BN>(&map_a, &map_b, p);                                                                \
  }

#define MXB200_GEMM_PAIR_KERNEL(name, TN, FUSE)                                                                        \
  __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(mxb200::PairConfig<TN, FUSE>::kThreads, 1)               \
        name(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                     \
             const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,                 \
             const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_part,                  \
             const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_qt,                    \
             const mxb200::GemmParams p) {                                                                             \
    mxb200::pair_kernel_body<TN, FUSE>(&map_a, &map_b, &map_sfa, &map_sfb, &map_d, &map_part, &map_q, &map_qt, p);     \
  }

MXB200_GEMM_KERNEL(mxb200_gemm_128x128, 128)
MXB200_GEMM_KERNEL(mxb200_gemm_128x256, 256)
MXB200_GEMM_PAIR_KERNEL(mxb200_gemm_pair_256x192, 192, mxb200::kFuseNone)
MXB200_GEMM_PAIR_KERNEL(mxb200_gemm_pair_256x256, 256, mxb200::kFuseNone)
MXB200_GEMM_PAIR_KERNEL(mxb200_gemm_pair_256x192_relu_square, 192, mxb200::kFuseReluSquare)
MXB200_GEMM_PAIR_KERNEL(mxb200_gemm_pair_256x256_relu_square, 256, mxb200::kFuseReluSquare)
MXB200_GEMM_PAIR_KERNEL(mxb200_gemm_pair_256x192_relu_square_bwd, 192, mxb200::kFuseReluSquareBwd)
MXB200_GEMM_PAIR_KERNEL(mxb200_gemm_pair_256x256_relu_square_bwd, 256, mxb200::kFuseReluSquareBwd)

namespace mxb200 {
namespace {

using GemmKernel = void (*)(CUtensorMap, CUtensorMap, GemmParams);
using GemmPairKernel = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap,
                                CUtensorMap, GemmParams);

template <int BN>
constexpr GemmKernel one_cta_kernel() {
  return BN == 256 ? mxb200_gemm_128x256 : mxb200_gemm_128x128;
}

template <int TN, int kFuse>
constexpr GemmPairKernel pair_kernel() {
  if constexpr (kFuse == kFuseReluSquare)
    return TN == 256 ? mxb200_gemm_pair_256x256_relu_square : mxb200_gemm_pair_256x192_relu_square;
  else if constexpr (kFuse == kFuseReluSquareBwd)
    return TN == 256 ? mxb200_gemm_pair_256x256_relu_square_bwd : mxb200_gemm_pair_256x192_relu_square_bwd;
  else
    return TN == 256 ? mxb200_gemm_pair_256x256 : mxb200_gemm_pair_256x192;
}

// ------------------------------------------------------------------------------------------------ host side

// (rows, k) row-major bytes, box = box_rows x 128 bytes, 128-byte swizzle
int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr)
    return MXB200_ERR_DRIVER;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXB200_OK : MXB200_ERR_DRIVER;
}

// (M, N) row-major output, box = 32 rows x 64 bytes (32 bf16 or 16 fp32 columns), 64-byte swizzle: the shape one
// epilogue warp stores at a time.
int make_output_map(CUtensorMap* map, void* base, int64_t M, int64_t N, bool f32) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr)
    return MXB200_ERR_DRIVER;
  const cuuint64_t esize = f32 ? 4 : 2;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(N) * esize};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(64 / esize), 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXB200_OK : MXB200_ERR_DRIVER;
}

std::atomic<int> g_tile_n{0};
std::atomic<int> g_max_ctas{0};

// (rows / 128, k / 128) scale tiles of 32 x 16 bytes each, as a 4-D tensor {16, 32, k tiles, row tiles}; the box
// takes `tiles` row tiles of one k tile, i.e. tiles x 512 contiguous bytes in shared memory.
int make_scale_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int tiles) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr)
    return MXB200_ERR_DRIVER;
  const cuuint64_t kt = static_cast<cuuint64_t>(k / 128), rt = static_cast<cuuint64_t>(rows / 128);
  const cuuint64_t dims[4] = {16, 32, kt, rt};
  const cuuint64_t strides[3] = {16, 512, 512 * kt};
  const cuuint32_t box[4] = {16, 32, 1, static_cast<cuuint32_t>(tiles)};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXB200_OK : MXB200_ERR_DRIVER;
}

// How a shape is tiled: one-CTA kernel with 128 x 128 or 128 x 256 tiles, or the CTA-pair kernel with 256 x 192
// or 256 x 256.
struct TilePlan {
  bool pair;
  int tile_m, tile_n;
  int slots;         // tiles the machine runs at once
  int64_t tiles_m, tiles_n;
  int64_t tiles() const { return tiles_m * tiles_n; }
  size_t tile_bytes() const { return static_cast<size_t>(tile_m) * tile_n * sizeof(float); }
  int64_t counters() const { return tiles() * (pair ? 2 : 1); }
};

TilePlan plan_tiles(int64_t M, int64_t N, int64_t K, int sms, bool need_pair = false) {
  int forced = g_tile_n.load();
  if (need_pair && (forced == 128 || forced == 256))
    forced = 0;  // the fused-quantize epilogues exist in the CTA-pair kernel only
  TilePlan t{};
  if (forced == 512 || forced == 384 || need_pair || (forced == 0 && M >= 256 && N >= 256)) {
    t.pair = true, t.tile_m = 256, t.slots = std::max(sms / 2, 1);
    if (forced == 512) {
      t.tile_n = 256;
    } else if (forced == 384) {
      t.tile_n = 192;
    } else {
      // Estimated cycles: waves x (main loop + the hand-over between tiles). The main loop runs at the slower of
      // MMA execution (2 TN cycles per K step of 128) and what an SM can ingest (about 64 bytes per cycle); 256
      // pays an overlap bubble per tile. Measured on the d24 shapes this picks the faster width in every case,
      // including the long-K weight gradients whose tile count it raises past one wave (splitting K instead costs
      // more than it gains, see mxb200_gemm_splits).
      const int64_t k_iters = K / 128;
      double best = 0.0;
      for (int tn : {256, 192}) {
        const int64_t tiles = ((M + 255) / 256) * ((N + tn - 1) / tn);
        const int64_t units = tiles, iters = k_iters;
        // Pairs draw their tiles from a counter, so with many short tiles per pair the launch ends within a fraction
        // of a tile of the average share; with few long ones (the weight gradients) it ends on a whole round.
        const double share = static_cast<double>(units) / t.slots;
        const double waves = share >= 4.0 ? share + 0.25 : std::ceil(share);
        const double ingest = (16384.0 + tn * 64.0 + 1536.0) / 58.0;  // bytes a CTA loads per K step / (B/clk)
        const double per_tile = static_cast<double>(iters) * std::max(2.0 * tn, ingest) + (tn == 256 ? 1500.0 : 300.0);
        const double cost = waves * per_tile;
        if (best == 0.0 || cost < best * 0.995)
          best = cost, t.tile_n = tn;
      }
    }
  } else {
    t.pair = false, t.tile_m = 128, t.slots = std::max(sms, 1);
    t.tile_n = (forced == 128 || forced == 256) ? forced : (N >= 256 ? 256 : 128);
  }
  t.tiles_m = (M + t.tile_m - 1) / t.tile_m;
  t.tiles_n = (N + t.tile_n - 1) / t.tile_n;
  return t;
}

size_t counters_bytes(int64_t counters) {
  return static_cast<size_t>((counters * 4 + 255) / 256 * 256);
}

size_t workspace_bytes_for(const TilePlan& t, int splits) {
  return splits <= 1 ? 0 : counters_bytes(t.counters()) + static_cast<size_t>(t.tiles()) * splits * t.tile_bytes();
}

template <typename Kernel>
int set_smem_once(Kernel kernel, size_t bytes, bool* configured) {
  static std::mutex mu;
  int device = 0;
  cudaGetDevice(&device);
  std::lock_guard<std::mutex> lock(mu);
  if (device < 64 && !configured[device]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
    configured[device] = true;
  }
  return MXB200_OK;
}

template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int grid, cudaStream_t stream) {
  static bool configured[64] = {};
  if (int st = set_smem_once(one_cta_kernel<BN>(), Config<BN>::kSmemBytes, configured); st != MXB200_OK)
    return st;
  one_cta_kernel<BN>()<<<grid, kThreads, Config<BN>::kSmemBytes, stream>>>(ma, mb, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}

struct PairMaps {
  CUtensorMap a, b, sfa, sfb, d, part, q, qt;
};

template <int TN, int kFuse>
int launch_pair(const PairMaps& m, const GemmParams& p, int pairs, cudaStream_t stream) {
  using C = PairConfig<TN, kFuse>;
  static bool configured[64] = {};
  if (int st = set_smem_once(pair_kernel<TN, kFuse>(), C::kSmemBytes, configured); st != MXB200_OK)
    return st;
  pair_kernel<TN, kFuse>()<<<2 * pairs, C::kThreads, C::kSmemBytes, stream>>>(m.a, m.b, m.sfa, m.sfb, m.d,
                                                                                          m.part, m.q, m.qt, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}

template <int kFuse>
int launch_pair_width(int tile_n, const PairMaps& m, const GemmParams& p, int pairs, cudaStream_t stream) {
  return tile_n == 256 ? launch_pair<256, kFuse>(m, p, pairs, stream) : launch_pair<192, kFuse>(m, p, pairs, stream);
}

// (rows, cols) row-major bytes, box = 32 rows x 32 bytes: what one epilogue warp stores of a quantized layout
int make_bytes_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr)
    return MXB200_ERR_DRIVER;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols)};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXB200_OK : MXB200_ERR_DRIVER;
}

// Outputs of a fused-quantize GEMM (fuse != kFuseNone); see include/mxb200.h.
struct FusedOut {
  int fuse = kFuseNone;
  void* q = nullptr;
  void* q_scale = nullptr;
  void* q_t = nullptr;
  void* q_t_scale = nullptr;
  const void* h_in = nullptr;
};

int gemm(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d, int out_kind,
         const void* resid, int64_t M, int64_t N, int64_t K, const float* alpha, int accumulate, int splits,
         void* workspace, size_t workspace_bytes, void* stream, const FusedOut& fused = FusedOut{}) {
  DeviceInfo dev;
  if (int s = current_device(&dev); s != MXB200_OK)
    return s;
  const bool fusing = fused.fuse != kFuseNone;
  if (a == nullptr || a_scale == nullptr || b == nullptr || b_scale == nullptr ||
      (d == nullptr && fused.fuse != kFuseReluSquareBwd))
    return MXB200_ERR_NULL;
  if (fusing) {
    if (fused.q == nullptr || fused.q_scale == nullptr || fused.q_t == nullptr || fused.q_t_scale == nullptr ||
        (fused.fuse == kFuseReluSquareBwd && fused.h_in == nullptr))
      return MXB200_ERR_NULL;
    if (!aligned16(fused.q) || !aligned16(fused.q_scale) || !aligned16(fused.q_t) || !aligned16(fused.q_t_scale) ||
        (fused.h_in != nullptr && !aligned16(fused.h_in)))
      return MXB200_ERR_ALIGNMENT;
    if (out_kind != kOutBf16 || resid != nullptr || splits != 1)
      return MXB200_ERR_ARGUMENT;
  }
  if (M <= 0 || N <= 0 || K <= 0 || M % 128 != 0 || N % 128 != 0 || K % 128 != 0 || M > (1 << 30) || N > (1 << 30) ||
      K > (1 << 30))
    return MXB200_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(a_scale) || !aligned16(b) || !aligned16(b_scale) || (d != nullptr && !aligned16(d)) ||
      (resid != nullptr && !aligned16(resid)))
    return MXB200_ERR_ALIGNMENT;
  if (out_kind != kOutBf16 && out_kind != kOutF32)
    return MXB200_ERR_ARGUMENT;
  if (out_kind == kOutF32 && resid != nullptr)
    return MXB200_ERR_ARGUMENT;
  const int k_tiles = static_cast<int>(K / kBK);
  if (splits < 1 || splits > k_tiles || splits > 64)
    return MXB200_ERR_ARGUMENT;

  const TilePlan plan = plan_tiles(M, N, K, dev.sms, fusing);
  GemmParams p{};
  p.a_scale = static_cast<const uint8_t*>(a_scale);
  p.b_scale = static_cast<const uint8_t*>(b_scale);
  p.d = d;
  p.resid = out_kind == kOutBf16 ? resid : nullptr;
  p.alpha = out_kind == kOutF32 ? alpha : nullptr;
  p.M = static_cast<int>(M), p.N = static_cast<int>(N), p.K = static_cast<int>(K);
  p.tiles_m = static_cast<int>(plan.tiles_m);
  p.tiles_n = static_cast<int>(plan.tiles_n);
  p.k_tiles_total = k_tiles;
  p.k_tiles_split = (k_tiles + splits - 1) / splits;
  p.splits = (k_tiles + p.k_tiles_split - 1) / p.k_tiles_split;  // no empty slices
  p.panel = std::min(p.tiles_n, 8);
  p.out_kind = out_kind;
  p.accumulate = out_kind == kOutF32 ? (accumulate != 0) : 0;
  p.wide = (reinterpret_cast<uintptr_t>(d) & 31u) == 0 && (reinterpret_cast<uintptr_t>(resid) & 31u) == 0 &&
           (reinterpret_cast<uintptr_t>(fused.h_in) & 31u) == 0;
  p.q_scale = static_cast<uint8_t*>(fused.q_scale);
  p.qt_scale = static_cast<uint8_t*>(fused.q_t_scale);
  p.q_scale_tiles = static_cast<int>(N / 128);
  p.qt_scale_tiles = static_cast<int>(M / 128);
  p.h_in = fused.h_in;
  p.floor_rule = false;
  const int64_t tiles = plan.tiles();
  if (tiles * p.splits > 0x7fffffffLL)
    return MXB200_ERR_SHAPE;
  auto* s = static_cast<cudaStream_t>(stream);
  if (p.splits > 1) {
    const size_t need = workspace_bytes_for(plan, p.splits);
    if (workspace == nullptr || workspace_bytes < need)
      return MXB200_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
      return MXB200_ERR_ALIGNMENT;
    p.counters = static_cast<uint32_t*>(workspace);
    p.partials = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + counters_bytes(plan.counters()));
    if (cudaMemsetAsync(p.counters, 0, counters_bytes(plan.counters()), s) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
  }
  const int cap = g_max_ctas.load() > 0 ? g_max_ctas.load() : dev.sms;
  CUtensorMap ma, mb;
  if (plan.pair) {
    PairMaps m;
    if (int st = make_operand_map(&m.a, a, M, K, 128); st != MXB200_OK)
      return st;
    if (int st = make_operand_map(&m.b, b, N, K, plan.tile_n / 2); st != MXB200_OK)
      return st;
    if (int st = make_scale_map(&m.sfa, a_scale, M, K, 1); st != MXB200_OK)
      return st;
    if (int st = make_scale_map(&m.sfb, b_scale, N, K, 2); st != MXB200_OK)
      return st;
    if (d != nullptr) {
      if (int st = make_output_map(&m.d, d, M, N, out_kind == kOutF32); st != MXB200_OK)
        return st;
    } else {
      m.d = m.a;  // never used: the relu^2 backward form writes no plain output
    }
    m.part = m.d;  // unused without a K split
    if (p.splits > 1) {
      // partial half tiles, stacked: (tiles x splits x 2 halves x 128 rows, TN) fp32
      if (int st = make_output_map(&m.part, p.partials, tiles * p.splits * 256, plan.tile_n, true); st != MXB200_OK)
        return st;
    }
    m.q = m.qt = m.d;
    if (fusing) {
      if (int st = make_bytes_map(&m.q, fused.q, M, N); st != MXB200_OK)
        return st;
      if (int st = make_bytes_map(&m.qt, fused.q_t, N, M); st != MXB200_OK)
        return st;
    }
    const int pairs = static_cast<int>(std::min<int64_t>(tiles * p.splits, std::max(cap / 2, 1)));
    static std::atomic<uint32_t> launch_seq{0};
    p.sched_slot = static_cast<int>(launch_seq.fetch_add(1, std::memory_order_relaxed) % kSchedLaunchSlots);
    if (fused.fuse == kFuseReluSquare)
      return launch_pair_width<kFuseReluSquare>(plan.tile_n, m, p, pairs, s);
    if (fused.fuse == kFuseReluSquareBwd)
      return launch_pair_width<kFuseReluSquareBwd>(plan.tile_n, m, p, pairs, s);
    return launch_pair_width<kFuseNone>(plan.tile_n, m, p, pairs, s);
  }
  if (int st = make_operand_map(&ma, a, M, K, kBM); st != MXB200_OK)
    return st;
  if (int st = make_operand_map(&mb, b, N, K, plan.tile_n); st != MXB200_OK)
    return st;
  const int grid = static_cast<int>(std::min<int64_t>(tiles * p.splits, cap));
  return plan.tile_n == 256 ? launch<256>(ma, mb, p, grid, s) : launch<128>(ma, mb, p, grid, s);
}

}  // namespace

}  // namespace mxb200

extern "C" int mxb200_gemm_bf16(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d,
                                const void* resid, int64_t M, int64_t N, int64_t K, void* stream) {
  return mxb200::gemm(a, a_scale, b, b_scale, d, mxb200::kOutBf16, resid, M, N, K, nullptr, 0, 1, nullptr, 0, stream);
}

extern "C" int mxb200_gemm_f32(const void* a, const void* a_scale, const void* b, const void* b_scale, float* d,
                               int64_t M, int64_t N, int64_t K, const float* alpha, int accumulate, void* stream) {
  return mxb200::gemm(a, a_scale, b, b_scale, d, mxb200::kOutF32, nullptr, M, N, K, alpha, accumulate, 1, nullptr, 0,
                      stream);
}

extern "C" int mxb200_gemm_splits(int64_t M, int64_t N, int64_t K) {
  mxb200::DeviceInfo dev;
  if (mxb200::current_device(&dev) != MXB200_OK || M <= 0 || N <= 0 || K <= 0)
    return 1;
  const mxb200::TilePlan plan = mxb200::plan_tiles(M, N, K, dev.sms);
  const int64_t tiles = plan.tiles(), slots = plan.slots;
  const int64_t k_tiles = K / 128;
  // Splitting K costs a round trip of fp32 partial tiles through the workspace plus a serial reduction, and on
  // the d12-d26 shapes a narrower tile that fills a wave beat every split measured. It is kept for shapes that
  // cannot fill even a quarter of the machine with tiles alone and have a deep K to share out (d12's 768 x 768
  // weight gradient: 40 us with four splits against 47 us; with half the machine filled a split already loses).
  if (tiles * 4 > slots)
    return 1;
  int best = 1;
  for (int s = 2; s <= 4; s *= 2) {
    if (k_tiles / s < 32 || tiles * s > slots)
      break;
    best = s;
  }
  return best;
}

extern "C" size_t mxb200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int splits) {
  mxb200::DeviceInfo dev;
  if (splits <= 1 || M <= 0 || N <= 0 || K <= 0)
    return 0;
  if (mxb200::current_device(&dev) != MXB200_OK)
    dev.sms = 148;
  return mxb200::workspace_bytes_for(mxb200::plan_tiles(M, N, K, dev.sms), splits);
}

extern "C" int mxb200_gemm_splitk(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d,
                                  int out_kind, const void* resid, int64_t M, int64_t N, int64_t K, const float* alpha,
                                  int accumulate, int splits, void* workspace, size_t workspace_bytes, void* stream) {
  return mxb200::gemm(a, a_scale, b, b_scale, d, out_kind, resid, M, N, K, alpha, accumulate, splits, workspace,
                      workspace_bytes, stream);
}

extern "C" int mxb200_set_gemm_config(int tile_n, int max_ctas) {
  if ((tile_n != 0 && tile_n != 128 && tile_n != 256 && tile_n != 384 && tile_n != 512) || max_ctas < 0)
    return MXB200_ERR_ARGUMENT;
  mxb200::g_tile_n.store(tile_n);
  mxb200::g_max_ctas.store(max_ctas);
  return MXB200_OK;
}

namespace mxb200 {
namespace {

// One warp, one barrier that nobody arrives on: the same bounded wait as the GEMM's, with a caller-given limit.
__global__ void mxb200_selftest_wait_kernel(uint64_t limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  const uint64_t t0 = global_timer_ns();
  bool gave_up = false;
  while (!mbar_try_wait(&bar, 0)) {
    if (global_timer_ns() - t0 > limit_ns) {
      gave_up = true;
      break;
    }
  }
  if (gave_up && threadIdx.x == 0)
    atomicCAS(&g_watchdog_word, 0u, 0x80000000u | 0x7fu);
}

}  // namespace
}  // namespace mxb200

extern "C" int mxb200_selftest_bounded_wait(uint64_t limit_ns, void* stream) {
  mxb200::DeviceInfo dev;
  if (int s = mxb200::current_device(&dev); s != MXB200_OK)
    return s;
  if (limit_ns == 0 || limit_ns > 10000000ull)
    return MXB200_ERR_ARGUMENT;
  mxb200::mxb200_selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
  mxb200::g_launches.fetch_add(1, std::memory_order_relaxed);
  return mxb200::launch_status();
}

extern "C" int mxb200_device_status(uint32_t* word) {
  uint32_t w = 0;
  if (cudaDeviceSynchronize() != cudaSuccess)
    return MXB200_ERR_LAUNCH;
  if (cudaMemcpyFromSymbol(&w, mxb200::g_watchdog_word, sizeof(w)) != cudaSuccess)
    return MXB200_ERR_LAUNCH;
  if (w != 0) {
    const uint32_t zero = 0;
    cudaMemcpyToSymbol(mxb200::g_watchdog_word, &zero, sizeof(zero));
    // a launch that gave up did not finish its tile list: its scheduler counters are left mid-way
    static const uint32_t zeros[2 * mxb200::kSchedLaunchSlots] = {};
    cudaMemcpyToSymbol(mxb200::g_sched_words, zeros, sizeof(zeros));
  }
  if (const uint32_t norm = mxb200::take_norm_watchdog_word(); w == 0)
    w = norm;
  if (const uint32_t quant = mxb200::take_quantize_watchdog_word(); w == 0)
    w = quant;
  if (word != nullptr)
    *word = w;
  return w == 0 ? MXB200_OK : MXB200_ERR_WATCHDOG;
}

// See include/mxb200.h. Same kernel and same host path as mxb200_gemm_splitk; only the origin of the scratch differs.
extern "C" int mxb200_gemm_splitk_static(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                         void* d, int out_kind, const void* resid, int64_t M, int64_t N, int64_t K,
                                         const float* alpha, int accumulate, int splits, void* stream) {
  static std::mutex mu;
  static void* scratch_of_device[64] = {};
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return MXB200_ERR_DEVICE;
  void* scratch = nullptr;
  {
    // set-up, once per device and with that device current: translate the symbol into this device's address
    std::lock_guard<std::mutex> lock(mu);
    if (scratch_of_device[device] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, mxb200::g_static_splitk_scratch) != cudaSuccess || p == nullptr) {
        cudaGetLastError();
        return MXB200_ERR_DEVICE;
      }
      scratch_of_device[device] = p;
    }
    scratch = scratch_of_device[device];
  }
  if (splits > 1 && mxb200_gemm_workspace_bytes(M, N, K, splits) > MXB200_STATIC_SCRATCH_BYTES)
    return MXB200_ERR_WORKSPACE;  // the problem needs more scratch than the built-in array holds
  return mxb200::gemm(a, a_scale, b, b_scale, d, out_kind, resid, M, N, K, alpha, accumulate, splits, scratch,
                      MXB200_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int mxb200_gemm_relu_square(const void* a, const void* a_scale, const void* b, const void* b_scale, void* h,
                                       void* q, void* q_scale, void* q_t, void* q_t_scale, int64_t M, int64_t N,
                                       int64_t K, void* stream) {
  mxb200::FusedOut f;
  f.fuse = mxb200::kFuseReluSquare, f.q = q, f.q_scale = q_scale, f.q_t = q_t, f.q_t_scale = q_t_scale;
  return mxb200::gemm(a, a_scale, b, b_scale, h, mxb200::kOutBf16, nullptr, M, N, K, nullptr, 0, 1, nullptr, 0, stream, f);
}

extern "C" int mxb200_gemm_relu_square_bwd(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                           const void* h, void* dh, void* dh_scale, void* dh_t, void* dh_t_scale,
                                           int64_t M, int64_t N, int64_t K, void* stream) {
  mxb200::FusedOut f;
  f.fuse = mxb200::kFuseReluSquareBwd, f.q = dh, f.q_scale = dh_scale, f.q_t = dh_t, f.q_t_scale = dh_t_scale, f.h_in = h;
  return mxb200::gemm(a, a_scale, b, b_scale, nullptr, mxb200::kOutBf16, nullptr, M, N, K, nullptr, 0, 1, nullptr, 0,
                      stream, f);
}
