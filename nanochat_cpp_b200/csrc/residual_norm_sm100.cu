// Fused residual add + lambda blend + RMS norm whose normalized output leaves MX-quantized in both layouts: the
// producer of the quantized input of the QKV and MLP-fc GEMMs. Replaces nanochat-cpp's
// nanochat_residual_norm_mx_fwd_c* (src/nanochat/model/ops/residual_norm_kernel.cu:153-214, launcher :330-349),
// same bits. Per row of `cols` bf16 values:
//   s = r ? bf16(x + r) : x;  res = x0 ? bf16(bf16(lr * s) + bf16(l0 * x0)) : s   (lr, l0 rounded to bf16 first)
//   rstd = rsqrt(sum(res^2) / cols + eps);  n = bf16(res * rstd);  MX(n) row-wise and column-wise
// The roundings are the reference's (residual_norm_kernel.cu:80-128). A bf16 product is exact in fp32 and the fp32
// sum of two bf16 values rounds to bf16 as the exact sum does, so the add and the blend run as packed bf16x2
// instructions (add.rn / mul.rn, never contracted) with the same bits as the reference's fp32-then-round form.
// rstd is bit-exact only if the sum of squares is taken in the reference's order, so that part is fixed: a warp owns
// a row, lane l owns columns (it * 32 + l) * 8 .. + 7 for it = 0, 1, ..., accumulates them in order, and the warp
// combines with the xor-16-8-4-2-1 butterfly.
//
// Everything around that is laid out for HBM. A persistent CTA per SM owns tiles of 32 rows (one scale block of
// the column-wise layout) x all columns. One producer warp streams the input rows of this and the following tiles
// into a shared-memory ring with bulk async copies (one contiguous row of x, r, x0 per slot, completion on an
// mbarrier), as far ahead as the ring is deep, so loads stay in flight while the 16 consumer warps compute, store
// and run the column pass. A consumer warp takes a row from its slot, releases the slot after the first pass, parks
// the bf16 n in a shared tile and writes res, s, rstd and the row-wise MX bytes; after all 32 rows, each thread owns
// a column of the tile and writes 32 contiguous bytes of the transposed layout. Each input byte is read once and
// each output byte written once (x, r, x0: 2 B each; res, s: 2 B each; MX: 2 x (1 + 1/32) B per element).
// Every wait is bounded: after kWaitLimitNs it records its site in a device word, raises a CTA-wide flag that all
// other waits poll, and the CTA returns once its copies in flight have landed.
#include <algorithm>

#include <cuda_bf16.h>

#include "internal.h"
#include "bf16x2_sm100.cuh"
#include "mx_common.cuh"
#include "ptx_sm100.cuh"

namespace mxb200 {

__device__ uint32_t g_norm_watchdog_word;

namespace {

constexpr int kRows = 32;  // rows per tile
constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;  // + the producer warp
constexpr int kVec = 8;                    // bf16 per 16-byte vector
constexpr int kMaxCols = 2048;
constexpr int kMaxSlots = 24;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr uint64_t kDrainLimitNs = 50000000ull;

enum Site : uint32_t { kSiteRingEmpty = 1, kSiteRingTaken = 2, kSiteRingFull = 3, kSiteRowsDone = 4, kSiteColumnsDone = 5 };

struct NormParams {
  mxb200_residual_norm_mx a;
  int slots;       // ring depth in rows
  int inputs;      // streams per row: x (+ r) (+ x0)
  bool wide_out_t;
};

// Per row of a tile: full[r] completes when the row has landed, taken[r] when its consumer has it in registers; each
// completes once per tile and is watched by the producer and by the one warp that owns row r, phase after phase, so a
// one-bit parity is never ambiguous. The producer re-arms full[r] only after taken[r] of the tile before, which keeps
// it from running a whole phase ahead of a slow consumer. Per ring slot: empty[s] completes once per release.
struct RingBarriers {
  uint64_t full[kRows];
  uint64_t taken[kRows];
  uint64_t empty[kMaxSlots];
  uint64_t tile_sync;  // the consumer warps' barrier between the row and column passes
  uint32_t abort_flag;
};

__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, RingBarriers* bars, uint32_t site) {
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
        atomicCAS(&g_norm_watchdog_word, 0u, 0x80000000u | (blockIdx.x << 8) | site);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ bool wait_bounded_warp(uint64_t* bar, uint32_t parity, RingBarriers* bars, uint32_t site) {
  return __all_sync(0xffffffffu, wait_bounded(bar, parity, bars, site)) != 0;
}

template <int kIters>
__global__ void __launch_bounds__(kThreads, 1) mxb200_residual_norm_mx_kernel(const NormParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const mxb200_residual_norm_mx& a = p.a;
  const int cols = a.cols;
  const int pitch = cols + kVec;  // bf16 elements per parked row: 16 bytes of padding keep row starts on distinct banks
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * 2u;
  const uint32_t slot_bytes = row_bytes * static_cast<uint32_t>(p.inputs);
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem);
  unsigned char* ring = smem + static_cast<size_t>(kRows) * pitch * 2;
  RingBarriers* bars = reinterpret_cast<RingBarriers*>(ring + static_cast<size_t>(p.slots) * slot_bytes);
  const int lane = static_cast<int>(threadIdx.x) & 31, warp = static_cast<int>(threadIdx.x) >> 5;
  const bool add = a.r != nullptr, blend = a.x0 != nullptr;
  const int slots = p.slots;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kRows; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->taken[i], 1);
    }
    for (int i = 0; i < slots; ++i)
      mbar_init(&bars->empty[i], 1);
    mbar_init(&bars->tile_sync, kConsumerWarps);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const int64_t tiles = a.rows / kRows;

  if (warp == kConsumerWarps) {
    // ---- producer: one row per slot, in row order (the order the consumers take them)
    const uint32_t leader = elect_one() ? 1u : 0u;
    int slot = 0;
    uint32_t phase = 0, tile_parity = 0;
    int64_t issued = 0;
    bool ok = true;
    for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, tile_parity ^= 1u) {
      for (int r = 0; r < kRows; ++r) {
        uint64_t* full = &bars->full[r];
        // the slot's last row has been released, and the consumer of row r has taken the one of the tile before
        if (!wait_bounded_warp(&bars->empty[slot], phase ^ 1u, bars, kSiteRingEmpty) ||
            !wait_bounded_warp(&bars->taken[r], tile_parity ^ 1u, bars, kSiteRingTaken)) {
          ok = false;
          break;
        }
        const int64_t offset = (t * kRows + r) * static_cast<int64_t>(cols);
        unsigned char* dst = ring + static_cast<size_t>(slot) * slot_bytes;
        mbar_arrive_expect_tx(leader, full, slot_bytes);
        bulk_load(leader, dst, static_cast<const __nv_bfloat16*>(a.x) + offset, row_bytes, full);
        if (add)
          bulk_load(leader, dst + row_bytes, static_cast<const __nv_bfloat16*>(a.r) + offset, row_bytes, full);
        if (blend)
          bulk_load(leader, dst + (add ? 2u : 1u) * row_bytes, static_cast<const __nv_bfloat16*>(a.x0) + offset,
                    row_bytes, full);
        ++issued;
        if (++slot == slots) {
          slot = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok) {
      // leaving early: the copies already issued must land before this CTA's shared memory is given away
      for (int r = 0; r < kRows; ++r) {
        const int64_t arms = (issued + kRows - 1 - r) / kRows;
        if (arms == 0)
          continue;
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(&bars->full[r], static_cast<uint32_t>(arms - 1) & 1u) &&
               global_timer_ns() - t0 < kDrainLimitNs) {
        }
      }
    }
    return;
  }

  // ---- consumers
  const uint32_t lr2 = blend ? pack_bf16x2_rn(*a.lr, *a.lr) : 0u, l02 = blend ? pack_bf16x2_rn(*a.l0, *a.l0) : 0u;
  auto* out = static_cast<unsigned char*>(a.out.data);
  auto* out_scale = static_cast<unsigned char*>(a.out.scale);
  auto* out_t = static_cast<unsigned char*>(a.out_t.data);
  auto* out_t_scale = static_cast<unsigned char*>(a.out_t.scale);
  int slot = warp % slots;  // of this warp's next row: rows advance by 16 per step, slots wrap at the ring depth
  uint32_t sync_phase = 0, tile_parity = 0;
  const int step = kConsumerWarps % slots;

  for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x, tile_parity ^= 1u) {
    const int64_t row0 = t * kRows;
    for (int r = warp; r < kRows; r += kConsumerWarps) {
      const int64_t row = row0 + r;
      if (!wait_bounded_warp(&bars->full[r], tile_parity, bars, kSiteRingFull))
        return;
      // lane-based pointers: every access of the row below is one of these plus a compile-time multiple of 512 bytes
      const uint4* sx = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(slot) * slot_bytes) + lane;
      const uint4* sr = sx + cols / kVec;
      const uint4* sx0 = sx + (add ? 2 : 1) * (cols / kVec);
      uint4* res_row = reinterpret_cast<uint4*>(a.res) + (row * cols) / kVec + lane;
      uint4* s_row = (add && a.s != nullptr) ? reinterpret_cast<uint4*>(a.s) + (row * cols) / kVec + lane : nullptr;
      float ss = 0.f;
      uint4 nv[kIters];
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        if ((it * 32 + lane) * kVec < cols) {
          uint4 v = sx[it * 32];
          if (add) {
            const uint4 rv = sr[it * 32];
            v = make_uint4(add_bf16x2(v.x, rv.x), add_bf16x2(v.y, rv.y), add_bf16x2(v.z, rv.z), add_bf16x2(v.w, rv.w));
            if (s_row != nullptr)
              s_row[it * 32] = v;
          }
          if (!add && !blend)  // x + (-0) = x, except that a NaN leaves canonical as it does from the reference's re-rounding
            v = make_uint4(add_bf16x2(v.x, 0x80008000u), add_bf16x2(v.y, 0x80008000u), add_bf16x2(v.z, 0x80008000u),
                           add_bf16x2(v.w, 0x80008000u));
          if (blend) {
            const uint4 zv = sx0[it * 32];
            v = make_uint4(add_bf16x2(mul_bf16x2(lr2, v.x), mul_bf16x2(l02, zv.x)),
                           add_bf16x2(mul_bf16x2(lr2, v.y), mul_bf16x2(l02, zv.y)),
                           add_bf16x2(mul_bf16x2(lr2, v.z), mul_bf16x2(l02, zv.z)),
                           add_bf16x2(mul_bf16x2(lr2, v.w), mul_bf16x2(l02, zv.w)));
          }
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            ss = fmaf(lo_f32(w[k]), lo_f32(w[k]), ss);
            ss = fmaf(hi_f32(w[k]), hi_f32(w[k]), ss);
          }
          nv[it] = v;
          res_row[it * 32] = v;
        }
      }
      __syncwarp();
      if (lane == 0) {  // the row is in registers: the slot can take another, and row r of the next tile may be sent
        mbar_arrive(&bars->empty[slot]);
        mbar_arrive(&bars->taken[r]);
      }
      slot += step;
      if (slot >= slots)
        slot -= slots;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss / static_cast<float>(cols) + a.eps);
      if (lane == 0)
        a.rstd[row] = rstd;
      // n = bf16(res * rstd): parked for the column pass, quantized row-wise from registers (4 lanes per block)
      uint4* tile_row = reinterpret_cast<uint4*>(tile + r * pitch) + lane;
      uint2* out_row = reinterpret_cast<uint2*>(out + row * a.out.ld) + lane;
      uint4* n_row = reinterpret_cast<uint4*>(a.n) + (row * cols) / kVec + lane;
      // the scale byte of block b = it * 8 + lane / 4 sits at tile (row / 128, b / 4), byte offset(row % 128, b % 4)
      unsigned char* scale_row = out_scale + (static_cast<int64_t>(row >> 7) * a.out.scale_tiles + (lane >> 4)) * kScaleTileBytes +
                                 mx_scale_tile_offset(static_cast<int>(row & 127), (lane >> 2) & 3);
#pragma unroll
      for (int it = 0; it < kIters; ++it) {
        const int col = (it * 32 + lane) * kVec;
        const bool active = col < cols;  // whole 4-lane groups: cols % 32 == 0
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        uint32_t m = 0u;
        if (active) {
          const uint32_t src[4] = {nv[it].x, nv[it].y, nv[it].z, nv[it].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            w[k] = pack_bf16x2_rn(lo_f32(src[k]) * rstd, hi_f32(src[k]) * rstd);
            m = max_abs_skip_nan_bf16x2(m, w[k]);
          }
          tile_row[it * 32] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        // the packed maximum skips NaN as the quantizer's fmaxf does; the block's 4 lanes then agree on it (magnitudes
        // of bf16 order as unsigned integers)
        m &= 0x7fff7fffu;
        uint32_t mm = max(m & 0xffffu, m >> 16);
        mm = max(mm, __shfl_xor_sync(0xffffffffu, mm, 1));
        mm = max(mm, __shfl_xor_sync(0xffffffffu, mm, 2));
        const float amax = __uint_as_float(mm << 16);
        if (active) {
          const int e = mx_exponent(__float_as_uint(amax), false);
          const uint32_t mul2 = (mx_multiplier_bits(e) >> 16) * 0x10001u;
          uint2 o;
          o.x = e4m3x4_scaled(w[0], w[1], mul2);
          o.y = e4m3x4_scaled(w[2], w[3], mul2);
          out_row[it * 32] = o;
          if ((lane & 3) == 0)
            scale_row[it * 2 * kScaleTileBytes] = static_cast<unsigned char>(e);
          if (col < a.n_cols)
            n_row[it * 32] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&bars->tile_sync);
    if (!wait_bounded(&bars->tile_sync, sync_phase, bars, kSiteRowsDone))
      return;
    sync_phase ^= 1u;

    // ---- columns: a thread owns a column over the tile's 32 rows
    for (int c = static_cast<int>(threadIdx.x); c < cols; c += kConsumers) {
      uint32_t w[kRows / 2];  // rows 2k (low half) and 2k + 1 (high half)
      uint32_t m = 0u;
#pragma unroll
      for (int k = 0; k < kRows / 2; ++k) {
        const uint32_t even = *reinterpret_cast<const unsigned short*>(tile + (2 * k) * pitch + c);
        const uint32_t odd = *reinterpret_cast<const unsigned short*>(tile + (2 * k + 1) * pitch + c);
        w[k] = even | (odd << 16);
        m = max_abs_skip_nan_bf16x2(m, w[k]);
      }
      m &= 0x7fff7fffu;
      const float amax = __uint_as_float(max(m & 0xffffu, m >> 16) << 16);
      const int e = mx_exponent(__float_as_uint(amax), false);
      const uint32_t mul2 = (mx_multiplier_bits(e) >> 16) * 0x10001u;
      uint32_t q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        q[k] = e4m3x4_scaled(w[2 * k], w[2 * k + 1], mul2);
      unsigned char* dst = out_t + static_cast<int64_t>(c) * a.out_t.ld + row0;
      if (p.wide_out_t) {
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(q[0]), "r"(q[1]), "r"(q[2]),
                     "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7])
                     : "memory");
      } else {
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(q[0], q[1], q[2], q[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(q[4], q[5], q[6], q[7]);
      }
      const int b = static_cast<int>(row0 >> 5);
      out_t_scale[(static_cast<int64_t>(c >> 7) * a.out_t.scale_tiles + (b >> 2)) * kScaleTileBytes +
                  mx_scale_tile_offset(c & 127, b)] = static_cast<unsigned char>(e);
    }
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&bars->tile_sync);  // before the next tile overwrites the parked rows
    if (!wait_bounded(&bars->tile_sync, sync_phase, bars, kSiteColumnsDone))
      return;
    sync_phase ^= 1u;
  }
}

template <int kIters>
int launch(NormParams& p, const DeviceInfo& dev, cudaStream_t stream) {
  const size_t tile_bytes = static_cast<size_t>(kRows) * (p.a.cols + kVec) * sizeof(__nv_bfloat16);
  const size_t slot_bytes = static_cast<size_t>(p.inputs) * p.a.cols * sizeof(__nv_bfloat16);
  const size_t fixed = tile_bytes + sizeof(RingBarriers) + 128;
  if (static_cast<size_t>(dev.smem_optin) < fixed + 2 * slot_bytes)
    return MXB200_ERR_SHAPE;
  p.slots = static_cast<int>(std::min<size_t>(kMaxSlots, (dev.smem_optin - fixed) / slot_bytes));
  const size_t smem = tile_bytes + p.slots * slot_bytes + sizeof(RingBarriers);
  static std::atomic<int> configured_for{-1};
  if (configured_for.load() != dev.device) {
    if (cudaFuncSetAttribute(mxb200_residual_norm_mx_kernel<kIters>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             dev.smem_optin) != cudaSuccess)
      return MXB200_ERR_LAUNCH;
    configured_for.store(dev.device);
  }
  const int64_t tiles = p.a.rows / kRows;
  const int grid = static_cast<int>(std::min<int64_t>(tiles, static_cast<int64_t>(dev.sms)));
  mxb200_residual_norm_mx_kernel<kIters><<<grid, kThreads, smem, stream>>>(p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}

}  // namespace

uint32_t take_norm_watchdog_word() {
  uint32_t w = 0;
  if (cudaMemcpyFromSymbol(&w, g_norm_watchdog_word, sizeof(w)) != cudaSuccess)
    return 0;
  if (w != 0) {
    const uint32_t zero = 0;
    cudaMemcpyToSymbol(g_norm_watchdog_word, &zero, sizeof(zero));
  }
  return w;
}

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
      a.n_cols > a.cols || a.out.ld < a.cols || a.out_t.ld < a.rows || a.out.scale_tiles < a.cols / 128 ||
      a.out_t.scale_tiles < a.rows / 128)
    return MXB200_ERR_SHAPE;
  for (const void* ptr : {a.x, a.r, a.x0, static_cast<const void*>(a.s), static_cast<const void*>(a.res),
                          static_cast<const void*>(a.n), static_cast<const void*>(a.out.data),
                          static_cast<const void*>(a.out.scale), static_cast<const void*>(a.out_t.data),
                          static_cast<const void*>(a.out_t.scale)})
    if (ptr != nullptr && !aligned16(ptr))
      return MXB200_ERR_ALIGNMENT;
  if (a.out.ld % 16 != 0 || a.out_t.ld % 16 != 0)
    return MXB200_ERR_ALIGNMENT;
  NormParams p{a, 0, 1 + (a.r != nullptr) + (a.x0 != nullptr),
               (reinterpret_cast<uintptr_t>(a.out_t.data) & 31u) == 0 && a.out_t.ld % 32 == 0};
  auto* s = static_cast<cudaStream_t>(stream);
  switch ((a.cols + 255) / 256) {
    case 1: return launch<1>(p, dev, s);
    case 2: return launch<2>(p, dev, s);
    case 3: return launch<3>(p, dev, s);
    case 4: return launch<4>(p, dev, s);
    case 5: return launch<5>(p, dev, s);
    case 6: return launch<6>(p, dev, s);
    case 7: return launch<7>(p, dev, s);
    default: return launch<8>(p, dev, s);
  }
}
