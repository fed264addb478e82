// Loss pass of the chunked lm_head under MX: per row of bf16 logits the log-sum-exp of the soft-capped logits
// (capped = softcap * tanh(z / softcap)) and the cross-entropy loss lse - capped[target]. Replaces nanochat-cpp's
// nanochat_softcap_ce_loss (src/nanochat/model/ops/softcap_ce_kernel.cu:62-116 with kGrad = false), same bits: the
// gradient is not written here, the quantizer's softcap-gradient prologue recomputes it from the logits and this
// kernel's lse and emits it as MX directly (quantize_sm100.cu).
// The fp32 sum of exponentials is order-sensitive, and lse feeds every gradient value, so the order is the
// reference's: 256 threads per row, thread t adds columns t * 8 + 2048 * i + k in order of i then k, a butterfly
// (xor 16..1) inside each warp, then the eight warp sums again by butterfly in warp 0. |capped| <= softcap, so
// exp(capped - softcap) needs no running maximum.
// A row of 32768 logits costs one tanh and one exp per element: the pass is bound by the SFU/ALU work, not by HBM
// (64 KB per row).
#include <cuda_bf16.h>

#include "internal.h"

namespace mxb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kVec = 8;

__device__ __forceinline__ float row_sum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = static_cast<int>(threadIdx.x) & 31, warp = static_cast<int>(threadIdx.x) >> 5;
  if (lane == 0)
    smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < kThreads / 32 ? smem[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0)
      smem[0] = v;
  }
  __syncthreads();
  return smem[0];
}

__global__ void __launch_bounds__(kThreads) mxb200_softcap_ce_loss_kernel(const __nv_bfloat16* logits, int64_t ld,
                                                                          const int64_t* targets, int vocab, int padded,
                                                                          float softcap, float* loss, float* lse_out) {
  __shared__ float smem[kThreads / 32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* z = logits + row * ld;
  const int64_t target = targets[row];
  if (target < 0) {  // ignored row: loss 0, lse left unset
    if (loss != nullptr && threadIdx.x == 0)
      loss[row] = 0.f;
    return;
  }
  float sum = 0.f;
  for (int j = static_cast<int>(threadIdx.x) * kVec; j < padded; j += kThreads * kVec) {
    const uint4 raw = *reinterpret_cast<const uint4*>(z + j);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < kVec; ++k) {
      const float v = __uint_as_float((k & 1) ? (w[k >> 1] & 0xffff0000u) : (w[k >> 1] << 16));
      if (j + k < vocab)
        sum += expf(softcap * tanhf(v / softcap) - softcap);
    }
  }
  const float lse = softcap + logf(row_sum(sum, smem));
  if (threadIdx.x == 0) {
    if (loss != nullptr)
      loss[row] = lse - softcap * tanhf(__bfloat162float(z[target]) / softcap);
    if (lse_out != nullptr)
      lse_out[row] = lse;
  }
}

}  // namespace

}  // namespace mxb200

extern "C" int mxb200_softcap_ce_loss(const void* logits, int64_t rows, int64_t ld, const int64_t* targets, int vocab,
                                      int padded, float softcap, float* loss, float* lse, void* stream) {
  using namespace mxb200;
  DeviceInfo dev;
  if (int s = current_device(&dev); s != MXB200_OK)
    return s;
  if (logits == nullptr || targets == nullptr || (loss == nullptr && lse == nullptr))
    return MXB200_ERR_NULL;
  if (rows <= 0 || rows > 0x7fffffffLL || padded <= 0 || padded % kVec != 0 || ld < padded || ld % kVec != 0)
    return MXB200_ERR_SHAPE;
  if (vocab <= 0 || vocab > padded || !(softcap > 0.f))
    return MXB200_ERR_ARGUMENT;
  if (!aligned16(logits))
    return MXB200_ERR_ALIGNMENT;
  mxb200_softcap_ce_loss_kernel<<<static_cast<unsigned>(rows), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, targets, vocab, padded, softcap, loss, lse);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return launch_status();
}
