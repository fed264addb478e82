// Host-side pieces shared by the translation units of libmxb200.
#pragma once

#include <atomic>
#include <cstdint>

#include <cuda.h>
#include <cuda_runtime.h>

#include "mxb200.h"

namespace mxb200 {

extern std::atomic<uint64_t> g_launches;

struct DeviceInfo {
  int device = -1;
  int sms = 0;
  int cc_major = 0;
  int smem_optin = 0;
};

// Properties of the current device, cached per device. Returns MXB200_ERR_DEVICE unless it is sm_100.
int current_device(DeviceInfo* info);

// cuTensorMapEncodeTiled, looked up through the runtime (no link-time dependency on libcuda); null if unavailable.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn();

// The residual-norm kernel's watchdog word (non-zero after one of its bounded waits ran out), read and cleared.
uint32_t take_norm_watchdog_word();
// The same for the streaming quantizer.
uint32_t take_quantize_watchdog_word();

inline bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

inline int launch_status() {
  return cudaGetLastError() == cudaSuccess ? MXB200_OK : MXB200_ERR_LAUNCH;
}

}  // namespace mxb200
