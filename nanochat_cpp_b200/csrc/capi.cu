// Library-wide pieces of the C ABI: status strings, device check, launch accounting.
#include <mutex>

#include "internal.h"

namespace mxb200 {

std::atomic<uint64_t> g_launches{0};

int current_device(DeviceInfo* info) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0) {
    cudaGetLastError();
    return MXB200_ERR_DEVICE;
  }
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo local;
  DeviceInfo& d = device < 64 ? cache[device] : local;
  if (d.device != device) {
    int major = 0, sms = 0, smem = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) {
      cudaGetLastError();
      return MXB200_ERR_DEVICE;
    }
    d.device = device, d.cc_major = major, d.sms = sms, d.smem_optin = smem;
  }
  *info = d;
  return d.cc_major == 10 ? MXB200_OK : MXB200_ERR_DEVICE;
}

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

}  // namespace mxb200

extern "C" const char* mxb200_strerror(int status) {
  switch (status) {
    case MXB200_OK:
      return "ok";
    case MXB200_ERR_SHAPE:
      return "mxb200: dimensions must be positive multiples of 128 (and fit the views given)";
    case MXB200_ERR_ALIGNMENT:
      return "mxb200: pointers and leading dimensions must be 16-byte aligned (workspace: 256)";
    case MXB200_ERR_NULL:
      return "mxb200: a required pointer is null";
    case MXB200_ERR_ARGUMENT:
      return "mxb200: unsupported flag, enum value or combination of arguments";
    case MXB200_ERR_WORKSPACE:
      return "mxb200: split-K workspace missing or smaller than mxb200_gemm_workspace_bytes";
    case MXB200_ERR_DEVICE:
      return "mxb200: needs an sm_100 (B200) device current; there is no CPU fallback";
    case MXB200_ERR_DRIVER:
      return "mxb200: cuTensorMapEncodeTiled failed or is unavailable";
    case MXB200_ERR_LAUNCH:
      return "mxb200: CUDA reported an error at launch";
    case MXB200_ERR_WATCHDOG:
      return "mxb200: a bounded device-side wait ran out (see mxb200_device_status)";
    default:
      return "mxb200: unknown status";
  }
}

extern "C" uint64_t mxb200_launch_count(void) {
  return mxb200::g_launches.load(std::memory_order_relaxed);
}

extern "C" int mxb200_version(void) {
  return 100;
}
