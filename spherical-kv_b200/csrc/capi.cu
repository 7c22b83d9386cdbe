// Library-level C ABI helpers: error string, ABI version, per-device host state.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace sphkv {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

int sm_count_current_device() {
  static int cached[kMaxDevices];
  const int dev = current_device_slot();
  if (dev < 0) {
    set_error("sm_count: cudaGetDevice failed or device index >= %d", kMaxDevices);
    return SPHKV_E_LIMIT;
  }
  if (cached[dev] <= 0) {
    int n = 0;
    cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || n <= 0) {
      set_error("sm_count: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? -(int)e : SPHKV_E_ARG;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

int ensure_dynamic_smem(SmemOptIn& st, const void* kernel, int bytes, const char* what) {
  if (bytes <= 48 * 1024) return 0;
  const int dev = current_device_slot();
  if (dev < 0) {
    set_error("%s: cudaGetDevice failed or device index >= %d", what, kMaxDevices);
    return SPHKV_E_LIMIT;
  }
  if (st.bytes[dev] >= bytes) return 0;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute(%d B of dynamic shared memory): %s", what, bytes, cudaGetErrorString(e));
    return (int)e;
  }
  st.bytes[dev] = bytes;
  return 0;
}
}  // namespace sphkv

extern "C" int sphkv_sm_count(void) { return sphkv::sm_count_current_device(); }
extern "C" int sphkv_abi_version(void) { return SPHKV_ABI_VERSION; }
extern "C" const char* sphkv_last_error(void) { return sphkv::g_err; }
extern "C" int sphkv_struct_size(int which) {
  switch (which) {
    case 0: return (int)sizeof(sphkv_tiers);
    case 1: return (int)sizeof(sphkv_encode_params);
    case 2: return (int)sizeof(sphkv_decode_params);
    default: return -1;
  }
}
