// Library-level C ABI helpers: error string, ABI version, per-device host state.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

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

// ---- exchange buffers for split-KV across the GPUs of one node ---------------------------------
// The receive buffers of the peer exchange are written by kernels that run on OTHER
// GPUs, each in its own process.  They are allocated here with cudaMalloc (one allocation = one
// IPC handle, no sub-allocation offsets to carry around) and opened by the other ranks with the
// opening rank's device current, which is what maps the memory into that device's address space
// and turns peer access on.
extern "C" int sphkv_xchg_alloc(int64_t bytes, void** dev_ptr, unsigned char* handle64) {
  SPHKV_REQUIRE(bytes > 0 && dev_ptr && handle64, SPHKV_E_ARG, "xchg_alloc: bad argument");
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, (size_t)bytes);
  if (e == cudaSuccess) e = cudaMemset(ptr, 0, (size_t)bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    sphkv::set_error("xchg_alloc(%lld B): %s", (long long)bytes, cudaGetErrorString(e));
    if (ptr) cudaFree(ptr);
    return (int)e;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *dev_ptr = ptr;
  return 0;
}

extern "C" int sphkv_xchg_open(const unsigned char* handle64, void** dev_ptr) {
  SPHKV_REQUIRE(handle64 && dev_ptr, SPHKV_E_ARG, "xchg_open: NULL pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* ptr = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    sphkv::set_error("xchg_open: cudaIpcOpenMemHandle: %s (do the two GPUs reach each other?)", cudaGetErrorString(e));
    return (int)e;
  }
  *dev_ptr = ptr;
  return 0;
}

extern "C" int sphkv_xchg_close(void* opened_ptr) {
  if (opened_ptr == nullptr) return 0;
  cudaError_t e = cudaIpcCloseMemHandle(opened_ptr);
  if (e != cudaSuccess) {
    sphkv::set_error("xchg_close: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

extern "C" int sphkv_xchg_free(void* dev_ptr) {
  if (dev_ptr == nullptr) return 0;
  cudaError_t e = cudaFree(dev_ptr);
  if (e != cudaSuccess) {
    sphkv::set_error("xchg_free: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}
