// Library-level C ABI helpers: error string, ABI version.
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
}  // namespace sphkv

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
