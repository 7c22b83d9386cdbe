// Shared device helpers for the sm_100a Spherical-KV kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sphkv.h"

// unroll factor of the centroid loops of the similarity searches (independent fma chains in flight)
#ifndef SPHKV_SEARCH_UNROLL
#define SPHKV_SEARCH_UNROLL 2
#endif
// all-tier code kernel: tokens per thread (4 = one CTA of 8 warps per SM, 232 registers; 2 = two
// CTAs per SM) and the unroll factor of its centroid loop
#ifndef SPHKV_CODE_TOKENS
#define SPHKV_CODE_TOKENS 4
#endif
#ifndef SPHKV_CODE_UNROLL
#define SPHKV_CODE_UNROLL 4
#endif
#define SPHKV_PRAGMA_(x) _Pragma(#x)
#define SPHKV_PRAGMA(x) SPHKV_PRAGMA_(x)
#define SPHKV_UNROLL_SEARCH SPHKV_PRAGMA(unroll SPHKV_SEARCH_UNROLL)
#define SPHKV_UNROLL_CODE_SEARCH SPHKV_PRAGMA(unroll SPHKV_CODE_UNROLL)

namespace sphkv {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---- error plumbing (host) -------------------------------------------------------
void set_error(const char* fmt, ...);
#define SPHKV_REQUIRE(cond, code, ...) \
  do {                                 \
    if (!(cond)) {                     \
      ::sphkv::set_error(__VA_ARGS__); \
      return (code);                   \
    }                                  \
  } while (0)

// ---- per-device host state ---------------------------------------------------------
// The SM count and a kernel's dynamic shared-memory opt-in belong to a device, not to the
// process, so what the host caches about them is indexed by the current device.
constexpr int kMaxDevices = 64;
int current_device_slot();      // cudaGetDevice(), or -1 when it fails / index >= kMaxDevices
int sm_count_current_device();  // > 0, or a negative error
struct SmemOptIn {
  int bytes[kMaxDevices];  // largest size this kernel was opted in for, per device (0 = never)
};
// Raises `kernel`'s dynamic shared-memory limit on the current device to `bytes` if it is not
// there yet.  Sizes up to 48 KB need no opt-in and are not recorded.
int ensure_dynamic_smem(SmemOptIn& st, const void* kernel, int bytes, const char* what);

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// ---- tensor-core / async-copy wrappers (inline PTX) ------------------------------
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                              uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
// 16-byte asynchronous copy of which only the first src_bytes (0 or 16) are read; the rest is zero
__device__ __forceinline__ void cp_async_16_zfill(uint32_t smem_addr, const void* gptr, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gptr), "r"(src_bytes));
}
__device__ __forceinline__ float4 lds_f4(uint32_t smem_addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_addr));
  return v;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
// Programmatic dependent launch.  A kernel launched with the stream-serialization attribute may
// become resident while the kernel before it in the stream is still running; it must not touch
// global memory until griddep_wait() returns (the predecessor has completed and its writes are
// visible).  griddep_launch() lets the kernel after this one become resident in the same way.
// Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
// streaming 128-bit global load that does not allocate in L1
__device__ __forceinline__ float4 ldg_stream_f4(const void* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];\n"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// ---- small numeric helpers --------------------------------------------------------
// fp32 pair -> (fp16x2 hi, fp16x2 lo) with hi + lo == value to ~2^-22 relative.
__device__ __forceinline__ void split_f16x2(float a, float b, uint32_t& hi, uint32_t& lo) {
  __half2 h = __floats2half2_rn(a, b);
  float2 hf = __half22float2(h);
  __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
  hi = *reinterpret_cast<uint32_t*>(&h);
  lo = *reinterpret_cast<uint32_t*>(&l);
}
__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void split_bf16x2(float a, float b, uint32_t& hi, uint32_t& lo) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  float2 hf = __bfloat1622float2(h);
  __nv_bfloat162 l = __floats2bfloat162_rn(a - hf.x, b - hf.y);
  hi = *reinterpret_cast<uint32_t*>(&h);
  lo = *reinterpret_cast<uint32_t*>(&l);
}

__device__ __forceinline__ float load_as_float(const void* base, int dtype, int64_t idx) {
  if (dtype == SPHKV_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == SPHKV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}
__device__ __forceinline__ void store_from_float(void* base, int dtype, int64_t idx, float v) {
  if (dtype == SPHKV_F32)
    reinterpret_cast<float*>(base)[idx] = v;
  else if (dtype == SPHKV_BF16)
    reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
}

// Work split shared by the decode kernel and its merge: CTA c of n covers global
// block indices [c*T/n, (c+1)*T/n).
__host__ __device__ __forceinline__ int64_t cta_range_start(int c, int n, int64_t T) {
  return (int64_t)c * T / n;
}

// One token of one KV head appended to a LayerPool page (decode_kernel.cu:10-84): nearest
// centroid per group on the normalised key, running-max radius scale with in-place
// re-quantisation of the slots already in the page, fp16 value row.  Called by every thread
// of a CTA of 32 * G threads (warp = group, lanes split the centroids); blockIdx.x = KV head.
__device__ __forceinline__ void pool_append_token(
    const float* __restrict__ k_post, const float* __restrict__ v_new,
    const float* __restrict__ decode_cb, uint8_t* __restrict__ theta_codes,
    uint8_t* __restrict__ radius_codes, float* __restrict__ r_scales, __half* __restrict__ v_pool,
    int64_t pid, int slot, int G, int g, int C, int G_max, int dh, int page_size, int is_new_page) {
  const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t v_base = (pid * page_size + slot) * dh;
  const int64_t code_base = (pid * page_size + slot) * G_max;
  for (int d = tid; d < dh; d += blockDim.x) v_pool[v_base + d] = __float2half(v_new[(int64_t)h * dh + d]);
  if (warp >= G) return;
  const int grp = warp;
  const float* k_g = k_post + (int64_t)h * dh + grp * g;
  float norm_sq = 0.f;
  for (int d = 0; d < g; ++d) norm_sq += k_g[d] * k_g[d];
  const float norm = sqrtf(norm_sq + 1e-16f);
  const float inv_norm = 1.0f / (norm + 1e-8f);
  const float* cb = decode_cb + ((int64_t)h * G * C + (int64_t)grp * C) * g;
  float best_sim = -1e30f;
  int best_code = 0;
  for (int c = lane; c < C; c += 32) {  // ascending per lane: strict > keeps the lowest index
    float sim = 0.f;
    for (int d = 0; d < g; ++d) sim += k_g[d] * inv_norm * cb[(int64_t)c * g + d];
    if (sim > best_sim) { best_sim = sim; best_code = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float os = __shfl_xor_sync(0xffffffffu, best_sim, o);
    const int oc = __shfl_xor_sync(0xffffffffu, best_code, o);
    if (os > best_sim || (os == best_sim && oc < best_code)) { best_sim = os; best_code = oc; }
  }
  float r_scale;
  const float prev_scale = is_new_page ? 0.f : r_scales[pid * G_max + grp];
  if (is_new_page || norm > prev_scale) {
    if (!is_new_page) {
      const float ratio = prev_scale / (norm + 1e-8f);
      for (int t = lane; t < slot; t += 32) {
        const int64_t idx = (pid * page_size + t) * G_max + grp;
        float rescaled = (float)radius_codes[idx] * ratio;
        rescaled = fminf(fmaxf(roundf(rescaled), 0.f), 255.f);
        radius_codes[idx] = (uint8_t)rescaled;
      }
    }
    r_scale = norm;
  } else {
    r_scale = prev_scale;
  }
  if (lane == 0) {
    theta_codes[code_base + grp] = (uint8_t)best_code;
    if (is_new_page || norm > prev_scale) r_scales[pid * G_max + grp] = norm;
    float r_q = roundf(norm / (r_scale + 1e-8f) * 255.0f);
    r_q = fminf(fmaxf(r_q, 0.f), 255.f);
    radius_codes[code_base + grp] = (uint8_t)r_q;
  }
}

}  // namespace sphkv
