// Device-resident LayerPool management.
//
//   sphkv_pool_build_pages   bulk construction of pool pages from encode output; replaces the
//                            per-page Python loop of LayerPool.__init__ (sphkv_lut.py:37-68)
//   sphkv_pool_append_step   roll-over allocation, block/bits table update, token append and
//                            ctx_lens bump in ONE launch with all bookkeeping state on the
//                            device; replaces the host code of LayerPool.append_and_compute
//                            (sphkv_lut.py:150-186: list edits, two torch.tensor(list)
//                            re-uploads, the arange copy into _pids, sphkv_encode_append and
//                            ctx_lens_gpu.add_(1))
//
// Neither call reads device memory from the host, allocates or synchronises, so a decode
// step built from them can be recorded into a CUDA graph and replayed.
#include "common.cuh"

namespace sphkv {

// state words of a pool (int32 [4] in device memory)
enum { kStCtx = 0, kStUsed = 1, kStArrived = 2, kStError = 3 };

// ---- bulk page construction -----------------------------------------------------------------
// One CTA per destination page.  desc[p] = {src_row, n_rows, G_t, dst_pid}: rows
// src_row .. src_row+n_rows of r / theta / v_src fill slots 0 .. n_rows of page dst_pid; slots
// and groups beyond stay zero.  Arithmetic of sphkv_lut.py:50-60 in the same fp32 order:
// scale = max(amax over the page's rows, 1e-8); code = clamp(rint(r / scale * 255), 0, 255).
__global__ void __launch_bounds__(128) pool_build_kernel(
    const float* __restrict__ r, const uint8_t* __restrict__ theta, const void* __restrict__ v_src,
    int v_dtype, int64_t code_stride, int64_t v_stride, const int32_t* __restrict__ desc,
    uint8_t* __restrict__ theta_codes, uint8_t* __restrict__ radius_codes,
    float* __restrict__ r_scales, __half* __restrict__ v_pool, int page_size, int G_max, int dh) {
  __shared__ float scale_s[64];
  const int4 d = reinterpret_cast<const int4*>(desc)[blockIdx.x];
  const int64_t src = d.x;
  const int n_rows = d.y, G_t = d.z;
  const int64_t pid = d.w;
  const int tid = threadIdx.x;
  for (int grp = tid; grp < G_max; grp += blockDim.x) {
    float s = 0.f;
    if (grp < G_t) {
      s = -INFINITY;
      for (int t = 0; t < n_rows; ++t) s = fmaxf(s, r[(src + t) * code_stride + grp]);
      s = fmaxf(s, 1e-8f);
    }
    scale_s[grp] = s;
    r_scales[pid * G_max + grp] = s;
  }
  __syncthreads();
  for (int i = tid; i < page_size * G_max; i += blockDim.x) {
    const int t = i / G_max, grp = i - t * G_max;
    uint8_t th = 0, rq = 0;
    if (t < n_rows && grp < G_t) {
      th = theta[(src + t) * code_stride + grp];
      const float q = rintf(__fmul_rn(__fdiv_rn(r[(src + t) * code_stride + grp], scale_s[grp]), 255.0f));
      rq = (uint8_t)fminf(fmaxf(q, 0.f), 255.f);
    }
    theta_codes[pid * page_size * G_max + i] = th;
    radius_codes[pid * page_size * G_max + i] = rq;
  }
  for (int i = tid; i < page_size * dh; i += blockDim.x) {
    const int t = i / dh, c = i - t * dh;
    const float x = t < n_rows ? load_as_float(v_src, v_dtype, (src + t) * v_stride + c) : 0.f;
    v_pool[pid * page_size * dh + i] = __float2half_rn(x);
  }
}

// ---- one decode-step append with device bookkeeping -----------------------------------------
// grid = KV heads, block = 32 * G.  Every CTA reads the state words, derives (slot, new page?)
// like sphkv_lut.py:153-168, head h claims physical page used + h when a page opens, appends its
// token, and bumps ctx_lens[h].  The last CTA to finish (ticket in state[2]) publishes the new
// state, so no CTA can observe a half-updated one.  Running out of pool pages or of table
// columns sets state[3] and leaves every array untouched from then on.
__global__ void pool_append_step_kernel(
    const float* __restrict__ k_post, const float* __restrict__ v_new,
    const float* __restrict__ decode_cb, uint8_t* __restrict__ theta_codes,
    uint8_t* __restrict__ radius_codes, float* __restrict__ r_scales, __half* __restrict__ v_pool,
    int32_t* __restrict__ block_table, int32_t* __restrict__ bits_table,
    int32_t* __restrict__ ctx_lens, int64_t* __restrict__ pids, int32_t* __restrict__ state,
    int dec_tier_idx, int G, int g, int C, int G_max, int dh, int page_size, int max_blocks,
    int n_pool_pages) {
  __shared__ int s_cur, s_used, s_err;
  const int h = blockIdx.x, num_kv = gridDim.x, tid = threadIdx.x;
  if (tid == 0) {
    s_cur = state[kStCtx];
    s_used = state[kStUsed];
    s_err = state[kStError];
  }
  __syncthreads();
  const int cur = s_cur, used = s_used;
  const int slot = cur % page_size, pg = cur / page_size;
  const bool is_new = slot == 0;
  const bool full = is_new && (used + num_kv > n_pool_pages || pg >= max_blocks);
  const bool ok = s_err == 0 && !full && cur >= 0;
  if (ok) {
    int64_t pid;
    if (is_new) {
      pid = used + h;
      if (tid == 0) {
        block_table[(int64_t)h * max_blocks + pg] = used + h;
        bits_table[(int64_t)h * max_blocks + pg] = dec_tier_idx;
        pids[h] = pid;
      }
    } else {
      pid = pids[h];
    }
    pool_append_token(k_post, v_new, decode_cb, theta_codes, radius_codes, r_scales, v_pool, pid, slot,
                      G, g, C, G_max, dh, page_size, is_new ? 1 : 0);
    if (tid == 0) ctx_lens[h] += 1;
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int ticket = atomicAdd(&state[kStArrived], 1);
    if (ticket == num_kv - 1) {  // every CTA has read the old state and finished its writes
      if (ok) {
        state[kStCtx] = cur + 1;
        if (is_new) state[kStUsed] = used + num_kv;
      } else if (s_err == 0) {
        state[kStError] = 1;
      }
      state[kStArrived] = 0;
      __threadfence();
    }
  }
}

}  // namespace sphkv

using namespace sphkv;

extern "C" int sphkv_pool_build_pages(const float* r, const uint8_t* theta, const void* v_src,
                                      int32_t v_dtype, int64_t code_stride, int64_t v_stride,
                                      const int32_t* page_desc, int32_t n_pages, uint8_t* theta_codes,
                                      uint8_t* radius_codes, float* r_scales, void* v_pool,
                                      int32_t page_size, int32_t G_max, int32_t dh, void* stream) {
  SPHKV_REQUIRE(r && theta && v_src && page_desc && theta_codes && radius_codes && r_scales && v_pool,
                SPHKV_E_ARG, "pool_build_pages: NULL pointer");
  SPHKV_REQUIRE(n_pages >= 0 && page_size > 0 && G_max > 0 && G_max <= 64 && dh > 0 &&
                    code_stride >= G_max && v_stride >= dh &&
                    (v_dtype == SPHKV_F32 || v_dtype == SPHKV_F16 || v_dtype == SPHKV_BF16),
                SPHKV_E_ARG, "pool_build_pages: bad size (n_pages=%d page_size=%d G_max=%d dh=%d)",
                n_pages, page_size, G_max, dh);
  SPHKV_REQUIRE((reinterpret_cast<uintptr_t>(page_desc) & 15) == 0, SPHKV_E_ARG,
                "pool_build_pages: page_desc must be 16-byte aligned");
  if (n_pages == 0) return SPHKV_OK;
  pool_build_kernel<<<n_pages, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      r, theta, v_src, v_dtype, code_stride, v_stride, page_desc, theta_codes, radius_codes, r_scales,
      reinterpret_cast<__half*>(v_pool), page_size, G_max, dh);
  return check_launch("pool_build_kernel");
}

extern "C" int sphkv_pool_append_step(const float* k_post, const float* v_new, const float* decode_cb,
                                      uint8_t* theta_codes, uint8_t* radius_codes, float* r_scales,
                                      void* v_pool, int32_t* block_table, int32_t* bits_table,
                                      int32_t* ctx_lens, int64_t* pids, int32_t* state,
                                      int32_t dec_tier_idx, int32_t G, int32_t g, int32_t C,
                                      int32_t G_max, int32_t dh, int32_t page_size, int32_t num_kv,
                                      int32_t max_blocks, int32_t n_pool_pages, void* stream) {
  SPHKV_REQUIRE(k_post && v_new && decode_cb && theta_codes && radius_codes && r_scales && v_pool &&
                    block_table && bits_table && ctx_lens && pids && state,
                SPHKV_E_ARG, "pool_append_step: NULL pointer");
  SPHKV_REQUIRE(num_kv > 0 && G > 0 && G <= 32 && g > 0 && C > 0 && G <= G_max && G * g <= dh &&
                    page_size > 0 && max_blocks > 0 && n_pool_pages > 0 && dec_tier_idx >= 0,
                SPHKV_E_ARG, "pool_append_step: G=%d g=%d C=%d G_max=%d dh=%d page_size=%d num_kv=%d", G,
                g, C, G_max, dh, page_size, num_kv);
  pool_append_step_kernel<<<num_kv, 32 * G, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      k_post, v_new, decode_cb, theta_codes, radius_codes, r_scales, reinterpret_cast<__half*>(v_pool),
      block_table, bits_table, ctx_lens, pids, state, dec_tier_idx, G, g, C, G_max, dh, page_size,
      max_blocks, n_pool_pages);
  return check_launch("pool_append_step_kernel");
}
