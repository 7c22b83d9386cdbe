// Kernels behind the reference's existing operator signatures.
//
//   sphkv_pool_decode         fused_decode.sphkv_decode        (fused_decode.py:12-26)
//   sphkv_pool_encode_append  fused_decode.sphkv_encode_append (fused_decode.py:28-35)
//   sphkv_qlut_logits         new_fused_decode.sphkv_logits    (new_fused_decode.py:22-43)
//   sphkv_ragged_logits       fused_decode.fused_decode_ragged (call sites only:
//                             spherical_kv_pipeline.py:1109-1125, 1866-1870)
//
// They read the LayerPool layout (sphkv_lut.py:77-103): one byte per centroid index and
// per radius code, post-RoPE keys, single sequence.  The arithmetic of
// decode_kernel.cu:10-246 is kept (sentinel mask for zero logits, +1e-8 in the final
// division, running-max radius scale with in-place re-quantisation); the work split is
// new: one CTA serves all query heads of a KV head per page through a q.centroid look-up
// table instead of staging a 64 KiB codebook per (query head, page).
#include "common.cuh"

namespace sphkv {

constexpr int kPoolThreads = 256;

// ---- pool decode: per (KV head, logical page) partial (m, l, acc) for each query head ----
// The q.centroid table depends only on (query head, tier), not on the page: a CTA builds the
// tables of ALL tiers of its KV head once, then each of its warps walks pages on its own (no
// CTA barrier per page): logits through the table, softmax statistics by shuffles, and one
// pass over the page's V rows that feeds the accumulators of four query heads at a time.
constexpr int kPoolWarps = kPoolThreads / 32;
constexpr int kMaxPagesPerWarp = 4;  // fewer when the grid would not fill the GPU

__global__ void __launch_bounds__(kPoolThreads) pool_page_kernel(
    const float* __restrict__ q_all, const float* __restrict__ cb_flat,
    const int* __restrict__ tier_G_arr, const int* __restrict__ tier_g_arr,
    const uint8_t* __restrict__ theta_codes, const uint8_t* __restrict__ radius_codes,
    const float* __restrict__ r_scales, const __half* __restrict__ v_pool,
    const int* __restrict__ block_table, const int* __restrict__ bits_table,
    float* __restrict__ partial_out, int num_q_heads, int kv_groups, int num_tiers, int max_blocks,
    int page_size, int dh, int G_max, int cb_max, int g_max, float sm_scale, int pages_per_warp) {
  const int hkv = blockIdx.x, tid = threadIdx.x;
  const int hq0 = hkv * kv_groups;
  const int warp = tid >> 5, lane = tid & 31;

  extern __shared__ __align__(16) uint8_t smem_raw[];
  float* sq = reinterpret_cast<float*>(smem_raw);                 // [kv_groups][dh]
  float* lut = sq + kv_groups * dh;                                // [num_tiers][kv_groups][G_max][cb_max]
  float* slog_all = lut + num_tiers * kv_groups * G_max * cb_max;  // [warps][kv_groups][page_size]
  float* srs_all = slog_all + kPoolWarps * kv_groups * page_size;  // [warps][G_max]
  float* slog = slog_all + warp * kv_groups * page_size;
  float* srs = srs_all + warp * G_max;

  for (int i = tid; i < kv_groups * dh; i += blockDim.x) sq[i] = q_all[(int64_t)hq0 * dh + i];
  __syncthreads();
  // q . centroid tables of every tier; same summation order as decode_kernel.cu:186-188
  for (int ti = 0; ti < num_tiers; ++ti) {
    const int G = tier_G_arr[ti], g = tier_g_arr[ti];
    const float* cb_t = cb_flat + ((int64_t)hkv * num_tiers + ti) * G_max * cb_max * g_max;
    const bool vec4 = ((g | g_max) & 3) == 0 && (reinterpret_cast<uintptr_t>(cb_flat) & 15) == 0;
    float* lt = lut + (int64_t)ti * kv_groups * G_max * cb_max;
    for (int i = tid; i < kv_groups * G * cb_max; i += blockDim.x) {
      const int c = i % cb_max, gg = (i / cb_max) % G, h = i / (cb_max * G);
      const float* qg = sq + h * dh + gg * g;
      const float* cw = cb_t + ((int64_t)gg * cb_max + c) * g_max;
      float dot = 0.f;
      if (vec4) {  // same left-to-right order, 16-byte loads
        for (int d = 0; d < g; d += 4) {
          const float4 w4 = __ldg(reinterpret_cast<const float4*>(cw + d));
          dot += qg[d] * w4.x;
          dot += qg[d + 1] * w4.y;
          dot += qg[d + 2] * w4.z;
          dot += qg[d + 3] * w4.w;
        }
      } else {
        for (int d = 0; d < g; ++d) dot += qg[d] * cw[d];
      }
      lt[(h * G_max + gg) * cb_max + c] = dot;
    }
  }
  __syncthreads();

  const int pg0 = blockIdx.y * kPoolWarps * pages_per_warp;
  for (int k = 0; k < pages_per_warp; ++k) {
    const int page_idx = pg0 + warp + k * kPoolWarps;  // warp-uniform
    if (page_idx >= max_blocks) break;
    const int phys = block_table[hkv * max_blocks + page_idx];
    if (phys < 0) {
      for (int h = 0; h < kv_groups; ++h) {
        float* po = partial_out + ((int64_t)(hq0 + h) * max_blocks + page_idx) * (dh + 2);
        if (lane == 0) { po[0] = -INFINITY; po[1] = 0.f; }
        for (int d = lane; d < dh; d += 32) po[2 + d] = 0.f;
      }
      continue;
    }
    const int tier_idx = bits_table[hkv * max_blocks + page_idx];
    const int G = tier_G_arr[tier_idx];
    const float* lt = lut + (int64_t)tier_idx * kv_groups * G_max * cb_max;
    __syncwarp();  // the previous page's readers of slog / srs are done
    for (int i = lane; i < G_max; i += 32) srs[i] = r_scales[(int64_t)phys * G_max + i];
    __syncwarp();
    // logits: lane = (token, query head) pairs.  A byte becomes a float by planting it in the
    // mantissa of 2^23 (exact, and keeps the conversion off the special-function pipe).
    const bool words = (G_max & 3) == 0;
    for (int i = lane; i < page_size * kv_groups; i += 32) {
      const int t = i % page_size, h = i / page_size;
      const uint8_t* th = theta_codes + ((int64_t)phys * page_size + t) * G_max;
      const uint8_t* rc = radius_codes + ((int64_t)phys * page_size + t) * G_max;
      const float* lh = lt + (int64_t)h * G_max * cb_max;
      float logit_sum = 0.f;
      if (words) {
        for (int g0 = 0; g0 < G; g0 += 4) {
          const uint32_t tw = __ldg(reinterpret_cast<const uint32_t*>(th + g0));
          const uint32_t rw = __ldg(reinterpret_cast<const uint32_t*>(rc + g0));
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (g0 + e < G) {
              const float rf = __uint_as_float(0x4B000000u | ((rw >> (8 * e)) & 0xFFu)) - 8388608.0f;
              const float r_hat = srs[g0 + e] * rf / 255.0f;
              logit_sum += r_hat * lh[(g0 + e) * cb_max + ((tw >> (8 * e)) & 0xFFu)];
            }
          }
        }
      } else {
        for (int gg = 0; gg < G; ++gg) {
          const float r_hat = srs[gg] * (float)rc[gg] / 255.0f;
          logit_sum += r_hat * lh[gg * cb_max + th[gg]];
        }
      }
      slog[h * page_size + t] = (logit_sum == 0.f) ? -1e9f : logit_sum * sm_scale;
    }
    __syncwarp();
    // softmax statistics per head; the logits are replaced in place by exp(logit - max)
    for (int h = 0; h < kv_groups; ++h) {
      float* lg = slog + h * page_size;
      float m = -INFINITY;
      for (int t = lane; t < page_size; t += 32) m = fmaxf(m, lg[t]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      float l = 0.f;
      for (int t = lane; t < page_size; t += 32) {
        const float pt = __expf(lg[t] - m);
        lg[t] = pt;
        l += pt;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
      if (lane == 0) {
        float* po = partial_out + ((int64_t)(hq0 + h) * max_blocks + page_idx) * (dh + 2);
        po[0] = m;
        po[1] = l;
      }
    }
    __syncwarp();
    // V accumulation: a lane owns 4 dimensions, one pass over the rows feeds four heads
    for (int h0 = 0; h0 < kv_groups; h0 += 4) {
      for (int d0 = 4 * lane; d0 < dh; d0 += 128) {
        float acc[4][4];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) acc[hh][0] = acc[hh][1] = acc[hh][2] = acc[hh][3] = 0.f;
        const __half* vp = v_pool + (int64_t)phys * page_size * dh + d0;
#pragma unroll 4
        for (int t = 0; t < page_size; ++t) {
          const uint2 raw = __ldg(reinterpret_cast<const uint2*>(vp + (int64_t)t * dh));
          const float2 va = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
          const float2 vb = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
#pragma unroll
          for (int hh = 0; hh < 4; ++hh) {
            if (h0 + hh < kv_groups) {
              const float pt = slog[(h0 + hh) * page_size + t];
              acc[hh][0] += pt * va.x;
              acc[hh][1] += pt * va.y;
              acc[hh][2] += pt * vb.x;
              acc[hh][3] += pt * vb.y;
            }
          }
        }
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
          if (h0 + hh < kv_groups) {
            float* po = partial_out + ((int64_t)(hq0 + h0 + hh) * max_blocks + page_idx) * (dh + 2) + 2 + d0;
            *reinterpret_cast<float2*>(po) = make_float2(acc[hh][0], acc[hh][1]);
            *reinterpret_cast<float2*>(po + 2) = make_float2(acc[hh][2], acc[hh][3]);
          }
        }
      }
    }
  }
}

// log-sum-exp merge of the page partials (decode_kernel.cu:221-246).  The reference folds the
// pages into a running (max, sum, acc) one after the other; here the maximum over the pages is
// found first and every page is weighted by exp(m_page - max) directly, which gives the same
// result without a serial chain of rescales: one CTA per query head, pages in chunks whose
// weights are shared through shared memory, threads over the head dimension.
constexpr int kReduceThreads = 1024;  // 32 dimension lanes x 32 page lanes
constexpr int kReduceChunk = 1024;

// grid (query heads, dh / 32): a CTA owns 32 output dimensions of one head
__global__ void __launch_bounds__(kReduceThreads) pool_reduce_kernel(const float* __restrict__ partial_out,
                                                                     float* __restrict__ out, int dh,
                                                                     int max_pages) {
  const int hq = blockIdx.x, tid = threadIdx.x, lane = tid & 31, pl = tid >> 5;  // lane = dimension lane
  const int d = blockIdx.y * 32 + lane;
  __shared__ float s_w[kReduceChunk];
  __shared__ float s_red[32];
  __shared__ float s_acc[32][33];
  __shared__ float s_l[32];
  const float* base = partial_out + (int64_t)hq * max_pages * (dh + 2);
  const int64_t row = dh + 2;
  float M = -INFINITY;
  for (int pg = tid; pg < max_pages; pg += kReduceThreads) {
    const float m_s = base[pg * row], l_s = base[pg * row + 1];
    if (!(m_s == -INFINITY && l_s == 0.f)) M = fmaxf(M, m_s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  if (lane == 0) s_red[pl] = M;
  __syncthreads();
  M = s_red[0];
  for (int i = 1; i < 32; ++i) M = fmaxf(M, s_red[i]);
  float l_f = 0.f, a_f = 0.f;
  for (int p0 = 0; p0 < max_pages; p0 += kReduceChunk) {
    const int np = min(kReduceChunk, max_pages - p0);
    __syncthreads();
    for (int i = tid; i < np; i += kReduceThreads) {
      const float m_s = base[(p0 + i) * row], l_s = base[(p0 + i) * row + 1];
      s_w[i] = (m_s == -INFINITY && l_s == 0.f) ? 0.f : __expf(m_s - M);
    }
    __syncthreads();
    // every page row was written by pool_page_kernel (zeros for holes): zero weights need no branch
#pragma unroll 4
    for (int i = pl; i < np; i += 32) {
      const float w = s_w[i];
      const float* pr = base + (p0 + i) * row;
      l_f += w * pr[1];
      if (d < dh) a_f += w * pr[2 + d];
    }
  }
  // fold the 32 page lanes in a fixed order
  s_acc[pl][lane] = a_f;
  if (lane == 0) s_l[pl] = l_f;
  __syncthreads();
  if (pl == 0 && d < dh) {
    float l_t = 0.f, a_t = 0.f;
    for (int k = 0; k < 32; ++k) {
      l_t += s_l[k];
      a_t += s_acc[k][lane];
    }
    out[(int64_t)hq * dh + d] = a_t / (l_t + 1e-8f);
  }
}

// ---- encode + append of one token per KV head, decode_kernel.cu:10-84 -----------------------
// grid = KV heads, block = 32 * G: warp = group, lanes split the centroids.  The arithmetic
// lives in pool_append_token (common.cuh), shared with the device-bookkeeping step kernel.
__global__ void pool_encode_append_kernel(
    const float* __restrict__ k_post, const float* __restrict__ v_new,
    const float* __restrict__ decode_cb, uint8_t* __restrict__ theta_codes,
    uint8_t* __restrict__ radius_codes, float* __restrict__ r_scales, __half* __restrict__ v_pool,
    const int64_t* __restrict__ pids, int slot, int G, int g, int C, int G_max, int dh,
    int page_size, int is_new_page) {
  pool_append_token(k_post, v_new, decode_cb, theta_codes, radius_codes, r_scales, v_pool,
                    pids[blockIdx.x], slot, G, g, C, G_max, dh, page_size, is_new_page);
}

// ---- logits from a precomputed q.centroid table (new_fused_decode.cpp:3-22) ------------------
// q_lut f32 [Hq][num_tiers][G_max][cb_size_max]; logits_out f32 [Hq][max_blocks*page_size].
// Holes, slots past ctx_lens and exact-zero logits get the -1e9 sentinel of
// decode_kernel.cu:194.  Tier geometry comes from the table itself: groups >= G of a tier
// have zero radius codes in the pool and contribute nothing.
__global__ void qlut_logits_kernel(const float* __restrict__ q_lut,
                                   const uint8_t* __restrict__ theta_codes,
                                   const uint8_t* __restrict__ radius_codes,
                                   const float* __restrict__ r_scales,
                                   const int* __restrict__ block_table,
                                   const int* __restrict__ bits_table,
                                   const int* __restrict__ ctx_lens, float* __restrict__ logits_out,
                                   int num_q_heads, int kv_groups, int num_tiers, int max_blocks,
                                   int page_size, int G_max, int cb_size_max, float sm_scale) {
  const int hkv = blockIdx.x, page_idx = blockIdx.y;
  const int phys = block_table[hkv * max_blocks + page_idx];
  const int tier_idx = phys >= 0 ? bits_table[hkv * max_blocks + page_idx] : 0;
  const int ctx = ctx_lens ? ctx_lens[hkv] : max_blocks * page_size;
  for (int i = threadIdx.x; i < kv_groups * page_size; i += blockDim.x) {
    const int h = i / page_size, t = i - h * page_size;
    const int hq = hkv * kv_groups + h;
    float outv = -1e9f;
    if (phys >= 0 && page_idx * page_size + t < ctx) {
      const uint8_t* th = theta_codes + ((int64_t)phys * page_size + t) * G_max;
      const uint8_t* rc = radius_codes + ((int64_t)phys * page_size + t) * G_max;
      const float* lut = q_lut + ((int64_t)hq * num_tiers + tier_idx) * G_max * cb_size_max;
      float s = 0.f;
      for (int gg = 0; gg < G_max; ++gg) {
        const float r_hat = r_scales[(int64_t)phys * G_max + gg] * (float)rc[gg] / 255.0f;
        s += r_hat * lut[gg * cb_size_max + th[gg]];
      }
      if (s != 0.f) outv = s * sm_scale;
    }
    logits_out[(int64_t)hq * max_blocks * page_size + (int64_t)page_idx * page_size + t] = outv;
  }
}

// ---- logits over bit-packed byte pages with per-token back-rotation --------------------------
// Restates spherical_kv_pipeline.py:2143-2176 per (token, query head): rotate q by the key
// position with the caller's HF-layout tables, normalise per group, clamp the cosine,
// weight by the de-quantised radius.  Output [Hq][n_pages * page_size]; slots with
// position < 0 or past the page count, and heads outside the page's KV head, get 0.
__global__ void ragged_logits_kernel(const uint8_t* __restrict__ pages,
                                     const int* __restrict__ ptable,
                                     const int* __restrict__ head_ids,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ cos_tbl,
                                     const float* __restrict__ sin_tbl, const float* __restrict__ q,
                                     const float* __restrict__ codebooks,
                                     float* __restrict__ logits_out, int grp, int num_kv, int dh,
                                     int G, int g, int b_theta, int page_size, int n_pages, int Hq,
                                     int table_rows, int radius_fmt) {
  const int pg = blockIdx.x;
  const int hkv = head_ids[pg];
  const int poff = ptable[3 * pg], toff = ptable[3 * pg + 1], roff = ptable[3 * pg + 2];
  const int count = pages[poff + 1];
  const int C = 1 << b_theta, half = dh >> 1;
  const float inv_sqrt = rsqrtf((float)dh);
  const int64_t out_stride = (int64_t)n_pages * page_size;
  for (int i = threadIdx.x; i < Hq * page_size; i += blockDim.x) {
    const int hq = i / page_size, t = i - hq * page_size;
    float outv = 0.f;
    const int pos = positions[(int64_t)pg * page_size + t];
    if (hq / grp == hkv && hkv < num_kv && t < count && pos >= 0 && pos < table_rows) {
      const float* qh = q + (int64_t)hq * dh;
      const float* cr = cos_tbl + (int64_t)pos * dh;
      const float* sr = sin_tbl + (int64_t)pos * dh;
      for (int gg = 0; gg < G; ++gg) {
        const int64_t bit = ((int64_t)t * G + gg) * b_theta;
        uint32_t w = 0;
        for (int bb = 0; bb < 2; ++bb) w |= (uint32_t)pages[toff + (bit >> 3) + bb] << (8 * bb);
        const int code = (int)((w >> (bit & 7)) & (uint32_t)(C - 1));
        float rad;
        if (radius_fmt == SPHKV_RADIUS_F16) {
          const uint16_t hv = (uint16_t)pages[roff + 2 * (t * G + gg)] |
                              ((uint16_t)pages[roff + 2 * (t * G + gg) + 1] << 8);
          rad = __half2float(__ushort_as_half(hv));
        } else {
          float sc;
          memcpy(&sc, pages + poff + 8 + 4 * gg, 4);
          rad = sc * (float)(int8_t)pages[roff + t * G + gg] / 127.0f;
        }
        const float* cw = codebooks + ((int64_t)(hkv * G + gg) * C + code) * g;
        float nsq = 0.f, dot = 0.f;
        for (int d = 0; d < g; ++d) {
          const int dd = gg * g + d;
          const float rh = dd < half ? -qh[dd + half] : qh[dd - half];
          const float qr = qh[dd] * cr[dd] - rh * sr[dd];
          nsq += qr * qr;
          dot += qr * cw[d];
        }
        const float qn = fmaxf(sqrtf(nsq), 1e-6f);
        const float cpg = fminf(fmaxf(dot / qn, -1.f), 1.f);
        outv += qn * cpg * rad;
      }
      outv *= inv_sqrt;
    }
    logits_out[(int64_t)hq * out_stride + (int64_t)pg * page_size + t] = outv;
  }
}

}  // namespace sphkv

using namespace sphkv;

static int sphkv_sm_count_or(int fallback) {
  const int sms = sm_count_current_device();
  return sms > 0 ? sms : fallback;
}

extern "C" int sphkv_pool_decode(const float* q_all, const float* cb_flat, const int32_t* tier_G,
                                 const int32_t* tier_g, const uint8_t* theta_codes,
                                 const uint8_t* radius_codes, const float* r_scales,
                                 const void* v_pool, const int32_t* block_table,
                                 const int32_t* bits_table, const int32_t* ctx_lens, float* out,
                                 float* partial_scratch, int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t kv_groups, int32_t num_tiers, int32_t max_blocks,
                                 int32_t page_size, int32_t dh, int32_t G_max, int32_t cb_max,
                                 int32_t g_max, float sm_scale, int32_t max_ctx, void* stream) {
  (void)ctx_lens;  // validity is encoded by block_table == -1 and the zero-logit sentinel,
  (void)max_ctx;   // as in decode_kernel.cu:120,139-144,194
  SPHKV_REQUIRE(q_all && cb_flat && tier_G && tier_g && theta_codes && radius_codes && r_scales &&
                    v_pool && block_table && bits_table && out && partial_scratch,
                SPHKV_E_ARG, "pool_decode: NULL pointer");
  SPHKV_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && kv_groups > 0 &&
                    num_q_heads == num_kv_heads * kv_groups,
                SPHKV_E_ARG, "pool_decode: Hq=%d Hkv=%d groups=%d", num_q_heads, num_kv_heads,
                kv_groups);
  SPHKV_REQUIRE(max_blocks > 0 && page_size > 0 && dh > 0 && dh <= 512 && (dh & 3) == 0 && G_max > 0 &&
                    cb_max > 0 && g_max > 0 && num_tiers > 0,
                SPHKV_E_ARG, "pool_decode: bad size");
  SPHKV_REQUIRE((reinterpret_cast<uintptr_t>(v_pool) & 7) == 0 && (reinterpret_cast<uintptr_t>(partial_scratch) & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(theta_codes) & 3) == 0 && (reinterpret_cast<uintptr_t>(radius_codes) & 3) == 0,
                SPHKV_E_ALIGN, "pool_decode: v_pool / partial_scratch need 8 B, code arrays 4 B alignment");
  const size_t smem = ((size_t)kv_groups * dh + (size_t)num_tiers * kv_groups * G_max * cb_max +
                       (size_t)kPoolWarps * ((size_t)kv_groups * page_size + G_max)) * sizeof(float);
  SPHKV_REQUIRE(smem <= 200 * 1024, SPHKV_E_LIMIT, "pool_decode: needs %zu B shared memory", smem);
  {
    static SmemOptIn opt_in;
    if (int rc = ensure_dynamic_smem(opt_in, (const void*)pool_page_kernel, (int)smem, "pool_decode")) return rc;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // pages per warp: up to kMaxPagesPerWarp (amortises the table build), fewer while the grid is small
  int ppw = (int)(((int64_t)num_kv_heads * max_blocks) / ((int64_t)kPoolWarps * 2 * sphkv_sm_count_or(148)));
  ppw = ppw < 1 ? 1 : (ppw > kMaxPagesPerWarp ? kMaxPagesPerWarp : ppw);
  const int ppc = kPoolWarps * ppw;
  pool_page_kernel<<<dim3(num_kv_heads, (max_blocks + ppc - 1) / ppc), kPoolThreads, smem, st>>>(
      q_all, cb_flat, tier_G, tier_g, theta_codes, radius_codes, r_scales,
      reinterpret_cast<const __half*>(v_pool), block_table, bits_table, partial_scratch,
      num_q_heads, kv_groups, num_tiers, max_blocks, page_size, dh, G_max, cb_max, g_max, sm_scale, ppw);
  if (int rc = check_launch("pool_page_kernel")) return rc;
  pool_reduce_kernel<<<dim3(num_q_heads, (dh + 31) / 32), kReduceThreads, 0, st>>>(partial_scratch, out, dh, max_blocks);
  return check_launch("pool_reduce_kernel");
}

extern "C" int sphkv_pool_encode_append(const float* k_post, const float* v_new,
                                        const float* decode_cb, uint8_t* theta_codes,
                                        uint8_t* radius_codes, float* r_scales, void* v_pool,
                                        const int64_t* pids, int32_t slot, int32_t G, int32_t g,
                                        int32_t C, int32_t G_max, int32_t dh, int32_t page_size,
                                        int32_t is_new_page, int32_t num_kv, void* stream) {
  SPHKV_REQUIRE(k_post && v_new && decode_cb && theta_codes && radius_codes && r_scales && v_pool &&
                    pids,
                SPHKV_E_ARG, "encode_append: NULL pointer");
  SPHKV_REQUIRE(num_kv > 0 && G > 0 && G <= 32 && g > 0 && C > 0 && G <= G_max && G * g <= dh &&
                    slot >= 0 && slot < page_size,
                SPHKV_E_ARG, "encode_append: G=%d g=%d C=%d G_max=%d dh=%d slot=%d page_size=%d", G,
                g, C, G_max, dh, slot, page_size);
  pool_encode_append_kernel<<<num_kv, 32 * G, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      k_post, v_new, decode_cb, theta_codes, radius_codes, r_scales,
      reinterpret_cast<__half*>(v_pool), pids, slot, G, g, C, G_max, dh, page_size, is_new_page);
  return check_launch("pool_encode_append_kernel");
}

extern "C" int sphkv_qlut_logits(const float* q_lut, const uint8_t* theta_codes,
                                 const uint8_t* radius_codes, const float* r_scales,
                                 const int32_t* block_table, const int32_t* bits_table,
                                 const int32_t* ctx_lens, float* logits_out, int32_t num_q_heads,
                                 int32_t num_kv_heads, int32_t kv_groups, int32_t num_tiers,
                                 int32_t max_blocks, int32_t page_size, int32_t G_max,
                                 int32_t cb_size_max, float sm_scale, int32_t max_ctx,
                                 void* stream) {
  (void)max_ctx;
  SPHKV_REQUIRE(q_lut && theta_codes && radius_codes && r_scales && block_table && bits_table &&
                    logits_out,
                SPHKV_E_ARG, "qlut_logits: NULL pointer");
  SPHKV_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads == num_kv_heads * kv_groups &&
                    max_blocks > 0 && page_size > 0 && G_max > 0 && cb_size_max > 0 && num_tiers > 0,
                SPHKV_E_ARG, "qlut_logits: bad size");
  qlut_logits_kernel<<<dim3(num_kv_heads, max_blocks), 128, 0,
                       reinterpret_cast<cudaStream_t>(stream)>>>(
      q_lut, theta_codes, radius_codes, r_scales, block_table, bits_table, ctx_lens, logits_out,
      num_q_heads, kv_groups, num_tiers, max_blocks, page_size, G_max, cb_size_max, sm_scale);
  return check_launch("qlut_logits_kernel");
}

extern "C" int sphkv_ragged_logits(const uint8_t* pages, const int32_t* ptable,
                                   const int32_t* head_ids, const int32_t* positions,
                                   const float* cos_tbl, const float* sin_tbl, const float* q,
                                   const float* codebooks, float* logits_out, int32_t grp,
                                   int32_t num_kv, int32_t dh, int32_t G, int32_t g, int32_t b_theta,
                                   int32_t page_size, int32_t n_pages, int32_t Hq,
                                   int32_t table_rows, int32_t radius_fmt, int32_t reserved,
                                   void* stream) {
  (void)reserved;
  SPHKV_REQUIRE(pages && ptable && head_ids && positions && cos_tbl && sin_tbl && q && codebooks &&
                    logits_out,
                SPHKV_E_ARG, "ragged_logits: NULL pointer");
  SPHKV_REQUIRE(n_pages > 0 && grp > 0 && num_kv > 0 && Hq == grp * num_kv && G * g == dh &&
                    (dh & 1) == 0 && b_theta >= 1 && b_theta <= 8 && page_size > 0 && table_rows > 0,
                SPHKV_E_ARG, "ragged_logits: bad size (Hq=%d grp=%d num_kv=%d G=%d g=%d dh=%d)", Hq,
                grp, num_kv, G, g, dh);
  ragged_logits_kernel<<<n_pages, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pages, ptable, head_ids, positions, cos_tbl, sin_tbl, q, codebooks, logits_out, grp, num_kv,
      dh, G, g, b_theta, page_size, n_pages, Hq, table_rows, radius_fmt);
  return check_launch("ragged_logits_kernel");
}

// ---- page-level importance EMA from per-block (m, l) --------------------------------------------
// _omega_ema_eager (spherical_kv_pipeline.py:952-987) in one launch: per query head the block
// weights exp(max(m - m_max, -60)) * l are normalised over the blocks, averaged over the query
// heads of a KV head and blended into omega with factor beta.  ml points at the (m, l) pairs of
// (query head, block): element (hq, blk) lives at ml[(hq * max_blocks + blk) * stride + {0, 1}]
// (stride = dh + 2 for the partial_scratch of sphkv_pool_decode, 2 for page_ml of
// sphkv_decode_paged).  omega [n_units][max_blocks] is updated in place; unit u owns query heads
// u * kv_groups .. (u + 1) * kv_groups - 1.
namespace sphkv {
__global__ void omega_ema_kernel(const float* __restrict__ ml, float* __restrict__ omega,
                                 int kv_groups, int max_blocks, int stride, float beta) {
  const int u = blockIdx.x;
  __shared__ float s_red[32];
  __shared__ float s_val;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  auto block_reduce = [&](float v, bool is_max) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float t = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, t) : v + t;
    }
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    if (warp == 0) {
      float x = lane < nw ? s_red[lane] : (is_max ? -INFINITY : 0.f);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, x, o);
        x = is_max ? fmaxf(x, t) : x + t;
      }
      if (lane == 0) s_val = x;
    }
    __syncthreads();
    const float r = s_val;
    __syncthreads();
    return r;
  };
  // mass accumulated over the group's query heads, blocks strided over the threads
  extern __shared__ float s_mass[];  // [max_blocks]
  for (int i = threadIdx.x; i < max_blocks; i += blockDim.x) s_mass[i] = 0.f;
  __syncthreads();
  for (int h = 0; h < kv_groups; ++h) {
    const float* base = ml + ((int64_t)(u * kv_groups + h) * max_blocks) * stride;
    float mx = -1e30f;
    for (int i = threadIdx.x; i < max_blocks; i += blockDim.x) {
      const float m = base[(int64_t)i * stride], l = base[(int64_t)i * stride + 1];
      mx = fmaxf(mx, l > 0.f ? m : -1e30f);
    }
    mx = block_reduce(mx, true);
    float z = 0.f;
    for (int i = threadIdx.x; i < max_blocks; i += blockDim.x) {
      const float m = base[(int64_t)i * stride], l = base[(int64_t)i * stride + 1];
      const float ms = l > 0.f ? m : -1e30f;
      z += __expf(fmaxf(ms - mx, -60.f)) * l;
    }
    z = fmaxf(block_reduce(z, false), 1e-12f);
    for (int i = threadIdx.x; i < max_blocks; i += blockDim.x) {
      const float m = base[(int64_t)i * stride], l = base[(int64_t)i * stride + 1];
      const float ms = l > 0.f ? m : -1e30f;
      s_mass[i] += __expf(fmaxf(ms - mx, -60.f)) * l / z;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < max_blocks; i += blockDim.x) {
    float* o = omega + (int64_t)u * max_blocks + i;
    *o = *o * beta + (s_mass[i] / (float)kv_groups) * (1.0f - beta);
  }
}
}  // namespace sphkv

extern "C" int sphkv_omega_ema(const float* ml, float* omega, int32_t n_units, int32_t kv_groups,
                               int32_t max_blocks, int32_t stride, float beta, void* stream) {
  SPHKV_REQUIRE(ml && omega, SPHKV_E_ARG, "omega_ema: NULL pointer");
  SPHKV_REQUIRE(n_units > 0 && kv_groups > 0 && max_blocks > 0 && stride >= 2, SPHKV_E_ARG,
                "omega_ema: n_units=%d kv_groups=%d max_blocks=%d stride=%d", n_units, kv_groups,
                max_blocks, stride);
  SPHKV_REQUIRE((size_t)max_blocks * 4 <= 160 * 1024, SPHKV_E_LIMIT,
                "omega_ema: max_blocks=%d exceeds 40960", max_blocks);
  const size_t smem = (size_t)max_blocks * 4;
  {
    static sphkv::SmemOptIn opt_in;
    if (int rc = sphkv::ensure_dynamic_smem(opt_in, (const void*)sphkv::omega_ema_kernel, (int)smem, "omega_ema"))
      return rc;
  }
  sphkv::omega_ema_kernel<<<n_units, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      ml, omega, kv_groups, max_blocks, stride, beta);
  return sphkv::check_launch("omega_ema_kernel");
}
