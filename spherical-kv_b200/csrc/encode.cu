// Spherical encode + page build.
//
// One CTA encodes bundles of 128 token slots (128/page_size pages) that share a (KV head,
// tier slot): warp = group, lane = four tokens (every centroid row read from shared memory
// feeds four dot products).  Per
// (token, group) the kernel computes the group radius and the nearest centroid, then the
// CTA assembles each page image in shared memory in the reference byte layout
//   [tier_id u8][count u8][fmt u8][5 x 0][G x f32 scale][LSB-first packed theta][radii]
// (paging.py:20-31, pagebuilder.py:8-33, bitpacking.py:5-29) and copies it out, together
// with the dense 16-bit V page.
//
// Arithmetic order (what "bit-exact" is defined against):
//   nsq   = fma chain d = 0..g-1 of k_d * k_d starting from 0;  r = sqrt(nsq)   (IEEE)
//   sim_c = fma chain d = 0..g-1 of k_d * cb[c][d] starting from 0
//   theta = first c maximising sim_c (strict >), as torch.argmax / decode_kernel.cu:45-55
//   scale = max_t r ; code = clamp(rint((r / max(scale, 1e-8)) * 127), -127, 127)
// The similarity is taken on the un-normalised group vector: dividing by r first
// (spherical_kv_pipeline.py:1138) scales every sim_c by the same positive factor.
#include <algorithm>
#include "common.cuh"

namespace sphkv {

struct EncodeArgs {
  sphkv_encode_params p;
  int bundles_per_cta;
  int warp_smem_bytes;  // page assembly: shared memory of one warp
  int search_chunk;     // search launch: consecutive bundles a CTA takes at a time (1 .. 8)
};

constexpr int kEncThreads = 256;

// two 16-bit elements (bf16 or f16) of one 32-bit word, widened exactly
__device__ __forceinline__ void unpack16(uint32_t w, int dtype, float& lo, float& hi) {
  if (dtype == SPHKV_BF16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    lo = __low2float(h);
    hi = __high2float(h);
  }
}

template <int GS>
__device__ __forceinline__ void load_group(const void* base, int dtype, int64_t off, float (&k)[GS]) {
  if (dtype == SPHKV_F32 && (((uintptr_t)base + off * 4) & 15) == 0) {
    const float4* s = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
#pragma unroll
    for (int i = 0; i < GS / 4; ++i) {
      const float4 v = ldg_stream_f4(s + i);
      k[4 * i] = v.x; k[4 * i + 1] = v.y; k[4 * i + 2] = v.z; k[4 * i + 3] = v.w;
    }
  } else if (dtype != SPHKV_F32 && (((uintptr_t)base + off * 2) & 15) == 0) {
    const uint4* s =
        reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + off);
#pragma unroll
    for (int i = 0; i < GS / 8; ++i) {
      const uint4 v = __ldg(s + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) unpack16(w[e], dtype, k[8 * i + 2 * e], k[8 * i + 2 * e + 1]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < GS; ++i) k[i] = load_as_float(base, dtype, off + i);
  }
}

// Eight consecutive V elements starting at element offset `off` of v_src, as one 16-byte chunk
// of the 16-bit V pool (copied when the types agree, else rounded to nearest even).
__device__ __forceinline__ uint4 load_v_chunk(const sphkv_encode_params& p, bool same, int64_t off) {
  if (same && (((uintptr_t)p.v_src + off * 2) & 15) == 0)
    return __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.v_src) + off));
  float v[8];
  if (p.v_src_dtype == SPHKV_F32 && (((uintptr_t)p.v_src + off * 4) & 15) == 0) {
    const float4 a0 = ldg_stream_f4(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.v_src) + off));
    const float4 a1 = ldg_stream_f4(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.v_src) + off + 4));
    v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w;
    v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = load_as_float(p.v_src, p.v_src_dtype, off + e);
  }
  uint32_t w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (p.v_pool_dtype == SPHKV_F16) {
      w[e] = pack_f16x2(v[2 * e], v[2 * e + 1]);
    } else {
      __nv_bfloat162 hb2 = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
      w[e] = *reinterpret_cast<uint32_t*>(&hb2);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

constexpr int kMaxBundlesPerCta = 8;  // consecutive bundles one CTA walks (they mostly share a codebook)

// Squared norm and nearest centroid of four tokens' GS-dim group vectors: the fixed fma chains that
// define the encoder bit for bit (d = 0 .. GS-1 from 0; first maximum wins).  Every centroid row
// read from shared memory (`cbg`, [C][GS]) feeds four dot products.
template <int GS>
__device__ __forceinline__ void search_four_tokens(const float (&k)[4][GS], const float* __restrict__ cbg, int C,
                                                   float (&nsq)[4], int (&code)[4]) {
#pragma unroll
  for (int h = 0; h < 4; ++h) nsq[h] = 0.f;
#pragma unroll
  for (int d = 0; d < GS; ++d)
#pragma unroll
    for (int h = 0; h < 4; ++h) nsq[h] = __fmaf_rn(k[h][d], k[h][d], nsq[h]);
  float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int h = 0; h < 4; ++h) code[h] = 0;
  SPHKV_UNROLL_SEARCH
  for (int c = 0; c < C; ++c) {
    const float4* row = reinterpret_cast<const float4*>(cbg + c * GS);
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < GS / 4; ++i) {
      const float4 v = row[i];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        sacc[h] = __fmaf_rn(k[h][4 * i], v.x, sacc[h]);
        sacc[h] = __fmaf_rn(k[h][4 * i + 1], v.y, sacc[h]);
        sacc[h] = __fmaf_rn(k[h][4 * i + 2], v.z, sacc[h]);
        sacc[h] = __fmaf_rn(k[h][4 * i + 3], v.w, sacc[h]);
      }
    }
#pragma unroll
    for (int h = 0; h < 4; ++h)
      if (sacc[h] > best[h]) { best[h] = sacc[h]; code[h] = c; }
  }
}

// The codebook of one (KV head, tier slot), [G][C][GS] packed, global -> shared memory.
template <int GS>
__device__ __forceinline__ void stage_slot_codebook(const sphkv_encode_params& p, int head, int slot, float* cb_s) {
  const int bits = p.tiers.bits[slot], G = p.dh / GS;
  const float4* src = reinterpret_cast<const float4*>(
      p.codebooks + ((int64_t)(head * p.tiers.n_slots + slot) * p.tiers.G_max) * p.tiers.C_max * p.tiers.g_max);
  float4* dst = reinterpret_cast<float4*>(cb_s);
  constexpr int Q4 = GS / 4;
  const int total = (G << bits) * Q4;
  const int row_stride4 = p.tiers.g_max >> 2;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int q4 = i % Q4, row = i / Q4;
    const int c = row & ((1 << bits) - 1), gam = row >> bits;
    dst[i] = __ldg(src + ((int64_t)gam * p.tiers.C_max + c) * row_stride4 + q4);
  }
}

// Everything in one kernel (the route without scratch): search, page images and V pages per bundle.
// With scratch the work is split instead: search_bundles_kernel writes radius + centroid index per
// (page slot, group) and assemble_pages_kernel builds the pages, so the FMA-bound search runs without
// the barriers and small dependent loads of the page bookkeeping.
template <int GS>
__global__ void __launch_bounds__(kEncThreads) encode_bundle_kernel(const EncodeArgs a) {
  const sphkv_encode_params& p = a.p;
  extern __shared__ __align__(16) uint8_t smem[];
  const int N = p.page_size, dh = p.dh;
  constexpr int TB = 128;                   // token slots per bundle
  const int ppb = TB / N;                   // pages per bundle (page_size <= 128)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = dh / GS, g_shift = 31 - __clz(G);
  const int n_shift = 31 - __clz(N);  // page_size is a power of two
  const int rb = p.radius_fmt == SPHKV_RADIUS_F16 ? 2 : 1;
  const int C_cap = p.tiers.C_max;

  float* cb_s = reinterpret_cast<float*>(smem);                       // [G][C][GS]
  float* r_s = cb_s + G * C_cap * GS;                                  // [TB][G]
  float* scale_s = r_s + TB * G;                                       // [8][8]
  int* count_s = reinterpret_cast<int*>(scale_s + 64);                 // [8]
  int* page_s = count_s + 8;                                           // [8]
  int* poff_s = page_s + 8;                                            // [8] byte offset of each page
  uint8_t* th_s = reinterpret_cast<uint8_t*>(poff_s + 8);              // [TB][G]
  uint8_t* img = th_s + TB * G;                                        // page images, 16-aligned
  img = reinterpret_cast<uint8_t*>(((uintptr_t)img + 15) & ~(uintptr_t)15);

  int loaded_key = -1;
  const int b_first = blockIdx.x * a.bundles_per_cta;
  const int b_last = min(p.n_bundles, b_first + a.bundles_per_cta);
  for (int bi = b_first; bi < b_last; ++bi) {
    const int32_t* bundle = p.bundles + 8 * (int64_t)bi;
    __syncthreads();  // previous bundle is done with shared memory
    // ---- pages of the bundle and their valid-token counts (valid slots form a prefix) ------
    {  // 8 warps, up to 8 pages
      int page = -1, cnt = 0;
      if (warp < ppb) page = bundle[warp];
      if (page >= 0) {
        const int32_t* si = p.src_index + (int64_t)page * N;
        for (int t0 = 0; t0 < N; t0 += 32) {
          const bool ok = (t0 + lane < N) && si[t0 + lane] >= 0;
          cnt += __popc(__ballot_sync(0xffffffffu, ok));
        }
      }
      if (lane == 0) {
        count_s[warp] = cnt;
        page_s[warp] = page;
        poff_s[warp] = page >= 0 ? p.ptable[3 * (int64_t)page] : 0;
      }
    }
    __syncthreads();
    int first = -1;
    for (int q = 0; q < ppb; ++q)
      if (first < 0 && page_s[q] >= 0) first = page_s[q];
    if (first < 0) continue;
    const int head = p.page_head[first], slot = p.page_slot[first];
    if (p.tiers.g[slot] != GS) continue;  // the launch for the other group size takes this bundle
    const int bits = p.tiers.bits[slot], C = 1 << bits;
    const int img_stride = ((8 + 4 * G + (N * G * bits + 7) / 8 + N * G * rb) + 15) & ~15;

    // ---- codebook of (head, slot) -> shared memory, 128-bit copies ---------------------------
    if (head * p.tiers.n_slots + slot != loaded_key) {
      stage_slot_codebook<GS>(p, head, slot, cb_s);
      loaded_key = head * p.tiers.n_slots + slot;
      __syncthreads();
    }

    // ---- radius + nearest centroid: warp = group, lane = token slots lane + 32 h, h < 4 ----
    if (warp < G) {
      const float* cbg = cb_s + (warp << bits) * GS;
      float k[4][GS];
      bool have[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const int ts = lane + 32 * h;  // token slot in bundle
        const int q = ts >> n_shift, tin = ts & (N - 1);
        const int page = page_s[q];
        int64_t row = -1;
        if (page >= 0) row = p.src_index[(int64_t)page * N + tin];
        have[h] = row >= 0;
        if (have[h]) {
          load_group<GS>(p.k_src, p.k_dtype,
                         row * p.k_row_stride + (int64_t)head * p.k_head_stride + warp * GS, k[h]);
        } else {
#pragma unroll
          for (int i = 0; i < GS; ++i) k[h][i] = 0.f;
        }
      }
      float nsq[4];
      int code[4];
      search_four_tokens<GS>(k, cbg, C, nsq, code);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const int ts = lane + 32 * h;
        const float rv = have[h] ? __fsqrt_rn(nsq[h]) : 0.f;
        r_s[ts * G + warp] = rv;
        th_s[ts * G + warp] = (uint8_t)code[h];
      }
    }
    __syncthreads();

    // ---- per-page, per-group scale = max radius over the page's tokens ----------------------
    if (warp < ppb) {
      const int cnt = count_s[warp];
      const int tbase = warp * N;
      const int gq = lane & 7, tq = lane >> 3;
      float mx = 0.f;
      if (gq < G)
        for (int t = tq; t < cnt; t += 4) mx = fmaxf(mx, r_s[(tbase + t) * G + gq]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      if (lane < 8) scale_s[warp * 8 + lane] = mx;
    }
    __syncthreads();

    // ---- page images: header, scales, packed theta words ---------------------------------------
    // Every loop below runs over the whole bundle (all pages at once), so the CTA's threads share
    // the work of the 128 / page_size pages evenly instead of a fraction of them looping per page.
    const int hdr = 8 + 4 * G;
    if ((int)threadIdx.x < 2 * ppb) {
      const int q = threadIdx.x >> 1, cnt = count_s[q];
      if (cnt > 0) {
        uint32_t w = 0;
        if ((threadIdx.x & 1) == 0)
          w = (uint32_t)(p.tiers.tier_id[slot] & 0xFF) | ((uint32_t)(cnt & 0xFF) << 8) |
              ((uint32_t)(p.radius_fmt & 0xFF) << 16);
        reinterpret_cast<uint32_t*>(img + q * img_stride)[threadIdx.x & 1] = w;
      }
    }
    if ((int)threadIdx.x < 8 * ppb) {
      const int q = threadIdx.x >> 3, gq = threadIdx.x & 7;
      if (gq < G && count_s[q] > 0)
        reinterpret_cast<float*>(img + q * img_stride + 8)[gq] = scale_s[q * 8 + gq];
    }
    {
      const int max_words = ((((N * G * bits + 7) >> 3) + 3) >> 2);
      for (int it = threadIdx.x; it < ppb * max_words; it += blockDim.x) {
        const int q = it / max_words, w = it - q * max_words;
        const int nvals = count_s[q] * G;
        const int th_words = ((((nvals * bits + 7) >> 3) + 3) >> 2);
        if (w >= th_words) continue;
        const int bit0 = w * 32;
        int i = bit0 / bits;  // first value overlapping this word
        uint32_t acc = 0;
        for (; i < nvals && i * bits < bit0 + 32; ++i) {
          const uint32_t v = th_s[q * N * G + i];
          const int sh = i * bits - bit0;
          acc |= sh >= 0 ? (v << sh) : (v >> (-sh));
        }
        reinterpret_cast<uint32_t*>(img + q * img_stride + hdr)[w] = acc;
      }
    }
    __syncthreads();
    // ---- radii (may overlay the zero tail of the last theta word) ----------------------------
    for (int i = threadIdx.x; i < TB * G; i += blockDim.x) {
      const int ts = i >> g_shift, gq = i & (G - 1);
      const int q = ts >> n_shift, tin = ts & (N - 1);
      const int cnt = count_s[q];
      if (tin >= cnt) continue;
      const float rr = r_s[i];
      if (rb == 1) {
        const float safe = fmaxf(scale_s[q * 8 + gq], 1e-8f);
        float qv = rintf(__fmul_rn(__fdiv_rn(rr, safe), 127.0f));
        qv = fminf(fmaxf(qv, -127.f), 127.f);
        img[q * img_stride + hdr + ((cnt * G * bits + 7) >> 3) + tin * G + gq] = (uint8_t)(int8_t)(int)qv;
      } else {
        // stage the half's bit pattern as a 32-bit word over the radius slot (same thread
        // read it above); the bytes are laid into the page image after the barrier
        unsigned short hv;
        asm volatile("cvt.rn.f16.f32 %0, %1;" : "=h"(hv) : "f"(rr));
        reinterpret_cast<uint32_t*>(r_s)[i] = (uint32_t)hv;
      }
    }
    if (rb == 2) {
      __syncthreads();
      const uint8_t* hb = reinterpret_cast<const uint8_t*>(r_s);
      for (int b2 = threadIdx.x; b2 < 2 * TB * G; b2 += blockDim.x) {
        const int i = b2 >> 1;
        const int ts = i >> g_shift, gq = i & (G - 1);
        const int q = ts >> n_shift, tin = ts & (N - 1);
        const int cnt = count_s[q];
        if (tin >= cnt) continue;
        img[q * img_stride + hdr + ((cnt * G * bits + 7) >> 3) + 2 * (tin * G + gq) + (b2 & 1)] = hb[i * 4 + (b2 & 1)];
      }
    }
    __syncthreads();
    // ---- copy page images out -------------------------------------------------------------------
    {
      const int max_img_words = img_stride >> 2;
      for (int it = threadIdx.x; it < ppb * max_img_words; it += blockDim.x) {
        const int q = it / max_img_words, w = it - q * max_img_words;
        const int cnt = count_s[q];
        if (cnt == 0) continue;
        const int bytes = hdr + ((cnt * G * bits + 7) >> 3) + cnt * G * rb;
        if (w < (bytes >> 2))
          reinterpret_cast<uint32_t*>(p.k_pages + poff_s[q])[w] =
              reinterpret_cast<const uint32_t*>(img + q * img_stride)[w];
      }
      if ((int)threadIdx.x < 4 * ppb) {
        const int q = threadIdx.x >> 2, t = threadIdx.x & 3;
        const int cnt = count_s[q];
        if (cnt > 0) {
          const int bytes = hdr + ((cnt * G * bits + 7) >> 3) + cnt * G * rb;
          if (t < (bytes & 3)) p.k_pages[poff_s[q] + (bytes & ~3) + t] = img[q * img_stride + (bytes & ~3) + t];
        }
      }
    }

    // ---- dense V pages (16-bit), empty slots zero-filled ----------------------------------------
    // One item = 8 elements (a 16-byte output chunk) of one token slot of the bundle.  A thread
    // takes four items per round: all row lookups first, then all loads, then all stores, so four
    // independent load chains are in flight instead of one.
    if (p.v_src != nullptr && p.v_pool != nullptr) {
      constexpr int kInFlight = 4;
      const int pr_shift = 31 - __clz(dh >> 3);  // 16-byte chunks per row (dh / 8, a power of two)
      const int items = TB << pr_shift;
      const bool same = p.v_src_dtype == p.v_pool_dtype;
      for (int i0 = threadIdx.x; i0 < items; i0 += kEncThreads * kInFlight) {
        int64_t off[kInFlight], dst[kInFlight];
        bool live[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          const int i = i0 + u * kEncThreads;
          const int ts = i >> pr_shift, d = (i & ((1 << pr_shift) - 1)) * 8;
          const int page = i < items ? page_s[ts >> n_shift] : -1;
          const int tin = ts & (N - 1);
          dst[u] = -1;
          off[u] = -1;
          if (page >= 0) {
            dst[u] = (((int64_t)page * N + tin) * dh + d) >> 3;
            const int64_t row = p.src_index[(int64_t)page * N + tin];
            if (row >= 0) off[u] = row * p.v_row_stride + (int64_t)head * p.v_head_stride + d;
          }
          live[u] = off[u] >= 0;
        }
        uint4 o[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          o[u] = live[u] ? load_v_chunk(p, same, off[u]) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
          if (dst[u] >= 0) reinterpret_cast<uint4*>(p.v_pool)[dst[u]] = o[u];
      }
    }
  }
}

// ---- search only (the split route) ---------------------------------------------------------
// Radius and nearest centroid of every token slot of every bundle, written to the scratch arrays
// r[(page * N + slot) * (dh / 16) + group] (f32) and theta[...] (u8).  Persistent: CTA c of n takes
// the chunks c, c + n, c + 2n, ... of `search_chunk` consecutive bundles (1 .. 8: consecutive bundles
// mostly share a codebook, and every CTA should still get several chunks; striding the chunks
// spreads the tiers, whose bundles differ fourfold in work, evenly over the CTAs); warp = group,
// lane = four token slots.  The only barrier is the codebook change between (head, tier) keys;
// otherwise a warp walks its bundles alone, and while it searches one bundle the page ids and
// source rows of the next are already loaded and its key rows are on their way to L2.
template <int GS>
__global__ void __launch_bounds__(kEncThreads, GS == 16 ? 2 : 1) search_bundles_kernel(const EncodeArgs a) {
  const sphkv_encode_params& p = a.p;
  extern __shared__ __align__(16) uint8_t smem[];
  float* cb_s = reinterpret_cast<float*>(smem);  // [G][C][GS] of the current (head, tier slot)
  const int N = p.page_size, dh = p.dh;
  const int ppb = 128 / N, n_shift = 31 - __clz(N);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = dh / GS, GST = dh >> 4;
  const int esize = p.k_dtype == SPHKV_F32 ? 4 : 2;
  const int chunk_len = a.search_chunk;
  float* scr_r = reinterpret_cast<float*>(p.scratch);
  uint8_t* scr_t = reinterpret_cast<uint8_t*>(p.scratch) + (int64_t)p.n_pages * N * GST * 4;
  // page and source row of this lane's four token slots of bundle bi
  auto lookup = [&](int64_t bi, int (&pg)[4], int (&row)[4]) {
    const int32_t* bundle = p.bundles + 8 * bi;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int ts = lane + 32 * h;
      pg[h] = bundle[ts >> n_shift];
      row[h] = pg[h] >= 0 ? p.src_index[(int64_t)pg[h] * N + (ts & (N - 1))] : -1;
    }
  };
  int loaded_key = -1;
  for (int64_t chunk = blockIdx.x; chunk * chunk_len < p.n_bundles; chunk += gridDim.x) {
    // lane q < chunk_len looks at bundle q of the chunk: which (head, tier slot), and is it of this
    // launch's group size?  One pair of dependent loads per chunk; bundles of the other group size
    // (the other launch takes them) cost nothing more.
    int my_head = -1, my_slot = 0;
    if (lane < chunk_len && chunk * chunk_len + lane < p.n_bundles) {
      const int32_t* bundle = p.bundles + 8 * (chunk * chunk_len + lane);
      int first = -1;
      for (int q = 0; q < ppb; ++q) {
        const int pq = bundle[q];
        if (first < 0 && pq >= 0) first = pq;
      }
      if (first >= 0) {
        my_head = p.page_head[first];
        my_slot = p.page_slot[first];
      }
    }
    unsigned todo = __ballot_sync(0xffffffffu, my_head >= 0 && p.tiers.g[my_slot] == GS);  // same in every warp
    int pg_n[4], row_n[4];
    if (todo) lookup(chunk * chunk_len + (__ffs(todo) - 1), pg_n, row_n);
    while (todo) {
      const int q = __ffs(todo) - 1;
      todo &= todo - 1;
      const int head = __shfl_sync(0xffffffffu, my_head, q), slot = __shfl_sync(0xffffffffu, my_slot, q);
      int pg[4], row[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) { pg[h] = pg_n[h]; row[h] = row_n[h]; }
      int head_n = -1;
      if (todo) {  // the next bundle of the chunk: its rows load while this one is searched
        const int qn = __ffs(todo) - 1;
        head_n = __shfl_sync(0xffffffffu, my_head, qn);
        lookup(chunk * chunk_len + qn, pg_n, row_n);
      }
      if (head * p.tiers.n_slots + slot != loaded_key) {
        __syncthreads();  // every warp is done with the previous codebook
        stage_slot_codebook<GS>(p, head, slot, cb_s);
        loaded_key = head * p.tiers.n_slots + slot;
        __syncthreads();
      }
      if (warp >= G) continue;
      if (head_n >= 0) {
#pragma unroll
        for (int h = 0; h < 4; ++h)
          if (row_n[h] >= 0)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(
                reinterpret_cast<const char*>(p.k_src) +
                ((int64_t)row_n[h] * p.k_row_stride + (int64_t)head_n * p.k_head_stride + warp * GS) * esize));
      }
      const int bits = p.tiers.bits[slot];
      float k[4][GS];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        if (row[h] >= 0) {
          load_group<GS>(p.k_src, p.k_dtype,
                         (int64_t)row[h] * p.k_row_stride + (int64_t)head * p.k_head_stride + warp * GS, k[h]);
        } else {
#pragma unroll
          for (int i = 0; i < GS; ++i) k[h][i] = 0.f;
        }
      }
      float nsq[4];
      int code[4];
      search_four_tokens<GS>(k, cb_s + (warp << bits) * GS, 1 << bits, nsq, code);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        if (pg[h] < 0) continue;
        const int64_t si = ((int64_t)pg[h] * N + ((lane + 32 * h) & (N - 1))) * GST + warp;
        scr_r[si] = row[h] >= 0 ? __fsqrt_rn(nsq[h]) : 0.f;
        scr_t[si] = (uint8_t)code[h];
      }
    }
  }
}

// ---- page assembly, one warp per page -----------------------------------------------------
// Builds page images from per-(token, group) radii and centroid indices that already exist:
// SRC 2 = the scratch arrays the search launch wrote ([(page * N + slot) * (dh / 16) + group]),
// SRC 3 = a per-token code cache (sphkv_encode_codes) gathered through src_index, i.e. re-paging
// after a tier change without touching the dense keys.  A warp owns a page from the first
// lookup to the last byte, so there is no CTA barrier and the only dependent global loads are
// page index -> src_index row -> code; with 64 warps per SM thousands of pages are in flight.
// Per-warp shared memory: rows i32[N] | r f32[N*G] | scale f32[8] | theta u8[N*G] | page image.
template <int SRC>
__global__ void __launch_bounds__(kEncThreads) assemble_pages_kernel(const EncodeArgs a) {
  const sphkv_encode_params& p = a.p;
  extern __shared__ __align__(16) uint8_t smem[];
  const int N = p.page_size, dh = p.dh, GST = dh >> 4;
  const int ppb_shift = __clz(N) - 24;  // log2 of the 128 / N pages per bundle (N is 16 .. 128)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* mine = smem + (size_t)warp * a.warp_smem_bytes;
  int* rows_w = reinterpret_cast<int*>(mine);
  float* r_w = reinterpret_cast<float*>(rows_w + N);
  float* scale_w = r_w + N * GST;
  uint8_t* th_w = reinterpret_cast<uint8_t*>(scale_w + 8);
  uint8_t* img = th_w + N * GST;  // 16-byte aligned: every term above is a multiple of 16
  const float* scr_r = reinterpret_cast<const float*>(p.scratch);
  const uint8_t* scr_t = reinterpret_cast<const uint8_t*>(p.scratch) + (int64_t)p.n_pages * N * GST * 4;
  const int rb = p.radius_fmt == SPHKV_RADIUS_F16 ? 2 : 1;
  const int64_t items = (int64_t)p.n_bundles << ppb_shift;
  for (int64_t it = (int64_t)blockIdx.x * (kEncThreads / 32) + warp; it < items; it += (int64_t)gridDim.x * (kEncThreads / 32)) {
    const int page = p.bundles[8 * (it >> ppb_shift) + (it & ((1 << ppb_shift) - 1))];
    if (page < 0) continue;
    const int head = p.page_head[page], slot = p.page_slot[page];
    const int64_t poff = p.ptable[3 * (int64_t)page];
    const int gs = p.tiers.g[slot], bits = p.tiers.bits[slot];
    const int G = dh / gs, g_shift = 31 - __clz(G);
    const float* code_r = SRC == 3 ? p.code_r[slot] + (int64_t)head * p.code_rows * G : nullptr;
    const uint8_t* code_t = SRC == 3 ? p.code_theta[slot] + (int64_t)head * p.code_rows * G : nullptr;
    __syncwarp();  // the previous page's image has been copied out
    // ---- source rows and the valid-token count (valid slots form a prefix) -------------------
    int cnt = 0;
    for (int t0 = 0; t0 < N; t0 += 32) {
      const int row = t0 + lane < N ? p.src_index[(int64_t)page * N + t0 + lane] : -1;
      if (t0 + lane < N) rows_w[t0 + lane] = row;
      cnt += __popc(__ballot_sync(0xffffffffu, row >= 0));
    }
    __syncwarp();
    // ---- radii and centroid indices of the page -----------------------------------------------
    for (int i = lane; i < N * G; i += 32) {
      const int tin = i >> g_shift, gq = i & (G - 1);
      float rv = 0.f;
      uint8_t tv = 0;
      if (SRC == 2) {
        const int64_t si = ((int64_t)page * N + tin) * GST + gq;
        rv = scr_r[si];
        tv = scr_t[si];
      } else {
        const int row = rows_w[tin];
        if (row >= 0) {
          rv = code_r[(int64_t)row * G + gq];
          tv = code_t[(int64_t)row * G + gq];
        }
      }
      r_w[i] = rv;
      th_w[i] = tv;
    }
    __syncwarp();
    // ---- per-group scale = max radius over the page's tokens ----------------------------------
    {
      const int gq = lane & 7, tq = lane >> 3;
      float mx = 0.f;
      if (gq < G)
        for (int t = tq; t < cnt; t += 4) mx = fmaxf(mx, r_w[t * G + gq]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      if (lane < 8) scale_w[lane] = mx;
    }
    __syncwarp();
    if (cnt > 0) {
      // ---- header, scales, LSB-first theta words ----------------------------------------------
      const int hdr = 8 + 4 * G;
      const int nvals = cnt * G;
      const int th_bytes = (nvals * bits + 7) >> 3;
      const int th_words = (th_bytes + 3) >> 2;
      if (lane < 2)
        reinterpret_cast<uint32_t*>(img)[lane] =
            lane == 0 ? (uint32_t)(p.tiers.tier_id[slot] & 0xFF) | ((uint32_t)(cnt & 0xFF) << 8) |
                            ((uint32_t)(p.radius_fmt & 0xFF) << 16)
                      : 0u;
      if (lane < G) reinterpret_cast<float*>(img + 8)[lane] = scale_w[lane];
      for (int w = lane; w < th_words; w += 32) {
        const int bit0 = w * 32;
        const int i0 = bit0 / bits;                             // first value overlapping this word
        const int i1 = min(nvals, (bit0 + 31) / bits + 1);      // one past the last
        // values enter a 64-bit window that starts 8 bits below the word, so a value that begins
        // in the previous word (bits <= 8) needs no right shift
        int sh = i0 * bits - bit0 + 8;
        unsigned long long acc = 0;
        for (int i = i0; i < i1; ++i, sh += bits) acc |= (unsigned long long)th_w[i] << sh;
        reinterpret_cast<uint32_t*>(img + hdr)[w] = (uint32_t)(acc >> 8);
      }
      __syncwarp();
      // ---- radii (may overlay the zero tail of the last theta word) ---------------------------
      uint8_t* rad = img + hdr + th_bytes;
      for (int i = lane; i < nvals; i += 32) {
        const float rr = r_w[i];
        if (rb == 1) {
          const float safe = fmaxf(scale_w[i & (G - 1)], 1e-8f);
          float qv = rintf(__fmul_rn(__fdiv_rn(rr, safe), 127.0f));
          qv = fminf(fmaxf(qv, -127.f), 127.f);
          rad[i] = (uint8_t)(int8_t)(int)qv;
        } else {
          // the half's bit pattern goes over the radius slot as a 32-bit word (this lane read it
          // just above); its two bytes are laid into the image below
          reinterpret_cast<uint32_t*>(r_w)[i] = (uint32_t)__half_as_ushort(__float2half_rn(rr));
        }
      }
      __syncwarp();
      if (rb == 2) {
        const uint8_t* hb = reinterpret_cast<const uint8_t*>(r_w);
        for (int b2 = lane; b2 < 2 * nvals; b2 += 32) rad[b2] = hb[(b2 >> 1) * 4 + (b2 & 1)];
        __syncwarp();
      }
      // ---- copy the image out ----------------------------------------------------------------
      const int bytes = hdr + th_bytes + nvals * rb;
      for (int w = lane; w < (bytes >> 2); w += 32)
        reinterpret_cast<uint32_t*>(p.k_pages + poff)[w] = reinterpret_cast<const uint32_t*>(img)[w];
      if (lane < (bytes & 3)) p.k_pages[poff + (bytes & ~3) + lane] = img[(bytes & ~3) + lane];
    }
    // ---- dense V page (16-bit), empty slots zero-filled ---------------------------------------
    if (p.v_src != nullptr && p.v_pool != nullptr) {
      const int pr_shift = 31 - __clz(dh >> 3);  // 16-byte chunks per row (dh / 8, a power of two)
      const bool same = p.v_src_dtype == p.v_pool_dtype;
      for (int i = lane; i < (N << pr_shift); i += 32) {
        const int tin = i >> pr_shift, d = (i & ((1 << pr_shift) - 1)) * 8;
        const int row = rows_w[tin];
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (row >= 0) o = load_v_chunk(p, same, (int64_t)row * p.v_row_stride + (int64_t)head * p.v_head_stride + d);
        reinterpret_cast<uint4*>(p.v_pool)[(((int64_t)page * N + tin) * dh + d) >> 3] = o;
      }
    }
  }
}

// ---- all-tier code cache ---------------------------------------------------------------------
// Radius and nearest centroid of every (token, KV head, group) for EVERY tier slot in one pass
// over the keys (the pre-encode of spherical_kv_pipeline.py:1535-1553, which calls
// _encode_keys_with_codebooks once per tier).  A thread holds four tokens' 32-dim slice; the two
// 16-dim halves serve the g = 16 tiers, the whole slice the g = 32 tiers, and the squared norm
// of the 32-dim group continues the fma chain of its first half, so every value equals what
// the per-tier encoder computes (same fixed order).  Output per slot s, head-major like the
// reference's per-(layer, head) cache: r[s][head][row][G_s] f32, theta[s][head][row][G_s] u8.
struct CodesArgs {
  const void* k_src;
  const float* codebooks;
  float* r_out[SPHKV_MAX_TIER_SLOTS];
  uint8_t* th_out[SPHKV_MAX_TIER_SLOTS];
  int64_t k_row_stride, k_head_stride, rows;
  int64_t n_units, units_per_head;  // unit = one CTA pass: (8 / (dh / 32)) * 32 * kCodeTok rows of one head
  int k_dtype, dh;
  int kbuf_off;  // byte offset of the staged row blocks (8 warps x 32 * kCodeTok rows x 128 B)
  int cb_off[SPHKV_MAX_TIER_SLOTS];  // float offset of each slot's staged codebook
  sphkv_tiers tiers;
};

// tokens per thread of the code-cache kernel
constexpr int kCodeTok = SPHKV_CODE_TOKENS;

template <int OFF, int GS>
__device__ __forceinline__ void search_slice(const float (&k)[kCodeTok][32], const float* __restrict__ cbg, int C,
                                             int (&code)[kCodeTok]) {
  float best[kCodeTok];
#pragma unroll
  for (int h = 0; h < kCodeTok; ++h) { best[h] = -INFINITY; code[h] = 0; }
  SPHKV_UNROLL_CODE_SEARCH
  for (int c = 0; c < C; ++c) {
    const float4* row = reinterpret_cast<const float4*>(cbg + c * GS);
    float sacc[kCodeTok];
#pragma unroll
    for (int h = 0; h < kCodeTok; ++h) sacc[h] = 0.f;
#pragma unroll
    for (int i = 0; i < GS / 4; ++i) {
      const float4 v = row[i];
#pragma unroll
      for (int h = 0; h < kCodeTok; ++h) {
        sacc[h] = __fmaf_rn(k[h][OFF + 4 * i], v.x, sacc[h]);
        sacc[h] = __fmaf_rn(k[h][OFF + 4 * i + 1], v.y, sacc[h]);
        sacc[h] = __fmaf_rn(k[h][OFF + 4 * i + 2], v.z, sacc[h]);
        sacc[h] = __fmaf_rn(k[h][OFF + 4 * i + 3], v.w, sacc[h]);
      }
    }
#pragma unroll
    for (int h = 0; h < kCodeTok; ++h)
      if (sacc[h] > best[h]) { best[h] = sacc[h]; code[h] = c; }
  }
}

// CTAs per SM of the code-cache kernel (2 tokens per thread fit 128 registers, 4 need 232)
constexpr int kCodeCtasPerSm = kCodeTok <= 2 ? 2 : 1;
#ifndef SPHKV_CODE_WARPS
#define SPHKV_CODE_WARPS 8
#endif
constexpr int kCodeThreads = SPHKV_CODE_WARPS * 32;  // a multiple of four warps: dh / 32 warps share a token set

// Persistent: the (head, row block) units are dealt out in contiguous runs, one run per resident
// CTA.  A CTA stages a head's codebooks when its run enters that head (once or twice per CTA) and
// has no other barrier, so the warps of an SM drift apart and one warp's key loads hide under the
// others' searches.  STAGED: a warp's next row block travels global -> shared memory by 16-byte
// asynchronous copies (eight lanes per 128-byte row slice, so every sector is used whole) while
// the current block is searched; the chunk index is XOR-ed with the row so that both the copies
// and the later one-row-per-lane 128-bit reads touch every bank once.  Not STAGED (slices not
// 16-byte aligned, or no room beside the codebooks): each lane loads its own rows and asks L2
// for the next block's rows a block ahead.
template <bool STAGED>
__global__ void __launch_bounds__(kCodeThreads, kCodeCtasPerSm) encode_codes_kernel(const CodesArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* cb_s = reinterpret_cast<float*>(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G32 = a.dh >> 5;                  // 32-dim groups per head: 2 or 4
  const int grp = warp % G32, set = warp / G32;
  const int sets = (kCodeThreads / 32) / G32;  // token sets of 32 * kCodeTok per CTA
  constexpr int kBlockRows = 32 * kCodeTok;
  const int esize = a.k_dtype == SPHKV_F32 ? 4 : 2;
  const int64_t u_lo = a.n_units * blockIdx.x / gridDim.x, u_hi = a.n_units * (blockIdx.x + 1) / gridDim.x;
  const bool k32 = a.k_dtype == SPHKV_F32;
  const uint32_t kbuf = smem_u32(smem + a.kbuf_off) + warp * (kBlockRows * 128);  // this warp's row block
  auto issue_block = [&](int64_t uu) {
    const int64_t hd = uu / a.units_per_head;
    const int64_t c0 = hd * a.k_head_stride + grp * 32;
    const int64_t r0 = ((uu - hd * a.units_per_head) * sets + set) * kBlockRows;
    // lane -> (row lane / CH, chunk lane % CH) of every group of 32 / CH rows; one pointer walks the rows
    const int esz = k32 ? 4 : 2, ch_shift = k32 ? 3 : 2, rows_per_i = 32 >> ch_shift;
    const int r_l = lane >> ch_shift, c = lane & ((1 << ch_shift) - 1);
    // chunk swizzle: row & 7 for 128-byte rows, (row >> 1) & 3 for 64-byte rows.  Eight 64-byte rows
    // per step keep it fixed; four 128-byte rows per step flip bit 2 of it on odd steps.
    const int sw = k32 ? r_l : ((r_l >> 1) & 3);
    const char* src = reinterpret_cast<const char*>(a.k_src) + ((r0 + r_l) * a.k_row_stride + c0) * esz + c * 16;
    const int64_t src_step = a.k_row_stride * esz * rows_per_i;
    const uint32_t dst = kbuf + ((r_l << ch_shift) + (c ^ sw)) * 16;
    const uint32_t dst_odd = k32 ? kbuf + ((r_l << ch_shift) + (c ^ sw ^ 4)) * 16 : dst;
    const int64_t left = a.rows - r0 - r_l;  // rows of the block at or below this lane's first one
    if (left >= kBlockRows) {
#pragma unroll
      for (int i = 0; i < kBlockRows / 4; ++i) {
        if (i < kBlockRows / rows_per_i) cp_async_16(((i & 1) ? dst_odd : dst) + i * 512, src + i * src_step);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kBlockRows / 4; ++i) {
        if (i < kBlockRows / rows_per_i) {
          const bool in = (int64_t)i * rows_per_i < left;
          cp_async_16_zfill(((i & 1) ? dst_odd : dst) + i * 512, in ? src + i * src_step : reinterpret_cast<const char*>(a.k_src), in ? 16 : 0);
        }
      }
    }
    cp_async_commit();
  };
  if (STAGED && u_lo < u_hi) issue_block(u_lo);
  int head = -1;
  for (int64_t u = u_lo; u < u_hi; ++u) {
    const int u_head = (int)(u / a.units_per_head);
    if (u_head != head) {
      // stage every slot's codebook of this head: [G_s][C_s][g_s] packed
      if (head >= 0) __syncthreads();
      head = u_head;
      for (int s = 0; s < a.tiers.n_slots; ++s) {
        const int gs = a.tiers.g[s], bits = a.tiers.bits[s], G = a.dh / gs, q4n = gs >> 2;
        const float4* src = reinterpret_cast<const float4*>(
            a.codebooks + ((int64_t)(head * a.tiers.n_slots + s) * a.tiers.G_max) * a.tiers.C_max * a.tiers.g_max);
        float4* dst = reinterpret_cast<float4*>(cb_s + a.cb_off[s]);
        const int total = (G << bits) * q4n, row_stride4 = a.tiers.g_max >> 2;
        for (int i = threadIdx.x; i < total; i += blockDim.x) {
          const int q4 = i % q4n, row = i / q4n;
          dst[i] = __ldg(src + ((int64_t)(row >> bits) * a.tiers.C_max + (row & ((1 << bits) - 1))) * row_stride4 + q4);
        }
      }
      __syncthreads();
    }
    const int64_t col = (int64_t)head * a.k_head_stride + grp * 32;
    const int64_t row0 = ((u - (int64_t)head * a.units_per_head) * sets + set) * kBlockRows;
    if (!STAGED && u + 1 < u_hi) {
      const int64_t ncol = (u + 1) / a.units_per_head * a.k_head_stride + grp * 32;
      const int64_t nrow0 = ((u + 1) % a.units_per_head * sets + set) * kBlockRows;
#pragma unroll
      for (int h = 0; h < kCodeTok; ++h) {
        const int64_t nrow = nrow0 + lane + 32 * h;
        if (nrow < a.rows)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(a.k_src) + (nrow * a.k_row_stride + ncol) * esize));
      }
    }
    float k[kCodeTok][32];
    bool have[kCodeTok];
    if (STAGED) {
      cp_async_wait<0>();
      __syncwarp();
#pragma unroll
      for (int h = 0; h < kCodeTok; ++h) {
        have[h] = row0 + lane + 32 * h < a.rows;
        const int r = h * 32 + lane;
        if (k32) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 v = lds_f4(kbuf + r * 128 + ((c ^ (lane & 7)) << 4));
            k[h][4 * c] = v.x; k[h][4 * c + 1] = v.y; k[h][4 * c + 2] = v.z; k[h][4 * c + 3] = v.w;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float4 v = lds_f4(kbuf + r * 64 + ((c ^ ((lane >> 1) & 3)) << 4));
            const uint32_t w[4] = {__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w)};
#pragma unroll
            for (int e = 0; e < 4; ++e) unpack16(w[e], a.k_dtype, k[h][8 * c + 2 * e], k[h][8 * c + 2 * e + 1]);
          }
        }
      }
      __syncwarp();
      if (u + 1 < u_hi) issue_block(u + 1);
    } else
#pragma unroll
    for (int h = 0; h < kCodeTok; ++h) {
      const int64_t row = row0 + lane + 32 * h;
      have[h] = row < a.rows;
      if (have[h]) {
        load_group<32>(a.k_src, a.k_dtype, row * a.k_row_stride + col, k[h]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) k[h][i] = 0.f;
      }
    }
    float na[kCodeTok], nb[kCodeTok], nab[kCodeTok];
#pragma unroll
    for (int h = 0; h < kCodeTok; ++h) na[h] = nb[h] = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d)
#pragma unroll
      for (int h = 0; h < kCodeTok; ++h) {
        na[h] = __fmaf_rn(k[h][d], k[h][d], na[h]);
        nb[h] = __fmaf_rn(k[h][16 + d], k[h][16 + d], nb[h]);
      }
#pragma unroll
    for (int h = 0; h < kCodeTok; ++h) nab[h] = na[h];
#pragma unroll
    for (int d = 16; d < 32; ++d)
#pragma unroll
      for (int h = 0; h < kCodeTok; ++h) nab[h] = __fmaf_rn(k[h][d], k[h][d], nab[h]);

    for (int s = 0; s < a.tiers.n_slots; ++s) {
      if (a.r_out[s] == nullptr) continue;
      const int bits = a.tiers.bits[s], C = 1 << bits;
      if (a.tiers.g[s] == 16) {
        // both 16-dim halves of the slice, stored as one 8-byte radius pair and one 2-byte code pair
        const int G = a.dh >> 4;
        int code_a[kCodeTok], code_b[kCodeTok];
        search_slice<0, 16>(k, cb_s + a.cb_off[s] + ((2 * grp) << bits) * 16, C, code_a);
        search_slice<16, 16>(k, cb_s + a.cb_off[s] + ((2 * grp + 1) << bits) * 16, C, code_b);
#pragma unroll
        for (int h = 0; h < kCodeTok; ++h) {
          if (!have[h]) continue;
          const int64_t o = ((int64_t)head * a.rows + row0 + lane + 32 * h) * G + 2 * grp;
          *reinterpret_cast<float2*>(a.r_out[s] + o) = make_float2(__fsqrt_rn(na[h]), __fsqrt_rn(nb[h]));
          *reinterpret_cast<uint16_t*>(a.th_out[s] + o) = (uint16_t)(code_a[h] | (code_b[h] << 8));
        }
      } else {
        int code[kCodeTok];
        search_slice<0, 32>(k, cb_s + a.cb_off[s] + (grp << bits) * 32, C, code);
#pragma unroll
        for (int h = 0; h < kCodeTok; ++h) {
          if (!have[h]) continue;
          const int64_t o = ((int64_t)head * a.rows + row0 + lane + 32 * h) * G32 + grp;
          a.r_out[s][o] = __fsqrt_rn(nab[h]);
          a.th_out[s][o] = (uint8_t)code[h];
        }
      }
    }
  }
}

int validate_tiers(const sphkv_tiers& t, int dh);

}  // namespace sphkv

using namespace sphkv;

template <int GS>
static int launch_encode(const EncodeArgs& a, bool split, int smem_bytes, cudaStream_t st) {
  if (split) {
    // persistent: as many CTAs as are resident at once, each striding over chunks of bundles
    static SmemOptIn opt_in;
    const int cb_bytes = a.p.dh * a.p.tiers.C_max * 4;
    if (int rc = ensure_dynamic_smem(opt_in, (const void*)search_bundles_kernel<GS>, cb_bytes, "encode search")) return rc;
    const int resident = sm_count_current_device() * (GS == 16 ? 2 : 1);
    EncodeArgs b = a;
    b.search_chunk = std::max(1, std::min(8, a.p.n_bundles / (resident * 4)));  // >= 4 chunks per CTA, <= 8 bundles each
    const int grid = std::max(1, std::min((a.p.n_bundles + b.search_chunk - 1) / b.search_chunk, resident));
    search_bundles_kernel<GS><<<grid, kEncThreads, cb_bytes, st>>>(b);
    return check_launch("search_bundles_kernel");
  }
  const int grid = (a.p.n_bundles + a.bundles_per_cta - 1) / a.bundles_per_cta;
  encode_bundle_kernel<GS><<<grid, kEncThreads, smem_bytes, st>>>(a);
  return check_launch("encode_bundle_kernel");
}

// One warp per page of the bundle list, every tier slot in the same launch.
static int launch_assemble(EncodeArgs& a, bool from_codes, cudaStream_t st) {
  const sphkv_encode_params& p = a.p;
  const int N = p.page_size, GST = p.dh >> 4;
  const int img = ((8 + 4 * GST + N * GST + N * GST * 2) + 15) & ~15;  // 8-bit codes, f16 radii: the largest image
  a.warp_smem_bytes = 4 * N + 4 * N * GST + 32 + N * GST + img;
  const int smem_bytes = a.warp_smem_bytes * (kEncThreads / 32);
  static SmemOptIn opt_in[2];
  const void* fn = from_codes ? (const void*)assemble_pages_kernel<3> : (const void*)assemble_pages_kernel<2>;
  if (int rc = ensure_dynamic_smem(opt_in[from_codes], fn, smem_bytes, "assemble_pages")) return rc;
  const int64_t items = (int64_t)p.n_bundles * (128 / N);
  const int64_t ctas = (items + kEncThreads / 32 - 1) / (kEncThreads / 32);
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(ctas, (int64_t)sm_count_current_device() * 8));
  if (from_codes)
    assemble_pages_kernel<3><<<grid, kEncThreads, smem_bytes, st>>>(a);
  else
    assemble_pages_kernel<2><<<grid, kEncThreads, smem_bytes, st>>>(a);
  return check_launch("assemble_pages_kernel");
}

extern "C" int64_t sphkv_encode_scratch_bytes(int32_t n_pages, int32_t page_size, int32_t dh) {
  if (n_pages <= 0 || page_size <= 0 || dh <= 0) return SPHKV_E_ARG;
  return ((int64_t)n_pages * page_size * (dh / 16) * 5 + 15) / 16 * 16;
}

static int encode_impl(const sphkv_encode_params* pp, void* stream, bool from_codes) {
  SPHKV_REQUIRE(pp != nullptr, SPHKV_E_ARG, "encode: params is NULL");
  const sphkv_encode_params& p = *pp;
  if (p.n_bundles == 0) return 0;
  SPHKV_REQUIRE(p.src_index && p.bundles && p.page_head && p.page_slot && p.ptable && p.k_pages,
                SPHKV_E_ARG, "encode: a required pointer is NULL");
  if (from_codes) {
    SPHKV_REQUIRE(p.code_rows > 0, SPHKV_E_ARG, "pages_from_codes: code_rows=%lld", (long long)p.code_rows);
    for (int s = 0; s < p.tiers.n_slots && s < SPHKV_MAX_TIER_SLOTS; ++s)
      SPHKV_REQUIRE(p.code_r[s] && p.code_theta[s], SPHKV_E_ARG,
                    "pages_from_codes: code cache of tier slot %d is NULL", s);
  } else {
    SPHKV_REQUIRE(p.k_src && p.codebooks, SPHKV_E_ARG, "encode: k_src / codebooks is NULL");
  }
  SPHKV_REQUIRE(p.n_bundles > 0 && p.n_pages > 0, SPHKV_E_ARG, "encode: n_bundles=%d n_pages=%d",
                p.n_bundles, p.n_pages);
  SPHKV_REQUIRE(p.dh == 64 || p.dh == 128, SPHKV_E_ARG, "encode: dh=%d (64 or 128)", p.dh);
  SPHKV_REQUIRE(p.page_size == 16 || p.page_size == 32 || p.page_size == 64 || p.page_size == 128,
                SPHKV_E_ARG, "encode: page_size=%d (16, 32, 64 or 128)", p.page_size);
  SPHKV_REQUIRE(p.k_dtype >= 0 && p.k_dtype <= 2 && p.v_src_dtype >= 0 && p.v_src_dtype <= 2,
                SPHKV_E_DTYPE, "encode: k_dtype=%d v_src_dtype=%d", p.k_dtype, p.v_src_dtype);
  SPHKV_REQUIRE(p.v_pool == nullptr || p.v_pool_dtype == SPHKV_F16 || p.v_pool_dtype == SPHKV_BF16,
                SPHKV_E_DTYPE, "encode: v_pool_dtype=%d", p.v_pool_dtype);
  SPHKV_REQUIRE(p.radius_fmt == SPHKV_RADIUS_I8 || p.radius_fmt == SPHKV_RADIUS_F16, SPHKV_E_ARG,
                "encode: radius_fmt=%d", p.radius_fmt);
  SPHKV_REQUIRE(((uintptr_t)p.k_pages & 3) == 0, SPHKV_E_ALIGN, "encode: k_pages needs 4 B alignment");
  if (int rc = validate_tiers(p.tiers, p.dh)) return rc;
  SPHKV_REQUIRE((from_codes || ((uintptr_t)p.codebooks & 15) == 0) && (p.tiers.g_max & 3) == 0 &&
                    ((uintptr_t)p.v_pool & 15) == 0,
                SPHKV_E_ALIGN, "encode: codebooks / v_pool need 16 B alignment, g_max a multiple of 4");
  // shared memory: codebook of the widest tier + staging + page images
  const int N = p.page_size, TB = 128, ppb = TB / N;
  int smem_bytes = 0;
  for (int s = 0; s < p.tiers.n_slots; ++s) {
    const int G = p.dh / p.tiers.g[s];
    const int img = ((8 + 4 * G + (N * G * p.tiers.bits[s] + 7) / 8 + N * G * 2) + 15) & ~15;
    const int need = p.dh * p.tiers.C_max * 4 + TB * G * 4 + 64 * 4 + 96 + TB * G + 16 + ppb * img;
    smem_bytes = need > smem_bytes ? need : smem_bytes;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  EncodeArgs a;
  a.p = p;
  {  // long runs per CTA amortise the codebook staging, but only once every SM has several CTAs
    int sms = sm_count_current_device();
    if (sms <= 0) sms = 148;
    int bpc = p.n_bundles / (sms * 8);
    a.bundles_per_cta = bpc < 1 ? 1 : (bpc > kMaxBundlesPerCta ? kMaxBundlesPerCta : bpc);
  }
  const int64_t scratch_need = sphkv_encode_scratch_bytes(p.n_pages, p.page_size, p.dh);
  const bool split = p.scratch != nullptr && p.scratch_bytes >= scratch_need &&
                     ((uintptr_t)p.scratch & 15) == 0;
  if (from_codes) return launch_assemble(a, true, st);
  {
    static SmemOptIn opt_in[2];
    const void* kernels[2] = {(const void*)encode_bundle_kernel<16>, (const void*)encode_bundle_kernel<32>};
    for (int i = 0; i < 2; ++i)
      if (int rc = ensure_dynamic_smem(opt_in[i], kernels[i], smem_bytes, "encode")) return rc;
  }
  // One search launch per group size present; each skips the bundles of the other size.
  bool any16 = false, any32 = false;
  for (int s = 0; s < p.tiers.n_slots; ++s) (p.tiers.g[s] == 16 ? any16 : any32) = true;
  if (any16) {
    if (int rc = launch_encode<16>(a, split, smem_bytes, st)) return rc;
  }
  if (any32) {
    if (int rc = launch_encode<32>(a, split, smem_bytes, st)) return rc;
  }
  return split ? launch_assemble(a, false, st) : 0;
}

extern "C" int sphkv_encode_pages(const sphkv_encode_params* p, void* stream) {
  return encode_impl(p, stream, false);
}

extern "C" int sphkv_pages_from_codes(const sphkv_encode_params* p, void* stream) {
  return encode_impl(p, stream, true);
}

extern "C" int sphkv_encode_codes(const void* k_src, int32_t k_dtype, int64_t k_row_stride,
                                  int64_t k_head_stride, int64_t rows, int32_t Hkv, int32_t dh,
                                  const float* codebooks, const sphkv_tiers* tiers, float* const* r_out,
                                  uint8_t* const* theta_out, void* stream) {
  SPHKV_REQUIRE(k_src && codebooks && tiers && r_out && theta_out, SPHKV_E_ARG, "encode_codes: NULL pointer");
  SPHKV_REQUIRE(rows >= 0 && Hkv > 0 && (dh == 64 || dh == 128) && k_dtype >= 0 && k_dtype <= 2, SPHKV_E_ARG,
                "encode_codes: rows=%lld Hkv=%d dh=%d k_dtype=%d", (long long)rows, Hkv, dh, k_dtype);
  if (int rc = validate_tiers(*tiers, dh)) return rc;
  SPHKV_REQUIRE(((uintptr_t)codebooks & 15) == 0 && (tiers->g_max & 3) == 0, SPHKV_E_ALIGN,
                "encode_codes: codebooks need 16 B alignment, g_max a multiple of 4");
  if (rows == 0) return 0;
  CodesArgs a;
  a.k_src = k_src; a.codebooks = codebooks;
  a.k_row_stride = k_row_stride; a.k_head_stride = k_head_stride; a.rows = rows;
  a.k_dtype = k_dtype; a.dh = dh; a.tiers = *tiers;
  int off = 0;
  bool any = false;
  for (int s = 0; s < SPHKV_MAX_TIER_SLOTS; ++s) {
    a.r_out[s] = s < tiers->n_slots ? r_out[s] : nullptr;
    a.th_out[s] = s < tiers->n_slots ? theta_out[s] : nullptr;
    a.cb_off[s] = off;
    if (s < tiers->n_slots) {
      SPHKV_REQUIRE((a.r_out[s] == nullptr) == (a.th_out[s] == nullptr), SPHKV_E_ARG,
                    "encode_codes: slot %d needs both r_out and theta_out (or neither)", s);
      any = any || a.r_out[s] != nullptr;
      SPHKV_REQUIRE((reinterpret_cast<uintptr_t>(a.r_out[s]) & 7) == 0 && (reinterpret_cast<uintptr_t>(a.th_out[s]) & 1) == 0,
                    SPHKV_E_ARG, "encode_codes: slot %d outputs must be 8-byte (r) and 2-byte (theta) aligned", s);
      off += dh << tiers->bits[s];  // G_s * C_s * g_s floats
    }
  }
  SPHKV_REQUIRE(any, SPHKV_E_ARG, "encode_codes: no output requested");
  SPHKV_REQUIRE(off * 4 <= 200 * 1024, SPHKV_E_LIMIT, "encode_codes: codebooks need %d B of shared memory", off * 4);
  // row blocks staged through shared memory when every 32-element slice starts on a 16-byte
  // boundary and the blocks fit beside the codebooks
  const int esz = k_dtype == SPHKV_F32 ? 4 : 2;
  const int kbuf_bytes = (kCodeThreads / 32) * 32 * kCodeTok * 128;
  const bool staged = (reinterpret_cast<uintptr_t>(k_src) & 15) == 0 && (k_row_stride * esz) % 16 == 0 &&
                      (k_head_stride * esz) % 16 == 0 && (off * 4 + kbuf_bytes) * kCodeCtasPerSm <= 220 * 1024;
  a.kbuf_off = off * 4;
  const int smem_bytes = off * 4 + (staged ? kbuf_bytes : 0);
  {
    static SmemOptIn opt_in[2];
    const void* fn = staged ? (const void*)encode_codes_kernel<true> : (const void*)encode_codes_kernel<false>;
    if (int rc = ensure_dynamic_smem(opt_in[staged], fn, smem_bytes, "encode_codes")) return rc;
  }
  const int per_cta = (kCodeThreads / 32) / (dh >> 5) * 32 * kCodeTok;  // rows per CTA and pass
  a.units_per_head = (rows + per_cta - 1) / per_cta;
  a.n_units = a.units_per_head * Hkv;
  const int64_t resident = (int64_t)sm_count_current_device() * kCodeCtasPerSm;  // CTAs that fit at once
  const dim3 grid((unsigned)std::max<int64_t>(1, std::min(a.n_units, resident)));
  if (staged)
    encode_codes_kernel<true><<<grid, kCodeThreads, smem_bytes, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  else
    encode_codes_kernel<false><<<grid, kCodeThreads, smem_bytes, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("encode_codes_kernel");
}
