// Spherical encode + page build.
//
// One CTA encodes a bundle of 64 token slots (64/page_size pages, or 64-token chunks of
// one larger page) that share a (KV head, tier slot): warp = group, lane = token.  Per
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
#include "common.cuh"

namespace sphkv {

struct EncodeArgs {
  sphkv_encode_params p;
};

constexpr int kEncThreads = 256;

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
      for (int e = 0; e < 4; ++e) {
        if (dtype == SPHKV_BF16) {
          k[8 * i + 2 * e] = __uint_as_float(w[e] << 16);
          k[8 * i + 2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
        } else {
          const __half2 h = *reinterpret_cast<const __half2*>(&w[e]);
          k[8 * i + 2 * e] = __low2float(h);
          k[8 * i + 2 * e + 1] = __high2float(h);
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < GS; ++i) k[i] = load_as_float(base, dtype, off + i);
  }
}

template <int GS>
__global__ void __launch_bounds__(kEncThreads) encode_bundle_kernel(const EncodeArgs a) {
  const sphkv_encode_params& p = a.p;
  extern __shared__ __align__(16) uint8_t smem[];
  const int N = p.page_size, dh = p.dh;
  const int TB = N > 64 ? N : 64;           // token slots per bundle
  const int n_chunks = TB / 64;
  const int ppb = N >= 64 ? 1 : 64 / N;     // pages per bundle
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int32_t* bundle = p.bundles + 4 * (int64_t)blockIdx.x;
  int first = -1;
  for (int q = 0; q < ppb; ++q)
    if (first < 0 && bundle[q] >= 0) first = bundle[q];
  if (first < 0) return;
  const int head = p.page_head[first], slot = p.page_slot[first];
  if (p.tiers.g[slot] != GS) return;  // the launch for the other group size takes this bundle
  const int bits = p.tiers.bits[slot], C = 1 << bits, G = dh / GS;
  const int rb = p.radius_fmt == SPHKV_RADIUS_F16 ? 2 : 1;

  float* cb_s = reinterpret_cast<float*>(smem);                       // [G][C][GS]
  float* r_s = cb_s + G * C * GS;                                      // [TB][G]
  float* scale_s = r_s + TB * G;                                       // [4][8]
  int* count_s = reinterpret_cast<int*>(scale_s + 32);                 // [4]
  uint8_t* th_s = reinterpret_cast<uint8_t*>(count_s + 4);             // [TB][G]
  uint8_t* img = th_s + TB * G;                                        // page images, 16-aligned
  img = reinterpret_cast<uint8_t*>(((uintptr_t)img + 15) & ~(uintptr_t)15);
  const int img_stride = ((8 + 4 * G + (N * G * bits + 7) / 8 + N * G * rb) + 15) & ~15;

  // ---- codebook of (head, slot) -> shared memory ---------------------------------------
  {
    const float* src =
        p.codebooks + ((int64_t)(head * p.tiers.n_slots + slot) * p.tiers.G_max) * p.tiers.C_max *
                          p.tiers.g_max;
    const int total = G * C * GS;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int d = i % GS, c = (i / GS) % C, gam = i / (GS * C);
      cb_s[i] = src[((int64_t)gam * p.tiers.C_max + c) * p.tiers.g_max + d];
    }
  }
  // ---- valid-token count per page (valid slots form a prefix) -----------------------------
  if (threadIdx.x < 4) {
    int cnt = 0;
    if (threadIdx.x < ppb && bundle[threadIdx.x] >= 0) {
      const int32_t* si = p.src_index + (int64_t)bundle[threadIdx.x] * N;
      while (cnt < N && si[cnt] >= 0) ++cnt;
    }
    count_s[threadIdx.x] = cnt;
  }
  __syncthreads();

  // ---- radius + nearest centroid: warp = group, lane = token slot (two per thread) -------
  if (warp < G) {
    const float* cbg = cb_s + warp * C * GS;
    for (int ch = 0; ch < n_chunks; ++ch) {
      float k0[GS], k1[GS];
      int tok[2];
      bool have[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int ts = ch * 64 + lane + 32 * h;  // token slot in bundle
        const int q = N >= 64 ? 0 : ts / N, tin = N >= 64 ? ts : ts % N;
        tok[h] = ts;
        const int page = bundle[q];
        int64_t row = -1;
        if (page >= 0) row = p.src_index[(int64_t)page * N + tin];
        have[h] = row >= 0;
        float (&kk)[GS] = h ? k1 : k0;
        if (have[h]) {
          load_group<GS>(p.k_src, p.k_dtype,
                         row * p.k_row_stride + (int64_t)head * p.k_head_stride + warp * GS, kk);
        } else {
#pragma unroll
          for (int i = 0; i < GS; ++i) kk[i] = 0.f;
        }
      }
      float n0 = 0.f, n1 = 0.f;
#pragma unroll
      for (int d = 0; d < GS; ++d) {
        n0 = __fmaf_rn(k0[d], k0[d], n0);
        n1 = __fmaf_rn(k1[d], k1[d], n1);
      }
      float best0 = -INFINITY, best1 = -INFINITY;
      int code0 = 0, code1 = 0;
      for (int c = 0; c < C; ++c) {
        const float4* row = reinterpret_cast<const float4*>(cbg + c * GS);
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int i = 0; i < GS / 4; ++i) {
          const float4 v = row[i];
          s0 = __fmaf_rn(k0[4 * i], v.x, s0); s1 = __fmaf_rn(k1[4 * i], v.x, s1);
          s0 = __fmaf_rn(k0[4 * i + 1], v.y, s0); s1 = __fmaf_rn(k1[4 * i + 1], v.y, s1);
          s0 = __fmaf_rn(k0[4 * i + 2], v.z, s0); s1 = __fmaf_rn(k1[4 * i + 2], v.z, s1);
          s0 = __fmaf_rn(k0[4 * i + 3], v.w, s0); s1 = __fmaf_rn(k1[4 * i + 3], v.w, s1);
        }
        if (s0 > best0) { best0 = s0; code0 = c; }
        if (s1 > best1) { best1 = s1; code1 = c; }
      }
      r_s[tok[0] * G + warp] = have[0] ? __fsqrt_rn(n0) : 0.f;
      r_s[tok[1] * G + warp] = have[1] ? __fsqrt_rn(n1) : 0.f;
      th_s[tok[0] * G + warp] = (uint8_t)code0;
      th_s[tok[1] * G + warp] = (uint8_t)code1;
    }
  }
  __syncthreads();

  // ---- per-page, per-group scale = max radius over the page's tokens ----------------------
  if (warp < ppb) {
    const int cnt = count_s[warp];
    const int tbase = N >= 64 ? 0 : warp * N;
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
  for (int q = 0; q < ppb; ++q) {
    const int cnt = count_s[q];
    if (cnt == 0) continue;
    uint8_t* im = img + q * img_stride;
    const int tbase = N >= 64 ? 0 : q * N;
    const int hdr = 8 + 4 * G;
    const int nvals = cnt * G;
    const int th_bytes = (nvals * bits + 7) >> 3;
    const int th_words = (th_bytes + 3) >> 2;
    if (threadIdx.x < 2) {
      uint32_t w = 0;
      if (threadIdx.x == 0)
        w = (uint32_t)(p.tiers.tier_id[slot] & 0xFF) | ((uint32_t)(cnt & 0xFF) << 8) |
            ((uint32_t)(p.radius_fmt & 0xFF) << 16);
      reinterpret_cast<uint32_t*>(im)[threadIdx.x] = w;
    }
    if (threadIdx.x < G) reinterpret_cast<float*>(im + 8)[threadIdx.x] = scale_s[q * 8 + threadIdx.x];
    for (int w = threadIdx.x; w < th_words; w += blockDim.x) {
      const int bit0 = w * 32;
      int i = bit0 / bits;  // first value overlapping this word
      uint32_t acc = 0;
      for (; i < nvals && i * bits < bit0 + 32; ++i) {
        const uint32_t v = th_s[tbase * G + i];
        const int sh = i * bits - bit0;
        acc |= sh >= 0 ? (v << sh) : (v >> (-sh));
      }
      reinterpret_cast<uint32_t*>(im + hdr)[w] = acc;
    }
  }
  __syncthreads();
  // ---- radii (may overlay the zero tail of the last theta word) ----------------------------
  for (int q = 0; q < ppb; ++q) {
    const int cnt = count_s[q];
    if (cnt == 0) continue;
    uint8_t* im = img + q * img_stride;
    const int tbase = N >= 64 ? 0 : q * N;
    const int roff = 8 + 4 * G + ((cnt * G * bits + 7) >> 3);
    for (int i = threadIdx.x; i < cnt * G; i += blockDim.x) {
      const int gq = i % G;
      const float rr = r_s[tbase * G + i];
      if (rb == 1) {
        const float safe = fmaxf(scale_s[q * 8 + gq], 1e-8f);
        float qv = rintf(__fmul_rn(__fdiv_rn(rr, safe), 127.0f));
        qv = fminf(fmaxf(qv, -127.f), 127.f);
        im[roff + i] = (uint8_t)(int8_t)(int)qv;
      } else {
        // stage the half's bit pattern as a 32-bit word over the radius slot (same thread
        // read it above); the bytes are laid into the page image after the barrier
        unsigned short hv;
        asm volatile("cvt.rn.f16.f32 %0, %1;" : "=h"(hv) : "f"(rr));
        reinterpret_cast<uint32_t*>(r_s)[tbase * G + i] = (uint32_t)hv;
      }
    }
  }
  if (rb == 2) {
    __syncthreads();
    for (int q = 0; q < ppb; ++q) {
      const int cnt = count_s[q];
      if (cnt == 0) continue;
      uint8_t* im = img + q * img_stride;
      const int tbase = N >= 64 ? 0 : q * N;
      const int roff = 8 + 4 * G + ((cnt * G * bits + 7) >> 3);
      const uint8_t* hb = reinterpret_cast<const uint8_t*>(r_s + tbase * G);
      for (int b = threadIdx.x; b < 2 * cnt * G; b += blockDim.x)
        im[roff + b] = hb[(b >> 1) * 4 + (b & 1)];
    }
  }
  __syncthreads();
  // ---- copy page images out -------------------------------------------------------------------
  for (int q = 0; q < ppb; ++q) {
    const int cnt = count_s[q];
    if (cnt == 0) continue;
    const int page = bundle[q];
    const uint8_t* im = img + q * img_stride;
    const int bytes = 8 + 4 * G + ((cnt * G * bits + 7) >> 3) + cnt * G * rb;
    uint8_t* dst = p.k_pages + p.ptable[3 * (int64_t)page];
    const int words = bytes >> 2;
    for (int w = threadIdx.x; w < words; w += blockDim.x)
      reinterpret_cast<uint32_t*>(dst)[w] = reinterpret_cast<const uint32_t*>(im)[w];
    if ((int)threadIdx.x < (bytes & 3)) dst[words * 4 + threadIdx.x] = im[words * 4 + threadIdx.x];
  }

  // ---- dense V pages (16-bit), empty slots zero-filled ------------------------------------------
  if (p.v_src != nullptr && p.v_pool != nullptr) {
    const int per_row = dh / 2;  // element pairs per row
    for (int q = 0; q < ppb; ++q) {
      const int page = bundle[q];
      if (page < 0) continue;
      for (int i = threadIdx.x; i < N * per_row; i += blockDim.x) {
        const int t = i / per_row, d = (i - t * per_row) * 2;
        const int64_t row = p.src_index[(int64_t)page * N + t];
        float v0 = 0.f, v1 = 0.f;
        if (row >= 0) {
          const int64_t off = row * p.v_row_stride + (int64_t)head * p.v_head_stride + d;
          v0 = load_as_float(p.v_src, p.v_src_dtype, off);
          v1 = load_as_float(p.v_src, p.v_src_dtype, off + 1);
        }
        uint32_t packed;
        if (p.v_pool_dtype == SPHKV_F16) {
          packed = pack_f16x2(v0, v1);
        } else {
          __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
          packed = *reinterpret_cast<uint32_t*>(&h);
        }
        reinterpret_cast<uint32_t*>(p.v_pool)[(((int64_t)page * N + t) * dh + d) >> 1] = packed;
      }
    }
  }
}

// ---- RoPE table ------------------------------------------------------------------------------
// row(pos)[(s*4 + j)*8 + e]     = cos(float(pos) * inv_freq[f]),
// row(pos)[(s*4 + j)*8 + 4 + e] = sin(...),  f = 16 s + 2 j + (e & 1) + 8 (e >> 1).
// The fp32 product is rounded first, as the HF rotary module does, then cos/sin are
// evaluated in double and rounded to fp32.
__global__ void rope_table_kernel(float* __restrict__ table, int max_pos, int dh,
                                  const float* __restrict__ inv_freq) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int half = dh / 2;
  if (i >= (int64_t)max_pos * half) return;
  const int pos = (int)(i / half), q = (int)(i - (int64_t)pos * half);
  const int e = q & 3, jj = (q >> 2) & 3, s = q >> 4;
  const int f = 16 * s + 2 * jj + (e & 1) + ((e >> 1) << 3);
  const float ang = __fmul_rn((float)pos, inv_freq[f]);
  double sn, cs;
  sincos((double)ang, &sn, &cs);
  float* row = table + (int64_t)pos * dh + (s * 4 + jj) * 8;
  row[e] = (float)cs;
  row[4 + e] = (float)sn;
}

int validate_tiers(const sphkv_tiers& t, int dh);

}  // namespace sphkv

using namespace sphkv;

extern "C" int sphkv_rope_table_build(float* table, int32_t max_pos, int32_t dh,
                                      const float* inv_freq, void* stream) {
  SPHKV_REQUIRE(table && inv_freq, SPHKV_E_ARG, "rope_table: NULL pointer");
  SPHKV_REQUIRE(max_pos > 0 && (dh == 64 || dh == 128), SPHKV_E_ARG, "rope_table: max_pos=%d dh=%d",
                max_pos, dh);
  SPHKV_REQUIRE(((uintptr_t)table & 15) == 0, SPHKV_E_ALIGN, "rope_table: table needs 16 B");
  const int64_t n = (int64_t)max_pos * (dh / 2);
  rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      table, max_pos, dh, inv_freq);
  return check_launch("rope_table_kernel");
}

extern "C" int sphkv_encode_pages(const sphkv_encode_params* pp, void* stream) {
  SPHKV_REQUIRE(pp != nullptr, SPHKV_E_ARG, "encode: params is NULL");
  const sphkv_encode_params& p = *pp;
  if (p.n_bundles == 0) return 0;
  SPHKV_REQUIRE(p.k_src && p.src_index && p.bundles && p.page_head && p.page_slot && p.ptable &&
                    p.codebooks && p.k_pages,
                SPHKV_E_ARG, "encode: a required pointer is NULL");
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
  SPHKV_REQUIRE(((uintptr_t)p.k_pages & 3) == 0 && ((uintptr_t)p.v_pool & 3) == 0, SPHKV_E_ALIGN,
                "encode: k_pages / v_pool need 4 B alignment");
  if (int rc = validate_tiers(p.tiers, p.dh)) return rc;
  // shared memory: largest codebook + staging + page images
  const int N = p.page_size, TB = N > 64 ? N : 64, ppb = N >= 64 ? 1 : 64 / N;
  int smem_bytes = 0;
  for (int s = 0; s < p.tiers.n_slots; ++s) {
    const int G = p.dh / p.tiers.g[s], C = 1 << p.tiers.bits[s];
    const int img = ((8 + 4 * G + (N * G * p.tiers.bits[s] + 7) / 8 + N * G * 2) + 15) & ~15;
    const int need = G * C * p.tiers.g[s] * 4 + TB * G * 4 + 32 * 4 + 16 + TB * G + 16 + ppb * img;
    smem_bytes = need > smem_bytes ? need : smem_bytes;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  EncodeArgs a;
  a.p = p;
  static int configured = 0;
  if (configured < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(encode_bundle_kernel<16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(encode_bundle_kernel<32>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) {
      set_error("encode: cudaFuncSetAttribute(%d B): %s", smem_bytes, cudaGetErrorString(e));
      return (int)e;
    }
    configured = smem_bytes;
  }
  // One launch per group size present; each skips the bundles of the other size.
  bool any16 = false, any32 = false;
  for (int s = 0; s < p.tiers.n_slots; ++s) (p.tiers.g[s] == 16 ? any16 : any32) = true;
  if (any16) {
    encode_bundle_kernel<16><<<p.n_bundles, kEncThreads, smem_bytes, st>>>(a);
    if (int rc = check_launch("encode_bundle_kernel<16>")) return rc;
  }
  if (any32) {
    encode_bundle_kernel<32><<<p.n_bundles, kEncThreads, smem_bytes, st>>>(a);
    if (int rc = check_launch("encode_bundle_kernel<32>")) return rc;
  }
  return 0;
}
