// Angle-domain decode attention over bit-packed, paged, codebook-quantised keys.
//
// One persistent CTA per SM (12 warps) walks a contiguous range of (KV head, batch row)
// blocks.  Each warp owns every 12th 16-token tile of the range and keeps an online-softmax
// state for all query heads of the KV head.  Per tile a warp
//   1. unpacks the tile's centroid indices and radii (lane = token x half of the groups),
//   2. rebuilds the 16 x dh key tile directly in mma A-fragment registers: gathers the
//      selected centroid rows from shared memory, scales by the radius and rotates by the
//      key's RoPE angle (cos/sin row of the key position, read through L2),
//   3. forms logits with fp16 hi/lo split operands on the tensor cores
//      (tokens x dh) * (dh x heads), fp32 accumulate,
//   4. runs the online softmax and accumulates V^T P^T with V tiles that cp.async streams
//      into a swizzled shared-memory ring.
// Every global load a tile needs is issued one or two tiles ahead.  Warp states are merged
// per CTA, CTA partials land in scratch, and a small kernel merges them by log-sum-exp.
//
// Numerics restate SphericalKVPipeline._compressed_head_attention_batched
// (spherical_kv_pipeline.py:2136-2177): logit = sum_g r_g * (q_rot_g . c_g) / sqrt(dh)
// with q back-rotated by the key position; rotating the rebuilt key forward instead is the
// same bilinear form.  Page bytes follow pagebuilder.py:8-33 / paging.py:20-31.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"

namespace sphkv {

#ifndef SPHKV_WARPS
#define SPHKV_WARPS 12
#endif
#ifndef SPHKV_CB_DUP
#define SPHKV_CB_DUP 0  // 1: store every codebook sub-row twice (bank-conflict-free gathers; measured slower)
#endif
constexpr int kWarps = SPHKV_WARPS;
constexpr int kCbPitch = SPHKV_CB_DUP ? 128 : 64;  // bytes per 16-dim codebook sub-row slot
#ifndef SPHKV_VSTAGES
#define SPHKV_VSTAGES 2
#endif
constexpr int kVStages = SPHKV_VSTAGES;  // V tiles in flight per warp: tile k + kVStages - 1 is
                                         // copied while tile k is consumed, so >= 2
static_assert(kVStages >= 2, "the V ring needs a stage to fill while another is read");
constexpr int kMetaRing = 32;  // tiles of metadata per warp, refilled 16 at a time
constexpr int kMaxUnitsInKernelPlan = 2048;

// kernel-development switch: compile sections of the tile loop out to count their
// instructions (results are wrong when non-zero); 0 in every shipped build
#ifndef SPHKV_X_SKIP
#define SPHKV_X_SKIP 0
#endif
constexpr int kSkip = SPHKV_X_SKIP;

// 16 bytes per tile
struct TileMeta {
  int phys;       // physical page id; -1 hole / invalid, -2 past the end
  int poff;       // page offset in the byte pool
  int toff;       // theta offset
  uint32_t misc;  // (radius_off - theta_off) | count << 16 | slot << 24
};
__device__ __forceinline__ int meta_count(const TileMeta& m) { return (m.misc >> 16) & 0xFF; }
__device__ __forceinline__ int meta_slot(const TileMeta& m) { return (m.misc >> 24) & 0x3; }
__device__ __forceinline__ int meta_roff(const TileMeta& m) { return m.toff + (int)(m.misc & 0xFFFF); }

struct DecodeArgs {
  sphkv_decode_params p;
  int cb_smem_off[SPHKV_MAX_TIER_SLOTS];  // byte offset of each slot's codebook in smem
  int cb_smem_bytes;
  int n_units;
  int n_ctas;
  int grp;
  int plan_in_kernel;  // every CTA derives the block prefix itself (n_units small enough)
  int32_t* pfx;
  float* rows;  // [(n_ctas + n_units)][8][dh + 2]
};

// shared-memory carve-up, shared by host and device
__host__ __device__ constexpr int smem_v_bytes(int dh) { return kWarps * kVStages * 16 * dh * 2; }
// query fragments: hi and lo copies, or one copy when both halves share the 8 MMA columns (packed)
__host__ __device__ constexpr int smem_q_bytes(int dh, bool pack) { return (pack ? 1 : 2) * (dh / 16) * 32 * 8; }
__host__ __device__ constexpr int smem_priv_bytes(int dh) {
  return 16 * (dh / 16) * 8 + 512 + kMetaRing * 16;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- plan: exclusive prefix of blocks per unit --------------------------------------
__global__ void plan_kernel(const int32_t* __restrict__ num_blocks, int n_units, int max_blocks,
                            int B, int Hkv, int32_t* __restrict__ pfx) {
  __shared__ int s_part[32];
  __shared__ int s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < n_units; base += blockDim.x) {
    int i = base + threadIdx.x;
    int v = 0;
    if (i < n_units) {
      v = num_blocks[(i % B) * Hkv + i / B];  // traversal order: KV head major, batch row minor
      v = v < 0 ? 0 : (v > max_blocks ? max_blocks : v);
    }
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) s_part[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = (lane < (int)(blockDim.x >> 5)) ? s_part[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      s_part[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    int carry = s_carry;
    int excl = carry + (warp > 0 ? s_part[warp - 1] : 0) + x - v;
    if (i < n_units) pfx[i] = excl;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) s_carry = excl + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) pfx[n_units] = s_carry;
}

// largest u in [0, n) with pfx[u] <= x < pfx[u+1]  (x < pfx[n] assumed)
__device__ __forceinline__ int find_unit(const int32_t* pfx, int n, int64_t x) {
  int lo = 0, hi = n;  // invariant: pfx[lo] <= x < pfx[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if ((int64_t)pfx[mid] <= x)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}

// words of a K page this lane needs for its (token, half-of-groups) unpack role
struct KWords {
  uint32_t th0, th1;       // aligned words holding this lane's theta bits
  uint32_t rd0, rd1, rd2;  // aligned words holding this lane's radius bytes
  float sc[4];             // per-group scales of this lane's groups
  int th_sh, rd_sh;        // bit shifts into the funnels
};

// Issue the global loads of one lane's K words.  SPG = 16-dim steps per group (g / 16).
template <int DH, int SPG>
__device__ __forceinline__ void load_kwords_t(const sphkv_decode_params& p, const TileMeta& m, int sub,
                                              int bits, int ut, int uhalf, KWords& w) {
  constexpr int HS = DH / 32, NG = HS / SPG, G = DH / (16 * SPG);
  const int tp = 16 * sub + ut;
  if (tp >= meta_count(m)) return;
  const int gam0 = uhalf * NG;
  const int bit = (tp * G + gam0) * bits;
  const int ba = m.toff + (bit >> 3);
  const uint32_t* wp = reinterpret_cast<const uint32_t*>(p.k_pages + (ba & ~3));
  w.th_sh = (ba & 3) * 8 + (bit & 7);
  w.th0 = wp[0];
  if (w.th_sh + NG * bits > 32) w.th1 = wp[1];
  const int rb = p.radius_fmt == SPHKV_RADIUS_F16 ? 2 : 1;
  const int ra = meta_roff(m) + (tp * G + gam0) * rb;
  const uint32_t* rp = reinterpret_cast<const uint32_t*>(p.k_pages + (ra & ~3));
  w.rd_sh = (ra & 3) * 8;
  const int need = (ra & 3) + NG * rb;  // bytes from the aligned word start
  w.rd0 = rp[0];
  if (need > 4) w.rd1 = rp[1];
  if (need > 8) w.rd2 = rp[2];
  if (rb == 1) {
    const float* sp = reinterpret_cast<const float*>(p.k_pages + m.poff + 8) + gam0;
#pragma unroll
    for (int i = 0; i < NG; ++i) w.sc[i] = sp[i];
  }
}

// Unpack this lane's codes and radii into (codebook row offset, radius) entries, one per
// 16-dim step: unp[token][step].
template <int DH, int SPG>
__device__ __forceinline__ void unpack_t(const KWords& w, const TileMeta& m, int sub, int bits, int fmt,
                                         uint32_t cbase, int ut, int uhalf, uint2* unp) {
  constexpr int KS = DH / 16, HS = KS / 2, NG = HS / SPG;
  const int gam0 = uhalf * NG;
  const uint32_t cmask = (1u << bits) - 1u;
  const uint32_t tb = __funnelshift_r(w.th0, w.th1, w.th_sh);
  const uint32_t rlo = __funnelshift_r(w.rd0, w.rd1, w.rd_sh);
  const uint32_t rhi = __funnelshift_r(w.rd1, w.rd2, w.rd_sh);
  const bool tok_ok = (16 * sub + ut) < meta_count(m);
  uint2 e[NG * SPG];
#pragma unroll
  for (int i = 0; i < NG; ++i) {
    const uint32_t code = (tb >> (i * bits)) & cmask;
    float rad;
    if (fmt == SPHKV_RADIUS_F16) {
      const uint32_t wv = (i < 2) ? rlo : rhi;
      rad = __half2float(__ushort_as_half((unsigned short)(wv >> ((i & 1) * 16))));
    } else {
      const int c8 = (int)(int8_t)((rlo >> (i * 8)) & 0xFFu);
      rad = (w.sc[i] * (float)c8) * (1.0f / 127.0f);
    }
    if (!tok_ok) rad = 0.f;
    const uint32_t row = (((uint32_t)(gam0 + i) << bits) + code) * SPG;
#pragma unroll
    for (int s2 = 0; s2 < SPG; ++s2)
      e[i * SPG + s2] = make_uint2(cbase + (row + s2) * (uint32_t)kCbPitch, __float_as_uint(rad));
  }
  uint2* dst = unp + ut * KS + gam0 * SPG;  // 16-byte aligned: KS and NG*SPG are even
#pragma unroll
  for (int i = 0; i < NG * SPG; i += 2)
    *reinterpret_cast<uint4*>(dst + i) = make_uint4(e[i].x, e[i].y, e[i + 1].x, e[i + 1].y);
}

// rotate one (low-half, high-half) float4 pair by (cos, sin) and split into fp16 hi/lo
// A-fragment registers
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// Operand precision of the QK^T contraction: both the rebuilt key tile and the query are
// split as hi + lo 16-bit halves and three products are accumulated in fp32
// (hi*hi + lo*hi + hi*lo).  SPHKV_SPLIT_BF16: bf16 halves (hi by truncation, no conversion
// instructions on the slow pipe; ~2^-16 relative); otherwise fp16 halves (~2^-21).
#ifdef SPHKV_SPLIT_BF16
__device__ __forceinline__ void split_pair(float2 v, uint32_t& hi, uint32_t& lo) {
  const uint32_t a = __float_as_uint(v.x), b = __float_as_uint(v.y);
  hi = __byte_perm(a, b, 0x7632);  // upper halves = truncated bf16 pair
  const float2 nh = f2(__uint_as_float((a & 0xFFFF0000u) ^ 0x80000000u),
                       __uint_as_float((b & 0xFFFF0000u) ^ 0x80000000u));
  const float2 l = __fadd2_rn(v, nh);
  __nv_bfloat162 lb = __floats2bfloat162_rn(l.x, l.y);
  lo = *reinterpret_cast<uint32_t*>(&lb);
}
#define SPHKV_QK_MMA mma_bf16_16816
#else
__device__ __forceinline__ void split_pair(float2 v, uint32_t& hi, uint32_t& lo) {
  split_f16x2(v.x, v.y, hi, lo);
}
#define SPHKV_QK_MMA mma_f16_16816
#endif

// rotate one (low-half, high-half) float4 pair by (cos, sin) and split into hi/lo
// A-fragment registers
template <bool ROT>
__device__ __forceinline__ void build_pair(float4 x, float4 y, float r0, float r1, const float4& c,
                                           const float4& sn, int tk, uint32_t (&a_lo_hi)[4],
                                           uint32_t (&a_lo_lo)[4], uint32_t (&a_hi_hi)[4],
                                           uint32_t (&a_hi_lo)[4]) {
#ifndef SPHKV_NO_F32X2
  const float2 rr0 = f2(r0, r0), rr1 = f2(r1, r1);
  float2 x0 = __fmul2_rn(f2(x.x, x.y), rr0), x1 = __fmul2_rn(f2(x.z, x.w), rr0);
  float2 y0 = __fmul2_rn(f2(y.x, y.y), rr1), y1 = __fmul2_rn(f2(y.z, y.w), rr1);
  float2 lo0 = x0, lo1 = x1, hi0 = y0, hi1 = y1;
  if (ROT) {
    const float2 c0 = f2(c.x, c.y), c1 = f2(c.z, c.w);
    const float2 s0 = f2(sn.x, sn.y), s1 = f2(sn.z, sn.w);
    const float2 n0 = f2(-sn.x, -sn.y), n1 = f2(-sn.z, -sn.w);
    lo0 = __ffma2_rn(y0, n0, __fmul2_rn(x0, c0));
    lo1 = __ffma2_rn(y1, n1, __fmul2_rn(x1, c1));
    hi0 = __ffma2_rn(x0, s0, __fmul2_rn(y0, c0));
    hi1 = __ffma2_rn(x1, s1, __fmul2_rn(y1, c1));
  }
#else
  x.x *= r0; x.y *= r0; x.z *= r0; x.w *= r0;
  y.x *= r1; y.y *= r1; y.z *= r1; y.w *= r1;
  float2 lo0 = f2(x.x, x.y), lo1 = f2(x.z, x.w), hi0 = f2(y.x, y.y), hi1 = f2(y.z, y.w);
  if (ROT) {
    lo0.x = fmaf(x.x, c.x, -(y.x * sn.x)); hi0.x = fmaf(y.x, c.x, x.x * sn.x);
    lo0.y = fmaf(x.y, c.y, -(y.y * sn.y)); hi0.y = fmaf(y.y, c.y, x.y * sn.y);
    lo1.x = fmaf(x.z, c.z, -(y.z * sn.z)); hi1.x = fmaf(y.z, c.z, x.z * sn.z);
    lo1.y = fmaf(x.w, c.w, -(y.w * sn.w)); hi1.y = fmaf(y.w, c.w, x.w * sn.w);
  }
#endif
  split_pair(lo0, a_lo_hi[tk], a_lo_lo[tk]);
  split_pair(lo1, a_lo_hi[2 + tk], a_lo_lo[2 + tk]);
  split_pair(hi0, a_hi_hi[tk], a_hi_lo[tk]);
  split_pair(hi1, a_hi_hi[2 + tk], a_hi_lo[2 + tk]);
}

// PACK (<= 4 query heads per KV head): the 8 mma columns carry [q_hi heads 0..3 | q_lo heads
// 0..3] (one product fewer per step) and later [P_hi | P_lo] (one product per V tile).
template <int DH, typename VT, bool ROT, bool EXTRA, bool PACK>
__global__ void __launch_bounds__(kWarps * 32, 1) decode_splitk_kernel(const DecodeArgs a) {
  constexpr int KS = DH / 16;  // 16-dim steps over the head dim
  constexpr int HS = KS / 2;   // steps in one rotary half
  constexpr int V_TILE = 16 * DH * 2;
  constexpr int V_WARP = kVStages * V_TILE;
  constexpr bool kBf16 = std::is_same<VT, __nv_bfloat16>::value;

  extern __shared__ __align__(1024) uint8_t smem[];
  const sphkv_decode_params& p = a.p;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, j = lane & 3;
  const int ut = lane >> 1, uhalf = lane & 1;  // unpack role: token, half of the groups

  uint8_t* v_ring = smem + warp * V_WARP;
  uint8_t* cb_smem = smem + smem_v_bytes(DH);
  const uint8_t* cb_lane = cb_smem + j * 16 + (SPHKV_CB_DUP ? (r & 1) * 64 : 0);  // this lane's chunk of its copy
  uint2* q_smem = reinterpret_cast<uint2*>(cb_smem + a.cb_smem_bytes);  // [PACK ? 1 : 2][KS][32]
  uint8_t* warp_priv = cb_smem + a.cb_smem_bytes + smem_q_bytes(DH, PACK) + warp * smem_priv_bytes(DH);
  uint2* unp = reinterpret_cast<uint2*>(warp_priv);                       // [16][KS]
  uint16_t* pbuf = reinterpret_cast<uint16_t*>(warp_priv + 16 * KS * 8);  // [2][8][16]
  TileMeta* meta = reinterpret_cast<TileMeta*>(warp_priv + 16 * KS * 8 + 512);

  // ---- block prefix per unit: computed by warp 0 of every CTA (CTA 0 publishes it for the
  //      merge kernel), or read from the plan kernel's output when there are many units ----
  const int32_t* pfx = a.pfx;
  if (a.plan_in_kernel) {
    int32_t* pfx_s = reinterpret_cast<int32_t*>(cb_smem + a.cb_smem_bytes + smem_q_bytes(DH, PACK) +
                                                kWarps * smem_priv_bytes(DH));
    if (warp == 0) {
      int carry = 0;
      for (int base = 0; base < a.n_units; base += 32) {
        const int i = base + lane;
        int v = 0;
        if (i < a.n_units) {
          v = p.num_blocks[(i % p.B) * p.Hkv + i / p.B];
          v = v < 0 ? 0 : (v > p.max_blocks ? p.max_blocks : v);
        }
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, x, o);
          if (lane >= o) x += y;
        }
        if (i < a.n_units) {
          pfx_s[i] = carry + x - v;
          if (blockIdx.x == 0) a.pfx[i] = carry + x - v;
        }
        carry += __shfl_sync(0xffffffffu, x, 31);
      }
      if (lane == 0) {
        pfx_s[a.n_units] = carry;
        if (blockIdx.x == 0) a.pfx[a.n_units] = carry;
      }
    }
    __syncthreads();
    pfx = pfx_s;
  }
  const int64_t T = pfx[a.n_units];
  if (T == 0) return;
  int64_t start = cta_range_start(blockIdx.x, a.n_ctas, T);
  const int64_t end = cta_range_start(blockIdx.x + 1, a.n_ctas, T);
  if (start >= end) return;
  int u = find_unit(pfx, a.n_units, start);

  const int N = p.page_size;
  const int TPP = N >> 4;                 // 16-token tiles per page: 1, 2, 4 or 8
  const int tpp_shift = 31 - __clz(TPP);
  const float qscale = p.sm_scale * kLog2e;
  const int fmt = p.radius_fmt;
  int cb_head_loaded = -1;
  // per tier slot: b_theta | steps-per-group << 8 | codebook offset in shared memory << 12,
  // held by lanes 0..3 and read with a shuffle (no indexing into kernel parameters)
  uint32_t tier_word = 0;
  if (lane < SPHKV_MAX_TIER_SLOTS && lane < p.tiers.n_slots) {
    int g_l = 16, b_l = 1, off_l = 0;
#pragma unroll
    for (int s = 0; s < SPHKV_MAX_TIER_SLOTS; ++s)
      if (s == lane) { g_l = p.tiers.g[s]; b_l = p.tiers.bits[s]; off_l = a.cb_smem_off[s]; }
    tier_word = (uint32_t)b_l | ((uint32_t)(g_l >> 4) << 8) | ((uint32_t)off_l << 12);
  }
  auto tier_of = [&](int slot) { return __shfl_sync(0xffffffffu, tier_word, slot); };

  while (start < end) {
    while ((int64_t)pfx[u + 1] <= start) ++u;  // skip units without blocks
    const int64_t seg_end = end < (int64_t)pfx[u + 1] ? end : (int64_t)pfx[u + 1];
    const int lb0 = (int)(start - pfx[u]);
    const int seg_tiles = (int)(seg_end - start) * TPP;
    // units are walked KV head major (u = hkv * B + b) so that neighbouring segments share
    // their codebooks; tables are indexed by the external unit id b * Hkv + hkv
    const int hkv = u / p.B, b = u - hkv * p.B;
    const int u_ext = b * p.Hkv + hkv;
    const int nt = seg_tiles > warp ? (seg_tiles - warp + kWarps - 1) / kWarps : 0;
    const int32_t* bt_row = p.block_table + (int64_t)u_ext * p.max_blocks;
    const int32_t* st_row = p.bits_table + (int64_t)u_ext * p.max_blocks;

    auto tile_lb = [&](int kk) { return lb0 + ((warp + kWarps * kk) >> tpp_shift); };
    auto tile_sub = [&](int kk) { return (warp + kWarps * kk) & (TPP - 1); };
    // per-tile statistics of this segment: tile kk of head n lands at ml_seg[n * ml_head + 2 * (warp + 12 kk)]
    float* ml_seg = nullptr;
    const int64_t ml_head = (int64_t)p.max_blocks * TPP * 2;
    if (EXTRA && p.page_ml != nullptr)
      ml_seg = p.page_ml + ((int64_t)b * p.Hq + (int64_t)hkv * a.grp) * ml_head + ((int64_t)lb0 * TPP + warp) * 2;

    // Tile metadata is fetched 16 tiles at a time, lane = tile (lanes 0..15).  The three
    // dependent loads (block table -> pointer table -> page header) are issued in separate
    // loop iterations so that no iteration waits for a load it issued itself.
    int mf_phys = -2, mf_slot = 0, mf_poff = 0, mf_toff = 0, mf_roff = 0;
    auto meta_stage0 = [&](int kbase) {
      const int kk = kbase + lane;
      mf_phys = -2; mf_slot = 0; mf_poff = mf_toff = mf_roff = 0;
      if (lane < 16 && kk < nt) {
        const int lb = tile_lb(kk);
        mf_phys = bt_row[lb];
        mf_slot = st_row[lb];
      }
    };
    auto meta_stage1 = [&]() {
      if (mf_phys == -2) return;
      if (mf_phys >= p.n_pages) {
        if (p.status) atomicOr(p.status, SPHKV_ST_BAD_BLOCK);
        mf_phys = -1;
      }
      if (mf_slot < 0 || mf_slot >= p.tiers.n_slots) {
        if (p.status) atomicOr(p.status, SPHKV_ST_BAD_SLOT);
        mf_phys = -1;
        mf_slot = 0;
      }
      if (mf_phys < 0) { mf_phys = -1; return; }
      mf_poff = p.ptable[3 * (int64_t)mf_phys + 0];
      mf_toff = p.ptable[3 * (int64_t)mf_phys + 1];
      mf_roff = p.ptable[3 * (int64_t)mf_phys + 2];
    };
    auto meta_stage2 = [&](int kbase) {
      if (lane >= 16) return;
      TileMeta m;
      m.phys = mf_phys; m.poff = mf_poff; m.toff = mf_toff;
      int count = 0;
      if (mf_phys >= 0) {
        const uint32_t hdr = *reinterpret_cast<const uint32_t*>(p.k_pages + mf_poff);
        count = (int)((hdr >> 8) & 0xFFu);
        if (count > N) count = N;
      }
      m.misc = (uint32_t)((mf_roff - mf_toff) & 0xFFFF) | ((uint32_t)count << 16) | ((uint32_t)mf_slot << 24);
      meta[(kbase + lane) & (kMetaRing - 1)] = m;
    };
    auto get_meta = [&](int kk) -> TileMeta {
      const uint4 v = *reinterpret_cast<const uint4*>(&meta[kk & (kMetaRing - 1)]);
      TileMeta m;
      m.phys = (int)v.x; m.poff = (int)v.y; m.toff = (int)v.z; m.misc = v.w;
      return m;
    };

    // V tile copy: lane owns 16-byte chunk column c = lane % (DH/8) of token rows
    // tau = q * (256/DH) + lane / (DH/8); destination chunks are XOR-swizzled by (tau & 7)
    auto issue_v = [&](int kk) {
      if (kk < nt && !(kSkip & 8)) {
        const TileMeta m = get_meta(kk);
        if (m.phys >= 0) {
          constexpr int CPR = DH / 8;       // chunks per token row
          constexpr int RPI = 32 / CPR;     // token rows per warp-wide copy instruction
          const int c = lane % CPR, t0 = lane / CPR;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.v_pool) +
                               ((int64_t)m.phys * N + 16 * tile_sub(kk)) * (DH * 2) + t0 * (DH * 2) + c * 16;
          const uint32_t dst = smem_u32(v_ring) + (uint32_t)(kk % kVStages) * V_TILE + (c >> 3) * 2048 +
                               t0 * 128;
#pragma unroll
          for (int q = 0; q < 16 / RPI; ++q) {
            const int tau = q * RPI + t0;
            cp_async_16(dst + q * RPI * 128 + (((c & 7) ^ (tau & 7)) << 4), src + q * RPI * DH * 2);
          }
        }
      }
      cp_async_commit();
    };

    auto load_kwords = [&](int kk, KWords& w) {
      w.th0 = w.th1 = w.rd0 = w.rd1 = w.rd2 = 0u;
      w.th_sh = w.rd_sh = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) w.sc[i] = 0.f;
      if (kk >= nt || (kSkip & 16)) return;
      const TileMeta m = get_meta(kk);
      if (m.phys < 0) return;
      const uint32_t tw = tier_of(meta_slot(m));
      if (((tw >> 8) & 0xF) == 1)
        load_kwords_t<DH, 1>(p, m, tile_sub(kk), tw & 0xFF, ut, uhalf, w);
      else
        load_kwords_t<DH, 2>(p, m, tile_sub(kk), tw & 0xFF, ut, uhalf, w);
    };
    // key positions of rows r and r+8 of tile kk (-1: no token)
    auto load_pos = [&](int kk, int (&ps)[2]) {
      ps[0] = ps[1] = -1;
      if (!ROT || kk >= nt) return;
      const TileMeta m = get_meta(kk);
      if (m.phys < 0) return;
      const int32_t* pp = p.positions + (int64_t)m.phys * N + 16 * tile_sub(kk);
      ps[0] = pp[r];
      ps[1] = pp[r + 8];
    };

    float4 cs[2][HS][2];
    auto issue_cs = [&](const int (&ps)[2]) {
      if constexpr (ROT && !(kSkip & 32)) {
#pragma unroll
      for (int tk = 0; tk < 2; ++tk) {
        int pos = ps[tk];
        if (pos >= p.max_pos) {
          if (p.status) atomicOr(p.status, SPHKV_ST_BAD_POSITION);
          pos = 0;
        }
        if (pos < 0) pos = 0;
        const float4* rp = reinterpret_cast<const float4*>(p.rope_table + (int64_t)pos * DH) + j * 2;
#pragma unroll
        for (int s = 0; s < HS; ++s) {
          // through L1 on purpose: a lane's cos and sin vectors share a 32-byte sector (and one
          // 256-bit load for both measured slower than the two 128-bit ones)
          cs[tk][s][0] = __ldg(rp + s * 8);
          cs[tk][s][1] = __ldg(rp + s * 8 + 1);
        }
      }
      }
    };

    auto stage_codebooks = [&]() {
      if (hkv == cb_head_loaded) return;
      const sphkv_tiers& tg = p.tiers;
      for (int s = 0; s < tg.n_slots; ++s) {
        // one thread per 16-dim sub-row: four 128-bit loads, four 128-bit stores in the
        // lane-quad order (2j, 2j+1, 2j+8, 2j+9)
        const int g = tg.g[s], bits = tg.bits[s], G = DH / g, spg = g >> 4;
        const float* src =
            p.codebooks + ((int64_t)(hkv * tg.n_slots + s) * tg.G_max) * tg.C_max * tg.g_max;
        float4* dst = reinterpret_cast<float4*>(cb_smem + a.cb_smem_off[s]);
        const int rows = (G << bits) * spg;
#pragma unroll 2
        for (int row = threadIdx.x; row < rows; row += blockDim.x) {
          const int sub2 = row & (spg - 1), gc = row / spg;
          const int c = gc & ((1 << bits) - 1), gam = gc >> bits;
          const float4* sp = reinterpret_cast<const float4*>(
              src + ((int64_t)gam * tg.C_max + c) * tg.g_max + sub2 * 16);
          const float4 v0 = __ldg(sp), v1 = __ldg(sp + 1), v2 = __ldg(sp + 2), v3 = __ldg(sp + 3);
          // each 64-byte sub-row is stored twice, at bytes 0 and 64 of a 128-byte slot: even
          // tokens read the first copy, odd tokens the second, so the two tokens served by one
          // shared-memory wavefront never meet in a bank
          const float4 w0 = make_float4(v0.x, v0.y, v2.x, v2.y), w1 = make_float4(v0.z, v0.w, v2.z, v2.w);
          const float4 w2 = make_float4(v1.x, v1.y, v3.x, v3.y), w3 = make_float4(v1.z, v1.w, v3.z, v3.w);
          constexpr int SL = kCbPitch / 16;
          dst[row * SL + 0] = w0; dst[row * SL + 1] = w1; dst[row * SL + 2] = w2; dst[row * SL + 3] = w3;
          if (SPHKV_CB_DUP) {
            dst[row * SL + 4] = w0; dst[row * SL + 5] = w1; dst[row * SL + 6] = w2; dst[row * SL + 7] = w3;
          }
        }
      }
      cb_head_loaded = hkv;
    };

    // query fragments, B operand [k = dim][n = head], fp16 hi/lo, pre-scaled by
    // sm_scale * log2(e); one copy per CTA in shared memory: q_smem[hl][step][lane]
    auto stage_q = [&]() {
      for (int i = threadIdx.x; i < KS * 32; i += blockDim.x) {
        const int s = i >> 5, ln = i & 31, n = ln >> 2, jj = ln & 3;
        const int head = PACK ? (n & 3) : n;
        const bool real = head < a.grp;
        const int64_t qbase = ((int64_t)b * p.Hq + (int64_t)hkv * a.grp + head) * DH;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int d = 16 * s + 2 * jj + (e & 1) + ((e >> 1) << 3);
          v[e] = real ? load_as_float(p.q, p.q_dtype, qbase + d) * qscale : 0.f;
        }
        uint2 hi, lo;
        split_pair(f2(v[0], v[1]), hi.x, lo.x);
        split_pair(f2(v[2], v[3]), hi.y, lo.y);
        if (PACK) {
          q_smem[i] = n < 4 ? hi : lo;   // columns 0..3: hi halves, 4..7: lo halves
        } else {
          q_smem[i] = hi;
          q_smem[KS * 32 + i] = lo;
        }
      }
    };

    // online-softmax state: this lane's two head columns (2j, 2j+1)
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    float acc[KS][4];
#pragma unroll
    for (int dt = 0; dt < KS; ++dt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[dt][e] = 0.f;

    // ---- prologue: the block-table -> pointer-table -> header chain of the first 16 tiles
    //      is interleaved with the codebook and query loads so their latencies overlap ----
    __syncthreads();  // the previous segment is done with shared memory
    meta_stage0(0);
    stage_codebooks();
    meta_stage1();
    stage_q();
    meta_stage2(0);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kVStages - 1; ++i) issue_v(i);
    KWords cur, nx;
    int pos_c[2], pos_1[2], pos_2[2];  // positions of tiles k, k+1, k+2
    load_kwords(0, cur);
    load_pos(0, pos_c);
    load_pos(1, pos_1);
    issue_cs(pos_c);

    for (int k = 0; k < nt; ++k) {
      {  // fetch the next 16 tiles' metadata into the idle half of the ring, in three steps
        const int ph = k & 15, kb = (k & ~15) + 16;
        if (ph == 0) meta_stage0(kb);
        else if (ph == 5) meta_stage1();
        else if (ph == 10) { meta_stage2(kb); __syncwarp(); }
      }
      issue_v(k + kVStages - 1);  // into the stage tile k - 1 has just released
      load_kwords(k + 1, nx);
      load_pos(k + 2, pos_2);
      const TileMeta m = get_meta(k);
      const int sub = tile_sub(k);
      const int cnt_tile = m.phys < 0 ? 0 : min(16, max(0, meta_count(m) - 16 * sub));

      if (cnt_tile > 0) {
        // ---- phase A: unpack codes/radii of (token ut, half uhalf) ------------------
        if constexpr (!(kSkip & 1)) {
          const uint32_t tw = tier_of(meta_slot(m));
          const uint32_t cbase = tw >> 12;
          if (((tw >> 8) & 0xF) == 1)
            unpack_t<DH, 1>(cur, m, sub, tw & 0xFF, fmt, cbase, ut, uhalf, unp);
          else
            unpack_t<DH, 2>(cur, m, sub, tw & 0xFF, fmt, cbase, ut, uhalf, unp);
        }
        __syncwarp();

        // ---- phase B: rebuild rotated key tile in A fragments, QK^T on tensor cores -
        float s_hh[4] = {0.f, 0.f, 0.f, 0.f}, s_lh[4] = {0.f, 0.f, 0.f, 0.f},
              s_hl[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < ((kSkip & 2) ? 0 : HS); ++s) {
          uint32_t a_lo_hi[4], a_lo_lo[4], a_hi_hi[4], a_hi_lo[4];
#pragma unroll
          for (int tk = 0; tk < 2; ++tk) {
            const int tau = r + 8 * tk;
            const uint2 e0 = unp[tau * KS + s];
            const uint2 e1 = unp[tau * KS + s + HS];
            const float4 x = *reinterpret_cast<const float4*>(cb_lane + e0.x);
            const float4 y = *reinterpret_cast<const float4*>(cb_lane + e1.x);
            build_pair<ROT>(x, y, __uint_as_float(e0.y), __uint_as_float(e1.y), cs[tk][s][0],
                            cs[tk][s][1], tk, a_lo_hi, a_lo_lo, a_hi_hi, a_hi_lo);
          }
          if (PACK) {
            const uint2 q0 = q_smem[s * 32 + lane], q1 = q_smem[(s + HS) * 32 + lane];
            SPHKV_QK_MMA(s_hh, a_lo_hi, q0.x, q0.y);
            SPHKV_QK_MMA(s_lh, a_lo_lo, q0.x, q0.y);
            SPHKV_QK_MMA(s_hh, a_hi_hi, q1.x, q1.y);
            SPHKV_QK_MMA(s_lh, a_hi_lo, q1.x, q1.y);
          } else {
            const uint2 qh0 = q_smem[s * 32 + lane], ql0 = q_smem[(KS + s) * 32 + lane];
            const uint2 qh1 = q_smem[(s + HS) * 32 + lane], ql1 = q_smem[(KS + s + HS) * 32 + lane];
            SPHKV_QK_MMA(s_hh, a_lo_hi, qh0.x, qh0.y);
            SPHKV_QK_MMA(s_lh, a_lo_lo, qh0.x, qh0.y);
            SPHKV_QK_MMA(s_hl, a_lo_hi, ql0.x, ql0.y);
            SPHKV_QK_MMA(s_hh, a_hi_hi, qh1.x, qh1.y);
            SPHKV_QK_MMA(s_lh, a_hi_lo, qh1.x, qh1.y);
            SPHKV_QK_MMA(s_hl, a_hi_hi, ql1.x, ql1.y);
          }
        }
        // the cos/sin registers are free now: fetch the next tile's rows
        issue_cs(pos_1);

        // ---- online softmax over the 16 token rows, per head column ------------------
        float sv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          sv[e] = s_hh[e] + (s_lh[e] + s_hl[e]);
          // packed columns: head h's logit = column h (x q_hi) + column 4+h (x q_lo)
          if (PACK) sv[e] += __shfl_xor_sync(0xffffffffu, sv[e], 2);
        }
        if (EXTRA && p.logits_out != nullptr) {
          const int lb = tile_lb(k);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = 2 * j + (e & 1), tok = r + ((e >> 1) << 3);
            if (n < a.grp && tok < cnt_tile && (!PACK || j < 2))
              p.logits_out[(((int64_t)b * p.Hq + (int64_t)hkv * a.grp + n) * p.max_blocks + lb) * N +
                           16 * sub + tok] = sv[e] * kLn2;
          }
        }
        const bool ok0 = r < cnt_tile && (!ROT || pos_c[0] >= 0);
        const bool ok1 = (r + 8) < cnt_tile && (!ROT || pos_c[1] >= 0);
        if (!ok0) sv[0] = sv[1] = -INFINITY;
        if (!ok1) sv[2] = sv[3] = -INFINITY;
        float tmax[2] = {fmaxf(sv[0], sv[2]), fmaxf(sv[1], sv[3])};
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          tmax[0] = fmaxf(tmax[0], __shfl_xor_sync(0xffffffffu, tmax[0], o));
          tmax[1] = fmaxf(tmax[1], __shfl_xor_sync(0xffffffffu, tmax[1], o));
        }
        float alpha[2], msafe[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float mn = fmaxf(m_run[c], tmax[c]);
          msafe[c] = (mn == -INFINITY) ? 0.f : mn;
          alpha[c] = fast_exp2(m_run[c] - msafe[c]);
          m_run[c] = mn;
        }
        float pv[4];
        pv[0] = fast_exp2(sv[0] - msafe[0]);
        pv[1] = fast_exp2(sv[1] - msafe[1]);
        pv[2] = fast_exp2(sv[2] - msafe[0]);
        pv[3] = fast_exp2(sv[3] - msafe[1]);
        l_run[0] = l_run[0] * alpha[0] + (pv[0] + pv[2]);
        l_run[1] = l_run[1] * alpha[1] + (pv[1] + pv[3]);
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
          for (int dt = 0; dt < KS; ++dt) {
            acc[dt][0] *= alpha[0]; acc[dt][1] *= alpha[1];
            acc[dt][2] *= alpha[0]; acc[dt][3] *= alpha[1];
          }
        }
        if (EXTRA && ml_seg != nullptr) {
          // per-tile (max, sum) in the natural-log domain for heads 2j, 2j+1
          float ls[2] = {pv[0] + pv[2], pv[1] + pv[3]};
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) {
            ls[0] += __shfl_xor_sync(0xffffffffu, ls[0], o);
            ls[1] += __shfl_xor_sync(0xffffffffu, ls[1], o);
          }
          if (r == 0) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int n = 2 * j + c;
              if (n < a.grp && (!PACK || j < 2)) {
                float* dst = ml_seg + n * ml_head + 2 * kWarps * k;
                const float tm = tmax[c];
                dst[0] = tm * kLn2;
                dst[1] = (tm == -INFINITY) ? 0.f : ls[c] * fast_exp2(msafe[c] - tm);
              }
            }
          }
        }

        // ---- P^T through shared memory into the B-operand layout -------------------
        // pbuf[h][head][token]: fp16 (or bf16 hi / lo for a bf16 V pool)
        {
          uint16_t* ph = pbuf;
          uint16_t* pl = pbuf + 8 * 16;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int head = 2 * j + (e & 1), tok = r + ((e >> 1) << 3);
            uint16_t hbits, lbits;
            if (kBf16) {
              const __nv_bfloat16 h = __float2bfloat16_rn(pv[e]);
              hbits = __bfloat16_as_ushort(h);
              lbits = __bfloat16_as_ushort(__float2bfloat16_rn(pv[e] - __bfloat162float(h)));
            } else {
              hbits = __half_as_ushort(__float2half_rn(pv[e]));
              lbits = 0;
            }
            if (PACK) {
              // columns 0..3 hold P (hi half), columns 4..7 the lo half (zero for an fp16 V pool)
              ph[head * 16 + tok] = j < 2 ? hbits : lbits;
            } else {
              ph[head * 16 + tok] = hbits;
              if (kBf16) pl[head * 16 + tok] = lbits;
            }
          }
        }
        cp_async_wait<kVStages - 1>();  // tile k's copy has landed (later ones may be in flight)
        __syncwarp();
        {
          const uint32_t* ph32 = reinterpret_cast<const uint32_t*>(pbuf);
          const uint32_t b0 = ph32[(r * 16 + 2 * j) >> 1];
          const uint32_t b1 = ph32[(r * 16 + 2 * j + 8) >> 1];
          uint32_t c0 = 0, c1 = 0;
          if (kBf16 && !PACK) {
            c0 = ph32[(8 * 16 + r * 16 + 2 * j) >> 1];
            c1 = ph32[(8 * 16 + r * 16 + 2 * j + 8) >> 1];
          }
          // ---- acc^T[dh][head] += V^T[dh][token] P^T[token][head] ---------------------
          const uint32_t vbase = smem_u32(v_ring + (k % kVStages) * V_TILE);
          const int mi = lane >> 3;
          const int tau = (lane & 7) + ((mi >> 1) << 3);
#pragma unroll
          for (int dt = 0; dt < ((kSkip & 4) ? 0 : KS); ++dt) {
            const int c = 2 * dt + (mi & 1);
            uint32_t af[4];
            ldmatrix_x4_trans(af, vbase + (c >> 3) * 2048 + tau * 128 + (((c & 7) ^ (tau & 7)) << 4));
            if (kBf16) {
              mma_bf16_16816(acc[dt], af, b0, b1);
              if (!PACK) mma_bf16_16816(acc[dt], af, c0, c1);
            } else {
              mma_f16_16816(acc[dt], af, b0, b1);
            }
          }
        }
        __syncwarp();
      } else {
        issue_cs(pos_1);
        cp_async_wait<kVStages - 1>();
        __syncwarp();
        if (EXTRA && ml_seg != nullptr && lane < a.grp) {  // a tile without tokens: (-inf, 0)
          float* dst = ml_seg + lane * ml_head + 2 * kWarps * k;
          dst[0] = -INFINITY;
          dst[1] = 0.f;
        }
      }
      cur = nx;
      pos_c[0] = pos_1[0]; pos_c[1] = pos_1[1];
      pos_1[0] = pos_2[0]; pos_1[1] = pos_2[1];
    }
    cp_async_wait<0>();

    // ---- merge the warps of this CTA and write one partial row ---------------------
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
      l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
    }
    __syncthreads();  // every warp is done with its V ring
    {
      float* wbuf = reinterpret_cast<float*>(v_ring);  // [8 heads][DH + 2]
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int n = 2 * j + c;
        if (r == 0) {
          wbuf[n * (DH + 2) + 0] = m_run[c];
          wbuf[n * (DH + 2) + 1] = l_run[c];
        }
#pragma unroll
        for (int dt = 0; dt < KS; ++dt) {
          wbuf[n * (DH + 2) + 2 + 16 * dt + r] = acc[dt][c];
          wbuf[n * (DH + 2) + 2 + 16 * dt + r + 8] = acc[dt][2 + c];
        }
      }
    }
    __syncthreads();
    {
      float* row = a.rows + (int64_t)(blockIdx.x + u) * 8 * (DH + 2);
      for (int i = threadIdx.x; i < a.grp * (DH + 2); i += blockDim.x) {
        const int n = i / (DH + 2), e = i - n * (DH + 2);
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w)
          M = fmaxf(M, reinterpret_cast<const float*>(smem + w * V_WARP)[n * (DH + 2)]);
        float outv;
        if (e == 0) {
          outv = M;
        } else {
          outv = 0.f;
          if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
              const float* wb = reinterpret_cast<const float*>(smem + w * V_WARP) + n * (DH + 2);
              const float mw = wb[0];
              if (mw != -INFINITY) {
                float val = wb[e];
                if (PACK && e >= 2) val += wb[4 * (DH + 2) + e];  // the P_lo columns
                outv += val * fast_exp2(mw - M);
              }
            }
          }
        }
        row[i] = outv;
      }
    }
    start = seg_end;
    ++u;
  }
}

template <int DH>
__global__ void __launch_bounds__(256) merge_rows_kernel(const DecodeArgs a) {
  constexpr int kChunk = 128;  // partial rows combined per pass
  const sphkv_decode_params& p = a.p;
  const int u = blockIdx.x;  // traversal index: hkv * B + b
  const int hkv = u / p.B, b = u - hkv * p.B;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ int s_c[2];
  __shared__ float s_M[8], s_L[8];
  __shared__ float s_w[8][kChunk];
  const int32_t* pfx = a.pfx;
  const int64_t T = pfx[a.n_units];
  const int64_t ps = pfx[u], pe = pfx[u + 1];
  if (threadIdx.x == 0) {
    int c_lo = 0, c_hi = -1;
    if (pe > ps && T > 0) {
      c_lo = (int)((ps * a.n_ctas) / T);
      if (c_lo >= a.n_ctas) c_lo = a.n_ctas - 1;
      while (c_lo > 0 && cta_range_start(c_lo, a.n_ctas, T) > ps) --c_lo;
      while (cta_range_start(c_lo + 1, a.n_ctas, T) <= ps) ++c_lo;
      c_hi = (int)(((pe - 1) * a.n_ctas) / T);
      if (c_hi >= a.n_ctas) c_hi = a.n_ctas - 1;
      while (c_hi > c_lo && cta_range_start(c_hi, a.n_ctas, T) >= pe) --c_hi;
      while (c_hi + 1 < a.n_ctas && cta_range_start(c_hi + 1, a.n_ctas, T) < pe) ++c_hi;
    }
    s_c[0] = c_lo;
    s_c[1] = c_hi;
  }
  __syncthreads();
  const int c_lo = s_c[0], c_hi = s_c[1], nrows = c_hi - c_lo + 1;
  auto row_m = [&](int n, int c) -> float {  // max of row (c, u) for head n; -inf if no such row
    if (cta_range_start(c, a.n_ctas, T) == cta_range_start(c + 1, a.n_ctas, T)) return -INFINITY;
    return a.rows[((int64_t)(c + u) * 8 + n) * (DH + 2)];
  };
  // pass 1: warp n -> global max and sum of head n
  if (warp < a.grp) {
    float M = -INFINITY;
    for (int i = lane; i < nrows; i += 32) M = fmaxf(M, row_m(warp, c_lo + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.f;
    if (M != -INFINITY)
      for (int i = lane; i < nrows; i += 32) {
        const float mw = row_m(warp, c_lo + i);
        if (mw != -INFINITY)
          L += a.rows[((int64_t)(c_lo + i + u) * 8 + warp) * (DH + 2) + 1] * exp2f(mw - M);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (lane == 0) { s_M[warp] = M; s_L[warp] = L; }
  }
  __syncthreads();
  // page-importance EMA (_omega_ema_eager, spherical_kv_pipeline.py:952-987) from the per-tile
  // (max, sum) the split-K kernel left in page_ml: per query head the block weights
  // exp(max(m - m_max, -60)) * l are normalised over the blocks, averaged over the heads of
  // this KV head and blended into omega.  m_max is the head's global maximum found above, and
  // the normaliser (the sum of the weights over all blocks) is the head's global sum: both
  // are sums of the same exp(logit - m_max) terms, so no second pass over the blocks is needed
  // (the -60 clamp changes terms below e^-60 of the largest one).
  if (p.omega != nullptr) {
    const int tpp = p.page_size >> 4;
    const int unit = b * p.Hkv + hkv;
    const int nb = min(p.num_blocks[unit], p.max_blocks);
    const int32_t* bt = p.block_table + (int64_t)unit * p.max_blocks;
    const float one_minus = (1.0f - p.ema_beta) / (float)a.grp;
    // blocks are spread over gridDim.y CTAs of this unit; each repeats the cheap pass 1
    for (int blk = blockIdx.y * blockDim.x + threadIdx.x; blk < p.max_blocks; blk += gridDim.y * blockDim.x) {
      float mass = 0.f;
      if (blk < nb && bt[blk] >= 0) {
        for (int n = 0; n < a.grp; ++n) {
          const float* t = p.page_ml +
                           (((int64_t)b * p.Hq + (int64_t)hkv * a.grp + n) * p.max_blocks + blk) * tpp * 2;
          float m = -INFINITY;
          for (int i = 0; i < tpp; ++i)
            if (t[2 * i + 1] > 0.f) m = fmaxf(m, t[2 * i]);
          if (m == -INFINITY) continue;
          float l = 0.f;
          for (int i = 0; i < tpp; ++i)
            if (t[2 * i + 1] > 0.f) l += t[2 * i + 1] * __expf(t[2 * i] - m);
          mass += __expf(fmaxf(m - s_M[n] * kLn2, -60.f)) * l / fmaxf(s_L[n], 1e-12f);
        }
      }
      float* o = p.omega + (int64_t)unit * p.max_blocks + blk;
      *o = *o * p.ema_beta + mass * one_minus;
    }
  }
  if (blockIdx.y != 0) return;  // only the first CTA of a unit writes the attention output
  // pass 2: weights per chunk of rows, then threads over (head, dim)
  float o_acc[(8 * DH + 255) / 256];
#pragma unroll
  for (int q = 0; q < (8 * DH + 255) / 256; ++q) o_acc[q] = 0.f;
  for (int c0 = 0; c0 < nrows; c0 += kChunk) {
    const int nc = min(kChunk, nrows - c0);
    for (int i = threadIdx.x; i < a.grp * nc; i += blockDim.x) {
      const int n = i / nc, ci = i - n * nc;
      const float mw = row_m(n, c_lo + c0 + ci);
      s_w[n][ci] = (mw == -INFINITY || s_M[n] == -INFINITY) ? 0.f : exp2f(mw - s_M[n]);
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < (8 * DH + 255) / 256; ++q) {
      const int i = threadIdx.x + q * 256;
      const int n = i / DH, d = i - n * DH;
      if (n < a.grp) {
        float o = o_acc[q];
        for (int ci = 0; ci < nc; ++ci) {
          const float w = s_w[n][ci];
          if (w != 0.f) o += w * a.rows[((int64_t)(c_lo + c0 + ci + u) * 8 + n) * (DH + 2) + 2 + d];
        }
        o_acc[q] = o;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int q = 0; q < (8 * DH + 255) / 256; ++q) {
    const int i = threadIdx.x + q * 256;
    const int n = i / DH, d = i - n * DH;
    if (n >= a.grp) continue;
    const float M = s_M[n], l = s_L[n], o = o_acc[q];
    const int64_t hq = (int64_t)b * p.Hq + (int64_t)hkv * a.grp + n;
    if (p.out_partial != nullptr) {
      float* dst = p.out_partial + hq * (DH + 2);
      if (d == 0) {
        dst[0] = M * kLn2;
        dst[1] = l;
      }
      dst[2 + d] = o;
    }
    if (p.out != nullptr) store_from_float(p.out, p.out_dtype, hq * DH + d, l > 0.f ? o / l : 0.f);
  }
}

// ---- merge of R partial sets (cross-GPU split-KV) ----------------------------------------
__global__ void merge_partials_kernel(const float* __restrict__ parts, int R, int n_rows, int dh,
                                      void* __restrict__ out, int out_dtype) {
  const int row = blockIdx.x;
  const int64_t stride = (int64_t)n_rows * (dh + 2);
  float M = -INFINITY;
  for (int rr = 0; rr < R; ++rr) {
    const float* pr = parts + rr * stride + (int64_t)row * (dh + 2);
    if (pr[1] > 0.f) M = fmaxf(M, pr[0]);
  }
  for (int d = threadIdx.x; d < dh; d += blockDim.x) {
    float l = 0.f, o = 0.f;
    if (M != -INFINITY) {
      for (int rr = 0; rr < R; ++rr) {
        const float* pr = parts + rr * stride + (int64_t)row * (dh + 2);
        if (!(pr[1] > 0.f)) continue;
        const float w = __expf(pr[0] - M);
        l += pr[1] * w;
        o += pr[2 + d] * w;
      }
    }
    store_from_float(out, out_dtype, (int64_t)row * dh + d, l > 0.f ? o / l : 0.f);
  }
}

// ---- host side --------------------------------------------------------------------------------
static int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

static int smem_cb_layout(const sphkv_tiers& t, int dh, int* offs) {
  int off = 0;
  for (int s = 0; s < t.n_slots; ++s) {
    offs[s] = off;
    off += dh * (1 << t.bits[s]) * 4 * (kCbPitch / 64);
  }
  return off;
}

int validate_tiers(const sphkv_tiers& t, int dh) {
  SPHKV_REQUIRE(t.n_slots >= 1 && t.n_slots <= SPHKV_MAX_TIER_SLOTS, SPHKV_E_ARG,
                "tiers.n_slots=%d outside 1..%d", t.n_slots, SPHKV_MAX_TIER_SLOTS);
  for (int s = 0; s < t.n_slots; ++s) {
    SPHKV_REQUIRE(t.g[s] == 16 || t.g[s] == 32, SPHKV_E_ARG, "tier slot %d: g=%d (16 or 32)", s,
                  t.g[s]);
    SPHKV_REQUIRE(t.bits[s] >= 1 && t.bits[s] <= 6, SPHKV_E_ARG, "tier slot %d: bits=%d (1..6)", s,
                  t.bits[s]);
    SPHKV_REQUIRE(dh % (2 * t.g[s]) == 0, SPHKV_E_ARG, "tier slot %d: dh=%d not a multiple of 2g",
                  s, dh);
    SPHKV_REQUIRE(dh / t.g[s] <= t.G_max && (1 << t.bits[s]) <= t.C_max && t.g[s] <= t.g_max,
                  SPHKV_E_ARG, "tier slot %d exceeds codebook tensor (G_max=%d C_max=%d g_max=%d)",
                  s, t.G_max, t.C_max, t.g_max);
  }
  return 0;
}

template <int DH, typename VT, bool ROT, bool EXTRA, bool PACK>
static int launch_decode_t(const DecodeArgs& a, int smem_bytes, cudaStream_t st) {
  static int configured_for = -1;
  auto kern = decode_splitk_kernel<DH, VT, ROT, EXTRA, PACK>;
  if (configured_for < smem_bytes) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(decode, %d B): %s", smem_bytes, cudaGetErrorString(e));
      return (int)e;
    }
    // Ask for the smallest shared-memory carve-out that holds this CTA (plus the 1 KB the system
    // reserves): what is left of the 256 KB array is L1, which serves the cos/sin table rows.
    // The hint is a percentage of 228 KB that the driver rounds UP to a supported size, so it is
    // rounded down here (the driver never goes below what the launch needs).
    cudaFuncAttributes fa;
    const int64_t stat = cudaFuncGetAttributes(&fa, kern) == cudaSuccess ? (int64_t)fa.sharedSizeBytes : 0;
    const int pct = (int)(((int64_t)smem_bytes + stat + 1024) * 100 / (228 * 1024));
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, pct > 100 ? 100 : pct);
    configured_for = smem_bytes;
  }
  kern<<<a.n_ctas, kWarps * 32, smem_bytes, st>>>(a);
  return check_launch("decode_splitk_kernel");
}

template <int DH, typename VT, bool ROT>
static int launch_decode_r(const DecodeArgs& a, int smem_bytes, cudaStream_t st) {
  const bool extra = a.p.logits_out != nullptr || a.p.page_ml != nullptr;
  const bool pack = a.grp <= 4;
  if (extra) return pack ? launch_decode_t<DH, VT, ROT, true, true>(a, smem_bytes, st)
                         : launch_decode_t<DH, VT, ROT, true, false>(a, smem_bytes, st);
  return pack ? launch_decode_t<DH, VT, ROT, false, true>(a, smem_bytes, st)
              : launch_decode_t<DH, VT, ROT, false, false>(a, smem_bytes, st);
}

template <int DH, typename VT>
static int launch_decode(const DecodeArgs& a, int smem_bytes, cudaStream_t st) {
  return a.p.rope_table != nullptr ? launch_decode_r<DH, VT, true>(a, smem_bytes, st)
                                   : launch_decode_r<DH, VT, false>(a, smem_bytes, st);
}

}  // namespace sphkv

using namespace sphkv;

extern "C" int sphkv_sm_count(void) {
  int dev = 0, n = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) {
    set_error("sm_count: %s", cudaGetErrorString(e));
    return -(int)e;
  }
  return n;
}

static int resolve_ctas(int n_ctas) {
  if (n_ctas > 0) return n_ctas;
  static int cached = 0;
  if (cached <= 0) cached = sphkv_sm_count();
  return cached;
}

extern "C" int64_t sphkv_decode_scratch_bytes(int32_t B, int32_t Hkv, int32_t dh, int32_t n_ctas) {
  n_ctas = resolve_ctas(n_ctas);
  if (n_ctas <= 0 || B <= 0 || Hkv <= 0 || dh <= 0) return SPHKV_E_ARG;
  const int64_t n_units = (int64_t)B * Hkv;
  return align_up((n_units + 1) * 4, 256) + (int64_t)(n_ctas + n_units) * 8 * (dh + 2) * 4;
}

extern "C" int sphkv_decode_paged(const sphkv_decode_params* pp, void* stream) {
  SPHKV_REQUIRE(pp != nullptr, SPHKV_E_ARG, "decode: params is NULL");
  const sphkv_decode_params& p = *pp;
  SPHKV_REQUIRE(p.q && p.k_pages && p.ptable && p.v_pool && p.block_table && p.bits_table &&
                    p.num_blocks && p.codebooks && p.scratch,
                SPHKV_E_ARG, "decode: a required pointer is NULL");
  SPHKV_REQUIRE(p.out || p.out_partial, SPHKV_E_ARG, "decode: out and out_partial both NULL");
  SPHKV_REQUIRE(p.rope_table == nullptr || p.positions != nullptr, SPHKV_E_ARG,
                "decode: rope_table given without positions");
  SPHKV_REQUIRE(p.omega == nullptr || p.page_ml != nullptr, SPHKV_E_ARG,
                "decode: omega needs page_ml (the per-tile statistics it is computed from)");
  SPHKV_REQUIRE(p.dh == 64 || p.dh == 128, SPHKV_E_ARG, "decode: dh=%d (64 or 128)", p.dh);
  SPHKV_REQUIRE(p.B > 0 && p.Hkv > 0 && p.Hq > 0 && p.Hq % p.Hkv == 0, SPHKV_E_ARG,
                "decode: B=%d Hq=%d Hkv=%d", p.B, p.Hq, p.Hkv);
  const int grp = p.Hq / p.Hkv;
  SPHKV_REQUIRE(grp <= SPHKV_MAX_GQA, SPHKV_E_LIMIT, "decode: %d query heads per KV head (max %d)",
                grp, SPHKV_MAX_GQA);
  SPHKV_REQUIRE(p.page_size == 16 || p.page_size == 32 || p.page_size == 64 || p.page_size == 128,
                SPHKV_E_ARG, "decode: page_size=%d (16, 32, 64 or 128)", p.page_size);
  SPHKV_REQUIRE(p.max_blocks > 0 && p.n_pages > 0, SPHKV_E_ARG, "decode: max_blocks=%d n_pages=%d",
                p.max_blocks, p.n_pages);
  SPHKV_REQUIRE(p.v_dtype == SPHKV_F16 || p.v_dtype == SPHKV_BF16, SPHKV_E_DTYPE,
                "decode: v_dtype=%d", p.v_dtype);
  SPHKV_REQUIRE(p.q_dtype >= 0 && p.q_dtype <= 2 && p.out_dtype >= 0 && p.out_dtype <= 2,
                SPHKV_E_DTYPE, "decode: q_dtype=%d out_dtype=%d", p.q_dtype, p.out_dtype);
  SPHKV_REQUIRE(p.radius_fmt == SPHKV_RADIUS_I8 || p.radius_fmt == SPHKV_RADIUS_F16, SPHKV_E_ARG,
                "decode: radius_fmt=%d", p.radius_fmt);
  SPHKV_REQUIRE(((uintptr_t)p.v_pool & 15) == 0 && ((uintptr_t)p.k_pages & 3) == 0 &&
                    ((uintptr_t)p.codebooks & 15) == 0 && (p.tiers.g_max & 3) == 0 &&
                    (p.rope_table == nullptr || ((uintptr_t)p.rope_table & 15) == 0) &&
                    ((uintptr_t)p.scratch & 255) == 0,
                SPHKV_E_ALIGN, "decode: v_pool/rope_table/codebooks need 16 B, k_pages 4 B, scratch 256 B");
  if (int rc = validate_tiers(p.tiers, p.dh)) return rc;

  DecodeArgs a;
  a.p = p;
  a.n_ctas = resolve_ctas(p.n_ctas);
  SPHKV_REQUIRE(a.n_ctas > 0, SPHKV_E_ARG, "decode: cannot resolve CTA count");
  a.n_units = p.B * p.Hkv;
  a.grp = grp;
  const int64_t need = sphkv_decode_scratch_bytes(p.B, p.Hkv, p.dh, a.n_ctas);
  SPHKV_REQUIRE(p.scratch_bytes >= need, SPHKV_E_SCRATCH, "decode: scratch %lld B < %lld B",
                (long long)p.scratch_bytes, (long long)need);
  a.pfx = reinterpret_cast<int32_t*>(p.scratch);
  a.rows = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.scratch) +
                                    align_up((int64_t)(a.n_units + 1) * 4, 256));
  a.cb_smem_bytes = smem_cb_layout(p.tiers, p.dh, a.cb_smem_off);
  a.plan_in_kernel = a.n_units <= kMaxUnitsInKernelPlan ? 1 : 0;
  const int smem_bytes = smem_v_bytes(p.dh) + a.cb_smem_bytes + smem_q_bytes(p.dh, a.grp <= 4) +
                         kWarps * smem_priv_bytes(p.dh) +
                         (a.plan_in_kernel ? (a.n_units + 1) * 4 : 0);
  SPHKV_REQUIRE(smem_bytes <= 227 * 1024, SPHKV_E_LIMIT,
                "decode: codebooks need %d B of shared memory (limit %d)", smem_bytes, 227 * 1024);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  if (!a.plan_in_kernel) {
    plan_kernel<<<1, 1024, 0, st>>>(p.num_blocks, a.n_units, p.max_blocks, p.B, p.Hkv, a.pfx);
    if (int rc = check_launch("plan_kernel")) return rc;
  }
  int rc;
  if (p.dh == 128)
    rc = p.v_dtype == SPHKV_F16 ? launch_decode<128, __half>(a, smem_bytes, st)
                                : launch_decode<128, __nv_bfloat16>(a, smem_bytes, st);
  else
    rc = p.v_dtype == SPHKV_F16 ? launch_decode<64, __half>(a, smem_bytes, st)
                                : launch_decode<64, __nv_bfloat16>(a, smem_bytes, st);
  if (rc) return rc;
  // with an importance update, extra CTAs per unit share the walk over the blocks
  const dim3 mgrid(a.n_units, p.omega ? (unsigned)min(16, (p.max_blocks + 255) / 256) : 1u);
  if (p.dh == 128)
    merge_rows_kernel<128><<<mgrid, 256, 0, st>>>(a);
  else
    merge_rows_kernel<64><<<mgrid, 256, 0, st>>>(a);
  return check_launch("merge_rows_kernel");
}

extern "C" int sphkv_merge_partials(const float* parts, int32_t R, int32_t n_rows, int32_t dh,
                                    void* out, int32_t out_dtype, void* stream) {
  SPHKV_REQUIRE(parts && out, SPHKV_E_ARG, "merge: NULL pointer");
  SPHKV_REQUIRE(R > 0 && n_rows > 0 && dh > 0, SPHKV_E_ARG, "merge: R=%d n_rows=%d dh=%d", R,
                n_rows, dh);
  SPHKV_REQUIRE(out_dtype >= 0 && out_dtype <= 2, SPHKV_E_DTYPE, "merge: out_dtype=%d", out_dtype);
  merge_partials_kernel<<<n_rows, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      parts, R, n_rows, dh, out, out_dtype);
  return check_launch("merge_partials_kernel");
}

// ---- decode without any caller- or library-side allocation -------------------------------
// Some hosts of this library cannot hand it scratch memory: an inference server that gave
// its whole HBM budget to the KV pools at start-up has nothing left for cudaMalloc to
// return, and a plug-in loaded into such a process has no allocator of its own to ask.  For
// them the split-K scratch of the decode kernels lives in the library image.
//
// Limits (the array is sized for them; every GPU that loads the library carries it until
// the process exits): B * Hkv <= 256 units, at most 160 CTAs, dh <= 128.
#define SPHKV_STATIC_MAX_UNITS 256
#define SPHKV_STATIC_MAX_CTAS 160
#define SPHKV_STATIC_SCRATCH_BYTES \
  (((SPHKV_STATIC_MAX_UNITS + 1) * 4 + 255) / 256 * 256 + \
   (SPHKV_STATIC_MAX_CTAS + SPHKV_STATIC_MAX_UNITS) * 8 * (128 + 2) * 4)
static __device__ __align__(256) unsigned char g_static_scratch[SPHKV_STATIC_SCRATCH_BYTES];

// g_static_scratch names a host-side handle here, not a device address; the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device
// current.
static void* static_scratch_for_current_device(int* rc_out) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("decode_static: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    *rc_out = e != cudaSuccess ? (int)e : SPHKV_E_LIMIT;
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      *rc_out = e != cudaSuccess ? (int)e : SPHKV_E_ARG;
      return nullptr;
    }
    cached[dev] = ptr;
  }
  *rc_out = 0;
  return cached[dev];
}

extern "C" int sphkv_decode_paged_static(const sphkv_decode_params* pp, void* stream) {
  SPHKV_REQUIRE(pp != nullptr, SPHKV_E_ARG, "decode_static: params is NULL");
  SPHKV_REQUIRE(pp->B > 0 && pp->Hkv > 0 && (int64_t)pp->B * pp->Hkv <= SPHKV_STATIC_MAX_UNITS,
                SPHKV_E_LIMIT, "decode_static: B*Hkv=%lld exceeds the built-in scratch (max %d units)",
                (long long)pp->B * pp->Hkv, SPHKV_STATIC_MAX_UNITS);
  SPHKV_REQUIRE(pp->dh > 0 && pp->dh <= 128, SPHKV_E_LIMIT,
                "decode_static: dh=%d exceeds the built-in scratch (max 128)", pp->dh);
  const int n_ctas = resolve_ctas(pp->n_ctas);
  SPHKV_REQUIRE(n_ctas > 0 && n_ctas <= SPHKV_STATIC_MAX_CTAS, SPHKV_E_LIMIT,
                "decode_static: %d CTAs exceed the built-in scratch (max %d); pass n_ctas", n_ctas,
                SPHKV_STATIC_MAX_CTAS);
  int rc = 0;
  void* scratch = static_scratch_for_current_device(&rc);
  if (scratch == nullptr) return rc;
  sphkv_decode_params q = *pp;
  q.n_ctas = n_ctas;
  q.scratch = scratch;
  q.scratch_bytes = SPHKV_STATIC_SCRATCH_BYTES;
  return sphkv_decode_paged(&q, stream);
}
