// Angle-domain decode attention over bit-packed, paged, codebook-quantised keys.
//
// One persistent CTA per SM walks a contiguous range of (batch row, KV head) blocks.
// Each warp owns every WARPS-th 16-token tile of the range and keeps an online-softmax
// state for all query heads of the KV head.  Per tile a warp
//   1. unpacks the tile's centroid indices and radii (lane = token x half of groups),
//   2. rebuilds the 16 x dh key tile directly in mma A-fragment registers: gathers the
//      selected centroid rows from shared memory, scales by the radius and rotates by
//      the key's RoPE angle (cos/sin row of the key position, read through L2),
//   3. forms logits with fp16 hi/lo split operands on the tensor cores
//      (tokens x dh) * (dh x heads), fp32 accumulate,
//   4. runs the online softmax and accumulates P^T V with V tiles that cp.async streams
//      into a swizzled shared-memory ring.
// Warp states are merged per CTA, CTA partials land in scratch, and a small kernel
// merges them by log-sum-exp.
//
// Numerics restate SphericalKVPipeline._compressed_head_attention_batched
// (spherical_kv_pipeline.py:2136-2177): logit = sum_g r_g * (q_rot_g . c_g) / sqrt(dh)
// with q back-rotated by the key position; rotating the rebuilt key forward instead
// is the same bilinear form.  Page bytes follow pagebuilder.py:8-33 / paging.py:20-31.
#include <stdarg.h>
#include <type_traits>
#include <stdio.h>

#include "common.cuh"

namespace sphkv {

constexpr int kWarps = 8;
constexpr int kVStages = 3;
constexpr int kMetaRing = 64;

struct TileMeta {  // 32 bytes
  int phys;        // physical page id, <0 = nothing to do
  int slot;        // tier slot
  int poff, toff, roff;
  int count;       // tokens in the page
  int sub;         // 16-token tile index inside the page
  int lb;          // logical block index inside the unit
};

struct DecodeArgs {
  sphkv_decode_params p;
  int cb_smem_off[SPHKV_MAX_TIER_SLOTS];  // byte offset of each slot's codebook in smem
  int cb_smem_bytes;
  int n_units;
  int n_ctas;
  int grp;
  int32_t* pfx;
  float* rows;  // [(n_ctas + n_units)][8][dh + 2]
};

// ---- plan: exclusive prefix of blocks per unit --------------------------------------
__global__ void plan_kernel(const int32_t* __restrict__ num_blocks, int n_units, int max_blocks,
                            int32_t* __restrict__ pfx) {
  __shared__ int s_part[32];
  __shared__ int s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < n_units; base += blockDim.x) {
    int i = base + threadIdx.x;
    int v = 0;
    if (i < n_units) {
      v = num_blocks[i];
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

template <int DH>
struct KWords {
  uint32_t th0, th1;       // aligned words holding this lane's theta bits
  uint32_t rd0, rd1, rd2;  // aligned words holding this lane's radius bytes
  float sc[4];             // per-group scales of this lane's groups
  int th_sh, rd_sh;        // bit shifts into the funnels
  int pos0, pos1;          // key positions of rows (lane>>2) and (lane>>2)+8
};

template <int DH, typename VT>
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

  uint8_t* v_ring = smem + warp * V_WARP;
  uint8_t* cb_smem = smem + kWarps * V_WARP;
  uint8_t* warp_priv = cb_smem + a.cb_smem_bytes + warp * (16 * KS * 8 + 512 + kMetaRing * 32);
  uint2* unp = reinterpret_cast<uint2*>(warp_priv);                       // [16][KS]
  uint16_t* pbuf = reinterpret_cast<uint16_t*>(warp_priv + 16 * KS * 8);  // [2][8][16]
  TileMeta* meta = reinterpret_cast<TileMeta*>(warp_priv + 16 * KS * 8 + 512);

  const int32_t* __restrict__ pfx = a.pfx;
  const int64_t T = pfx[a.n_units];
  if (T == 0) return;
  int64_t start = cta_range_start(blockIdx.x, a.n_ctas, T);
  const int64_t end = cta_range_start(blockIdx.x + 1, a.n_ctas, T);
  if (start >= end) return;
  int u = find_unit(pfx, a.n_units, start);

  const int N = p.page_size;
  const int TPP = N >> 4;
  const bool rot = p.rope_table != nullptr;
  const float qscale = p.sm_scale * kLog2e;
  int cb_head_loaded = -1;

  while (start < end) {
    while ((int64_t)pfx[u + 1] <= start) ++u;  // skip units without blocks
    const int64_t seg_end = end < (int64_t)pfx[u + 1] ? end : (int64_t)pfx[u + 1];
    const int lb0 = (int)(start - pfx[u]);
    const int seg_tiles = (int)(seg_end - start) * TPP;
    const int b = u / p.Hkv, hkv = u - b * p.Hkv;

    // ---- stage this KV head's codebooks (permuted for lane-quad float4 reads) ----
    __syncthreads();
    if (hkv != cb_head_loaded) {
      const sphkv_tiers& tg = p.tiers;
      for (int s = 0; s < tg.n_slots; ++s) {
        const int g = tg.g[s], C = 1 << tg.bits[s], G = DH / g, spg = g >> 4;
        const float* src =
            p.codebooks + ((int64_t)(hkv * tg.n_slots + s) * tg.G_max) * tg.C_max * tg.g_max;
        float* dst = reinterpret_cast<float*>(cb_smem + a.cb_smem_off[s]);
        const int total = G * C * g;
        for (int i = threadIdx.x; i < total; i += blockDim.x) {
          const int e = i & 3, jj = (i >> 2) & 3, row = i >> 4;
          const int sub2 = row % spg, gc = row / spg;
          const int c = gc % C, gam = gc / C;
          const int d = sub2 * 16 + 2 * jj + (e & 1) + ((e >> 1) << 3);
          dst[i] = src[((int64_t)gam * tg.C_max + c) * tg.g_max + d];
        }
      }
      cb_head_loaded = hkv;
    }
    __syncthreads();

    // ---- query fragments: B operand [k = dim][n = head], fp16 hi/lo, pre-scaled ----
    uint32_t qhi[KS][2], qlo[KS][2];
    {
      const int n = r;  // head column of this lane
      const bool real = n < a.grp;
      const int64_t qbase = ((int64_t)b * p.Hq + (int64_t)hkv * a.grp + n) * DH;
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int d = 16 * s + 2 * j + (e & 1) + ((e >> 1) << 3);
          v[e] = real ? load_as_float(p.q, p.q_dtype, qbase + d) * qscale : 0.f;
        }
        split_f16x2(v[0], v[1], qhi[s][0], qlo[s][0]);
        split_f16x2(v[2], v[3], qhi[s][1], qlo[s][1]);
      }
    }

    const int nt = seg_tiles > warp ? (seg_tiles - warp + kWarps - 1) / kWarps : 0;
    const int32_t* bt_row = p.block_table + (int64_t)u * p.max_blocks;
    const int32_t* st_row = p.bits_table + (int64_t)u * p.max_blocks;

    auto meta_fill = [&](int kbase) {
      const int kk = kbase + lane;
      TileMeta m;
      m.phys = -2; m.slot = 0; m.poff = m.toff = m.roff = 0; m.count = 0; m.sub = 0; m.lb = 0;
      if (kk < nt) {
        const int ti = warp + kWarps * kk;
        m.lb = lb0 + ti / TPP;
        m.sub = ti - (ti / TPP) * TPP;
        int phys = bt_row[m.lb];
        int slot = st_row[m.lb];
        if (phys >= p.n_pages) {
          if (p.status) atomicOr(p.status, SPHKV_ST_BAD_BLOCK);
          phys = -1;
        }
        if (slot < 0 || slot >= p.tiers.n_slots) {
          if (p.status) atomicOr(p.status, SPHKV_ST_BAD_SLOT);
          phys = -1;
          slot = 0;
        }
        m.slot = slot;
        if (phys >= 0) {
          m.poff = p.ptable[3 * (int64_t)phys + 0];
          m.toff = p.ptable[3 * (int64_t)phys + 1];
          m.roff = p.ptable[3 * (int64_t)phys + 2];
          const uint32_t hdr = *reinterpret_cast<const uint32_t*>(p.k_pages + m.poff);
          m.count = (int)((hdr >> 8) & 0xFFu);
          if (m.count > N) m.count = N;
        }
        m.phys = phys < 0 ? -1 : phys;
      }
      meta[kk & (kMetaRing - 1)] = m;
    };

    auto issue_v = [&](int kk) {
      if (kk < nt) {
        const TileMeta m = meta[kk & (kMetaRing - 1)];
        if (m.phys >= 0) {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.v_pool) +
                               ((int64_t)m.phys * N + 16 * m.sub) * DH * 2;
          const uint32_t dst = smem_u32(v_ring + (kk % kVStages) * V_TILE);
#pragma unroll
          for (int q = 0; q < (16 * DH / 8) / 32; ++q) {
            const int i = lane + 32 * q;
            const int tau = i / (DH / 8), c = i % (DH / 8);
            const uint32_t d =
                dst + (c >> 3) * 2048 + tau * 128 + (((c & 7) ^ (tau & 7)) << 4);
            cp_async_16(d, src + ((int64_t)tau * DH + c * 8) * 2);
          }
        }
      }
      cp_async_commit();
    };

    // lane = (token t = lane>>1, half = lane&1) for the unpack role
    const int ut = lane >> 1, uhalf = lane & 1;

    auto load_kwords = [&](int kk, KWords<DH>& w) {
      w.th0 = w.th1 = w.rd0 = w.rd1 = w.rd2 = 0u;
      w.th_sh = w.rd_sh = 0;
      w.pos0 = w.pos1 = -1;
#pragma unroll
      for (int i = 0; i < 4; ++i) w.sc[i] = 0.f;
      if (kk >= nt) return;
      const TileMeta m = meta[kk & (kMetaRing - 1)];
      if (m.phys < 0) return;
      const int g = p.tiers.g[m.slot], bits = p.tiers.bits[m.slot];
      const int G = DH / g, spg = g >> 4, ng = HS / spg, gam0 = uhalf * ng;
      const int tp = 16 * m.sub + ut;
      if (tp < m.count) {
        const int64_t bit = ((int64_t)tp * G + gam0) * bits;
        const int64_t ba = (int64_t)m.toff + (bit >> 3);
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(p.k_pages + (ba & ~3LL));
        w.th_sh = (int)((ba & 3) * 8 + (bit & 7));
        w.th0 = wp[0];
        if (w.th_sh + ng * bits > 32) w.th1 = wp[1];
        const int rb = p.radius_fmt == SPHKV_RADIUS_F16 ? 2 : 1;
        const int64_t ra = (int64_t)m.roff + ((int64_t)tp * G + gam0) * rb;
        const uint32_t* rp = reinterpret_cast<const uint32_t*>(p.k_pages + (ra & ~3LL));
        w.rd_sh = (int)((ra & 3) * 8);
        const int need = (int)(ra & 3) + ng * rb;  // bytes from the aligned word start
        w.rd0 = rp[0];
        if (need > 4) w.rd1 = rp[1];
        if (need > 8) w.rd2 = rp[2];
        const float* sp = reinterpret_cast<const float*>(p.k_pages + m.poff + 8) + gam0;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < ng) w.sc[i] = sp[i];
      }
      if (rot) {
        const int32_t* pp = p.positions + (int64_t)m.phys * N + 16 * m.sub;
        w.pos0 = pp[r];
        w.pos1 = pp[r + 8];
      }
    };

    float4 cs[2][HS][2];
    auto issue_cs = [&](const KWords<DH>& w) {
      if (!rot) return;
#pragma unroll
      for (int tk = 0; tk < 2; ++tk) {
        int pos = tk ? w.pos1 : w.pos0;
        if (pos >= p.max_pos) {
          if (p.status) atomicOr(p.status, SPHKV_ST_BAD_POSITION);
          pos = 0;
        }
        if (pos < 0) pos = 0;
        const float4* rp = reinterpret_cast<const float4*>(p.rope_table + (int64_t)pos * DH) + j * 2;
#pragma unroll
        for (int s = 0; s < HS; ++s) {
          cs[tk][s][0] = __ldg(rp + s * 8);
          cs[tk][s][1] = __ldg(rp + s * 8 + 1);
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

    // ---- prologue -------------------------------------------------------------------
    meta_fill(0);
    meta_fill(32);
    __syncwarp();
    issue_v(0);
    issue_v(1);
    KWords<DH> cur, nx;
    load_kwords(0, cur);
    issue_cs(cur);

    for (int k = 0; k < nt; ++k) {
      if (k > 0 && (k & 31) == 0) {
        meta_fill(k + 32);
        __syncwarp();
      }
      issue_v(k + 2);
      load_kwords(k + 1, nx);
      const TileMeta m = meta[k & (kMetaRing - 1)];
      const int cnt_tile = m.phys < 0 ? 0 : min(16, max(0, m.count - 16 * m.sub));

      if (cnt_tile > 0) {
        // ---- phase A: unpack codes/radii of (token ut, half uhalf) ------------------
        {
          const int g = p.tiers.g[m.slot], bits = p.tiers.bits[m.slot];
          const int C = 1 << bits, spg = g >> 4, ng = HS / spg, gam0 = uhalf * ng;
          const uint32_t cbase = (uint32_t)a.cb_smem_off[m.slot];
          const uint32_t tb = __funnelshift_r(cur.th0, cur.th1, cur.th_sh);
          const uint32_t rlo = __funnelshift_r(cur.rd0, cur.rd1, cur.rd_sh);
          const uint32_t rhi = __funnelshift_r(cur.rd1, cur.rd2, cur.rd_sh);
          const bool tok_ok = (16 * m.sub + ut) < m.count;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (i < ng) {
              const int code = (int)((tb >> (i * bits)) & (uint32_t)(C - 1));
              float rad;
              if (p.radius_fmt == SPHKV_RADIUS_F16) {
                const uint32_t wv = (i < 2) ? rlo : rhi;
                const uint16_t hv = (uint16_t)(wv >> ((i & 1) * 16));
                rad = __half2float(__ushort_as_half(hv));
              } else {
                const int c8 = (int)(int8_t)((rlo >> (i * 8)) & 0xFFu);
                rad = (cur.sc[i] * (float)c8) * (1.0f / 127.0f);
              }
              if (!tok_ok) rad = 0.f;
              const int gam = gam0 + i;
#pragma unroll
              for (int s2 = 0; s2 < 2; ++s2) {
                if (s2 < spg) {
                  const uint32_t off = cbase + (uint32_t)(((gam * C + code) * spg + s2) * 64);
                  unp[ut * KS + gam * spg + s2] = make_uint2(off, __float_as_uint(rad));
                }
              }
            }
          }
        }
        __syncwarp();

        // ---- phase B: rebuild rotated key tile in A fragments, QK^T on tensor cores -
        float s_hh[4] = {0.f, 0.f, 0.f, 0.f}, s_lh[4] = {0.f, 0.f, 0.f, 0.f},
              s_hl[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < HS; ++s) {
          uint32_t a_lo_hi[4], a_lo_lo[4], a_hi_hi[4], a_hi_lo[4];
#pragma unroll
          for (int tk = 0; tk < 2; ++tk) {
            const int tau = r + 8 * tk;
            const uint2 e0 = unp[tau * KS + s];
            const uint2 e1 = unp[tau * KS + s + HS];
            float4 x = *reinterpret_cast<const float4*>(cb_smem + e0.x + j * 16);
            float4 y = *reinterpret_cast<const float4*>(cb_smem + e1.x + j * 16);
            const float r0 = __uint_as_float(e0.y), r1 = __uint_as_float(e1.y);
            x.x *= r0; x.y *= r0; x.z *= r0; x.w *= r0;
            y.x *= r1; y.y *= r1; y.z *= r1; y.w *= r1;
            float4 lo = x, hi = y;
            if (rot) {
              const float4 c = cs[tk][s][0], sn = cs[tk][s][1];
              lo.x = x.x * c.x - y.x * sn.x; hi.x = y.x * c.x + x.x * sn.x;
              lo.y = x.y * c.y - y.y * sn.y; hi.y = y.y * c.y + x.y * sn.y;
              lo.z = x.z * c.z - y.z * sn.z; hi.z = y.z * c.z + x.z * sn.z;
              lo.w = x.w * c.w - y.w * sn.w; hi.w = y.w * c.w + x.w * sn.w;
            }
            split_f16x2(lo.x, lo.y, a_lo_hi[tk], a_lo_lo[tk]);
            split_f16x2(lo.z, lo.w, a_lo_hi[2 + tk], a_lo_lo[2 + tk]);
            split_f16x2(hi.x, hi.y, a_hi_hi[tk], a_hi_lo[tk]);
            split_f16x2(hi.z, hi.w, a_hi_hi[2 + tk], a_hi_lo[2 + tk]);
          }
          mma_f16_16816(s_hh, a_lo_hi, qhi[s][0], qhi[s][1]);
          mma_f16_16816(s_lh, a_lo_lo, qhi[s][0], qhi[s][1]);
          mma_f16_16816(s_hl, a_lo_hi, qlo[s][0], qlo[s][1]);
          mma_f16_16816(s_hh, a_hi_hi, qhi[s + HS][0], qhi[s + HS][1]);
          mma_f16_16816(s_lh, a_hi_lo, qhi[s + HS][0], qhi[s + HS][1]);
          mma_f16_16816(s_hl, a_hi_hi, qlo[s + HS][0], qlo[s + HS][1]);
        }
        // the cos/sin registers are free now: fetch the next tile's rows
        issue_cs(nx);

        // ---- online softmax over the 16 token rows, per head column ------------------
        float sv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) sv[e] = s_hh[e] + (s_lh[e] + s_hl[e]);
        if (p.logits_out != nullptr) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = 2 * j + (e & 1), tok = r + ((e >> 1) << 3);
            if (n < a.grp && tok < cnt_tile)
              p.logits_out[(((int64_t)b * p.Hq + (int64_t)hkv * a.grp + n) * p.max_blocks + m.lb) * N +
                           16 * m.sub + tok] = sv[e] * kLn2;
          }
        }
        const bool ok0 = r < cnt_tile && (!rot || cur.pos0 >= 0);
        const bool ok1 = (r + 8) < cnt_tile && (!rot || cur.pos1 >= 0);
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
          alpha[c] = exp2f(m_run[c] - msafe[c]);
          m_run[c] = mn;
        }
        float pv[4];
        pv[0] = exp2f(sv[0] - msafe[0]);
        pv[1] = exp2f(sv[1] - msafe[1]);
        pv[2] = exp2f(sv[2] - msafe[0]);
        pv[3] = exp2f(sv[3] - msafe[1]);
        l_run[0] = l_run[0] * alpha[0] + (pv[0] + pv[2]);
        l_run[1] = l_run[1] * alpha[1] + (pv[1] + pv[3]);
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
          for (int dt = 0; dt < KS; ++dt) {
            acc[dt][0] *= alpha[0]; acc[dt][1] *= alpha[1];
            acc[dt][2] *= alpha[0]; acc[dt][3] *= alpha[1];
          }
        }
        if (p.page_ml != nullptr && TPP == 1) {
          // per-block (max, sum) in the natural-log domain for heads 2j, 2j+1
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
              if (n < a.grp) {
                float* dst = p.page_ml +
                             (((int64_t)b * p.Hq + (int64_t)hkv * a.grp + n) * p.max_blocks + m.lb) * 2;
                const float tm = tmax[c];
                dst[0] = tm * kLn2;
                dst[1] = (tm == -INFINITY) ? 0.f : ls[c] * exp2f(msafe[c] - tm);
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
            if (kBf16) {
              const __nv_bfloat16 h = __float2bfloat16_rn(pv[e]);
              const __nv_bfloat16 l = __float2bfloat16_rn(pv[e] - __bfloat162float(h));
              ph[head * 16 + tok] = __bfloat16_as_ushort(h);
              pl[head * 16 + tok] = __bfloat16_as_ushort(l);
            } else {
              ph[head * 16 + tok] = __half_as_ushort(__float2half_rn(pv[e]));
            }
          }
        }
        cp_async_wait<2>();
        __syncwarp();
        {
          const uint32_t* ph32 = reinterpret_cast<const uint32_t*>(pbuf);
          const uint32_t b0 = ph32[(r * 16 + 2 * j) >> 1];
          const uint32_t b1 = ph32[(r * 16 + 2 * j + 8) >> 1];
          uint32_t c0 = 0, c1 = 0;
          if (kBf16) {
            c0 = ph32[(8 * 16 + r * 16 + 2 * j) >> 1];
            c1 = ph32[(8 * 16 + r * 16 + 2 * j + 8) >> 1];
          }
          // ---- acc^T[dh][head] += V^T[dh][token] P^T[token][head] ---------------------
          const uint32_t vbase = smem_u32(v_ring + (k % kVStages) * V_TILE);
          const int mi = lane >> 3;
          const int tau = (lane & 7) + ((mi >> 1) << 3);
#pragma unroll
          for (int dt = 0; dt < KS; ++dt) {
            const int c = 2 * dt + (mi & 1);
            uint32_t af[4];
            ldmatrix_x4_trans(af, vbase + (c >> 3) * 2048 + tau * 128 + (((c & 7) ^ (tau & 7)) << 4));
            if (kBf16) {
              mma_bf16_16816(acc[dt], af, b0, b1);
              mma_bf16_16816(acc[dt], af, c0, c1);
            } else {
              mma_f16_16816(acc[dt], af, b0, b1);
            }
          }
        }
        __syncwarp();
      } else {
        issue_cs(nx);
        cp_async_wait<2>();
        __syncwarp();
      }
      cur = nx;
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
              if (mw != -INFINITY) outv += wb[e] * exp2f(mw - M);
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

// ---- merge CTA partial rows per (batch row, KV head) -------------------------------------
template <int DH>
__global__ void merge_rows_kernel(const DecodeArgs a) {
  const sphkv_decode_params& p = a.p;
  const int u = blockIdx.x;
  const int b = u / p.Hkv, hkv = u - b * p.Hkv;
  const int32_t* pfx = a.pfx;
  const int64_t T = pfx[a.n_units];
  const int64_t ps = pfx[u], pe = pfx[u + 1];
  int c_lo = 0, c_hi = -1;
  if (pe > ps && T > 0) {
    c_lo = (int)((ps * a.n_ctas) / T);
    if (c_lo >= a.n_ctas) c_lo = a.n_ctas - 1;
    while (c_lo > 0 && cta_range_start(c_lo, a.n_ctas, T) > ps) --c_lo;
    while (cta_range_start(c_lo + 1, a.n_ctas, T) <= ps) ++c_lo;
    c_hi = c_lo;
    while (c_hi + 1 < a.n_ctas && cta_range_start(c_hi + 1, a.n_ctas, T) < pe) ++c_hi;
  }
  for (int i = threadIdx.x; i < a.grp * DH; i += blockDim.x) {
    const int n = i / DH, d = i - n * DH;
    float M = -INFINITY;
    for (int c = c_lo; c <= c_hi; ++c) {
      if (cta_range_start(c, a.n_ctas, T) == cta_range_start(c + 1, a.n_ctas, T)) continue;
      M = fmaxf(M, a.rows[((int64_t)(c + u) * 8 + n) * (DH + 2)]);
    }
    float l = 0.f, o = 0.f;
    if (M != -INFINITY) {
      for (int c = c_lo; c <= c_hi; ++c) {
        if (cta_range_start(c, a.n_ctas, T) == cta_range_start(c + 1, a.n_ctas, T)) continue;
        const float* row = a.rows + ((int64_t)(c + u) * 8 + n) * (DH + 2);
        const float mw = row[0];
        if (mw == -INFINITY) continue;
        const float w = exp2f(mw - M);
        l += row[1] * w;
        o += row[2 + d] * w;
      }
    }
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
    off += dh * (1 << t.bits[s]) * 4;
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

template <int DH, typename VT>
static int launch_decode(const DecodeArgs& a, int smem_bytes, cudaStream_t st) {
  static int configured_for = -1;
  auto kern = decode_splitk_kernel<DH, VT>;
  if (configured_for < smem_bytes) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(decode, %d B): %s", smem_bytes, cudaGetErrorString(e));
      return (int)e;
    }
    configured_for = smem_bytes;
  }
  kern<<<a.n_ctas, kWarps * 32, smem_bytes, st>>>(a);
  return check_launch("decode_splitk_kernel");
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
  SPHKV_REQUIRE(p.dh == 64 || p.dh == 128, SPHKV_E_ARG, "decode: dh=%d (64 or 128)", p.dh);
  SPHKV_REQUIRE(p.B > 0 && p.Hkv > 0 && p.Hq > 0 && p.Hq % p.Hkv == 0, SPHKV_E_ARG,
                "decode: B=%d Hq=%d Hkv=%d", p.B, p.Hq, p.Hkv);
  const int grp = p.Hq / p.Hkv;
  SPHKV_REQUIRE(grp <= SPHKV_MAX_GQA, SPHKV_E_LIMIT, "decode: %d query heads per KV head (max %d)",
                grp, SPHKV_MAX_GQA);
  SPHKV_REQUIRE(p.page_size >= 16 && p.page_size <= 128 && p.page_size % 16 == 0, SPHKV_E_ARG,
                "decode: page_size=%d (multiple of 16, 16..128)", p.page_size);
  SPHKV_REQUIRE(p.max_blocks > 0 && p.n_pages > 0, SPHKV_E_ARG, "decode: max_blocks=%d n_pages=%d",
                p.max_blocks, p.n_pages);
  SPHKV_REQUIRE(p.v_dtype == SPHKV_F16 || p.v_dtype == SPHKV_BF16, SPHKV_E_DTYPE,
                "decode: v_dtype=%d", p.v_dtype);
  SPHKV_REQUIRE(p.q_dtype >= 0 && p.q_dtype <= 2 && p.out_dtype >= 0 && p.out_dtype <= 2,
                SPHKV_E_DTYPE, "decode: q_dtype=%d out_dtype=%d", p.q_dtype, p.out_dtype);
  SPHKV_REQUIRE(p.radius_fmt == SPHKV_RADIUS_I8 || p.radius_fmt == SPHKV_RADIUS_F16, SPHKV_E_ARG,
                "decode: radius_fmt=%d", p.radius_fmt);
  SPHKV_REQUIRE(((uintptr_t)p.v_pool & 15) == 0 && ((uintptr_t)p.k_pages & 3) == 0 &&
                    (p.rope_table == nullptr || ((uintptr_t)p.rope_table & 15) == 0) &&
                    ((uintptr_t)p.scratch & 255) == 0,
                SPHKV_E_ALIGN, "decode: v_pool/rope_table need 16 B, k_pages 4 B, scratch 256 B");
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
  const int ks = p.dh / 16;
  const int smem_bytes = kWarps * kVStages * 16 * p.dh * 2 + a.cb_smem_bytes +
                         kWarps * (16 * ks * 8 + 512 + kMetaRing * 32);
  SPHKV_REQUIRE(smem_bytes <= 227 * 1024, SPHKV_E_LIMIT,
                "decode: codebooks need %d B of shared memory (limit %d)", smem_bytes, 227 * 1024);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  plan_kernel<<<1, 1024, 0, st>>>(p.num_blocks, a.n_units, p.max_blocks, a.pfx);
  if (int rc = check_launch("plan_kernel")) return rc;
  int rc;
  if (p.dh == 128)
    rc = p.v_dtype == SPHKV_F16 ? launch_decode<128, __half>(a, smem_bytes, st)
                                : launch_decode<128, __nv_bfloat16>(a, smem_bytes, st);
  else
    rc = p.v_dtype == SPHKV_F16 ? launch_decode<64, __half>(a, smem_bytes, st)
                                : launch_decode<64, __nv_bfloat16>(a, smem_bytes, st);
  if (rc) return rc;
  if (p.dh == 128)
    merge_rows_kernel<128><<<a.n_units, 128, 0, st>>>(a);
  else
    merge_rows_kernel<64><<<a.n_units, 128, 0, st>>>(a);
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
