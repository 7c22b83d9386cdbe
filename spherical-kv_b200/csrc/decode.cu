// Angle-domain decode attention over bit-packed, paged, codebook-quantised keys.
//
// One persistent CTA per SM walks a contiguous range of (KV head, batch row) blocks.  Each
// warp owns every kWarps-th 16-token tile of the range and keeps an online-softmax state for
// all query heads of the KV head.
//
// Lane map of a tile (lane = 4 r + j): rows r and r + 8 are the lane's two tokens; in each
// rotary half the lane owns the contiguous block of W = dh / 8 dimensions  W j .. W j + W - 1
// and, in the other half, the same block shifted by dh / 2 -- the RoPE partner of every value
// a lane holds is in the same lane, and for g = 16, dh = 128 a lane needs exactly two centroid
// indices and two radii per token, which it extracts itself from the page bytes.  Per tile a warp
//   1. reads its code / radius words straight from the page (issued one tile earlier),
//   2. gathers the selected centroid rows from shared memory (128-bit loads, chunk order
//      skewed by j so the four lanes of a token never meet in a bank), scales by the radius
//      and rotates by the key's RoPE angle; the cos/sin rows of the key positions arrive in
//      shared memory by bulk async copies issued half a tile ahead,
//   3. feeds the rotated values to the tensor cores as TF32 hi + lo parts
//      (tokens x dh) * (dh x heads), fp32 accumulate, query fragments held in registers,
//   4. runs the online softmax and accumulates V^T P^T; V tiles are fetched by the tensor
//      memory accelerator (2-D tiled copies with the 128-byte swizzle ldmatrix wants).
// Warp states are merged per CTA, CTA partials land in scratch, and a small kernel merges
// them by log-sum-exp.
//
// Numerics restate SphericalKVPipeline._compressed_head_attention_batched
// (spherical_kv_pipeline.py:2136-2177): logit = sum_g r_g * (q_rot_g . c_g) / sqrt(dh)
// with q back-rotated by the key position; rotating the rebuilt key forward instead is the
// same bilinear form.  Page bytes follow pagebuilder.py:8-33 / paging.py:20-31.
#include <cuda.h>  // CUtensorMap and its enums; the encoder is looked up at run time (no -lcuda)
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"

namespace sphkv {

#ifndef SPHKV_WARPS
#define SPHKV_WARPS 8
#endif
constexpr int kWarps = SPHKV_WARPS;
#ifndef SPHKV_VSTAGES
#define SPHKV_VSTAGES 3
#endif
constexpr int kVStages = SPHKV_VSTAGES;  // V tile buffers per warp: one being read, the others in flight
constexpr int kMetaRing = 32;  // tiles of metadata per warp, refilled 16 at a time
constexpr int kMaxUnitsInKernelPlan = 2048;
// operand split of the QK^T contraction: 2 = TF32 hi + lo (m16n8k8), 1 = bf16 hi + lo by
// truncation (m16n8k16)
#ifndef SPHKV_SPLIT
#define SPHKV_SPLIT 2
#endif
constexpr int kSplit = SPHKV_SPLIT;
// cos/sin rows: 1 = bulk async copies into shared memory, 0 = 128-bit loads into registers
#ifndef SPHKV_CS_STAGED
#define SPHKV_CS_STAGED 1
#endif
constexpr bool kCsStaged = SPHKV_CS_STAGED != 0;
// second, bank-disjoint copy of a g = 16 codebook for odd token rows: 0 never, 1 for
// slots of at most 16 centroids, 2 for every slot that fits
#ifndef SPHKV_CB_DUP
#define SPHKV_CB_DUP 1
#endif

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
  alignas(64) CUtensorMap v_map;  // V pool as [pages * page_size rows][dh], 16 x 64 boxes, 128-byte swizzle
  sphkv_decode_params p;
  int cb_smem_off[SPHKV_MAX_TIER_SLOTS];  // byte offset of each slot's codebook in smem
  int cb_dup[SPHKV_MAX_TIER_SLOTS];       // 1: two copies at a 128-byte row pitch
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
// one half of a cos/sin row (dh * 2 bytes) per token, 16 bytes of padding so that the two
// tokens a quarter-warp reads sit in different banks
__host__ __device__ constexpr int cs_pitch(int dh) { return dh * 2 + 16; }
__host__ __device__ constexpr int smem_cs_bytes(int dh) { return kCsStaged ? kWarps * 2 * 16 * cs_pitch(dh) : 0; }
// per warp: P^T buffer, tile metadata ring, mbarriers (kVStages for V, two for cos/sin)
__host__ __device__ constexpr int smem_priv_bytes() { return 512 + kMetaRing * 16 + 64; }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- mbarrier / bulk-copy wrappers (inline PTX) ----------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: the copies a warp waits for are its own, so a phase that does not complete
// within about a second means a lost copy; the caller then raises a status bit and the
// warp stops working instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > 2000000000LL) return false;
  }
  return true;
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// one row segment, global -> this CTA's shared memory, completion counted on an mbarrier
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// one box of a 2-D tensor map, global -> this CTA's shared memory
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// ---- RoPE table ------------------------------------------------------------------------
// Row of one position: for loop index i (0 .. W/4 - 1) and lane quad member j (0 .. 3) the
// four frequencies  W j + 4 ((i + j) mod (W/4)) + {0..3}  as {cos x 4, sin x 4}: 32 bytes per
// (i, j), so what the four lanes of a token read in one step is one 128-byte line, and the
// first half of the row is what the first half of the tile loop needs.
__host__ __device__ __forceinline__ int lane_freq(int dh, int i, int j, int e) {
  const int W = dh / 8, nch = W / 4;
  return W * j + 4 * ((i + j) & (nch - 1)) + e;
}
__global__ void rope_table_kernel(float* __restrict__ table, int max_pos, int dh,
                                  const float* __restrict__ inv_freq) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int half = dh / 2;
  if (idx >= (int64_t)max_pos * half) return;
  const int pos = (int)(idx / half), q = (int)(idx - (int64_t)pos * half);
  const int e = q & 3, j = (q >> 2) & 3, i = q >> 4;
  const int f = lane_freq(dh, i, j, e);
  const float ang = __fmul_rn((float)pos, inv_freq[f]);
  double sn, cs;
  sincos((double)ang, &sn, &cs);
  float* row = table + (int64_t)pos * dh + (i * 4 + j) * 8;
  row[e] = (float)cs;
  row[4 + e] = (float)sn;
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

// Page words a lane needs for its two tokens (index = 2 * token + rotary half): the aligned
// 32-bit word holding the start of the centroid index (and the next one when the index
// straddles it), the word(s) holding the radius, and the two per-group scales.
// The positions of the two tokens ride along.  Three of these rotate through the tile loop
// (tile k is consumed while the loads of tiles k + 1 and k + 2 are in flight); the loop is
// unrolled by three so that each set keeps its registers: copying a set forward would make
// every iteration wait for loads it has only just issued.
struct KRaw {
  uint32_t tw0[4], tw1[4], rw0[4], rw1[4];
  float sc[2];
  int pos[2];
};

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// PACK (<= 4 query heads per KV head): the 8 mma columns carry [q_hi heads 0..3 | q_lo heads
// 0..3] (one product fewer per step) and later [P_hi | P_lo] (one product per V tile).
template <int DH, typename VT, bool ROT, bool EXTRA, bool PACK>
__global__ void __launch_bounds__(kWarps * 32, 1) decode_splitk_kernel(const __grid_constant__ DecodeArgs a) {
  constexpr int KS = DH / 16;   // 16-dim output tiles of the V product
  constexpr int W = DH / 8;     // dims a lane owns in each rotary half
  constexpr int NCH = W / 4;    // 16-byte chunks of those dims
  constexpr int NH = NCH / 2;   // chunks per half of the tile loop
  constexpr int V_TILE = 16 * DH * 2;
  constexpr int V_WARP = kVStages * V_TILE;
  constexpr int CS_PITCH = cs_pitch(DH);
  constexpr int CS_HALF = 16 * CS_PITCH;
  constexpr bool kBf16 = std::is_same<VT, __nv_bfloat16>::value;
  constexpr bool STAGED = ROT && kCsStaged;
  // query fragment registers per (rotary half, chunk): TF32 two k8 steps x {b0, b1}, bf16 one k16 step
  constexpr int QR = kSplit == 2 ? 4 : 2;

  extern __shared__ __align__(1024) uint8_t smem[];
  const sphkv_decode_params& p = a.p;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, j = lane & 3;

  uint8_t* v_ring = smem + warp * V_WARP;
  uint8_t* cs_warp = smem + smem_v_bytes(DH) + warp * 2 * CS_HALF;
  uint8_t* cb_smem = smem + smem_v_bytes(DH) + smem_cs_bytes(DH);
  uint8_t* warp_priv = cb_smem + a.cb_smem_bytes + warp * smem_priv_bytes();
  uint16_t* pbuf = reinterpret_cast<uint16_t*>(warp_priv);  // [2][8][16]
  TileMeta* meta = reinterpret_cast<TileMeta*>(warp_priv + 512);
  const uint32_t bar_v = smem_u32(warp_priv + 512 + kMetaRing * 16);  // one per V stage
  const uint32_t bar_cs = bar_v + 8 * kVStages;                        // two cos/sin halves
  static_assert(8 * (kVStages + 2) <= 64, "mbarriers exceed their slot");
  const uint32_t cb_u32 = smem_u32(cb_smem);
  const uint32_t cs_lane = smem_u32(cs_warp) + r * CS_PITCH + j * 32;

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kVStages; ++i) mbar_init(bar_v + 8 * i, 1);
    mbar_init(bar_cs, 1);
    mbar_init(bar_cs + 8, 1);
    fence_async_smem();
  }
  __syncthreads();
  // V ring position of the next tile to issue / to wait for: stage index and phase parity
  uint32_t vi_stage = 0, vw_stage = 0, vw_phase = 0, cs_waited[2] = {0, 0};
  bool dead = false;  // a bounded wait ran out: stop working, keep meeting the CTA barriers

  // ---- block prefix per unit: computed by warp 0 of every CTA (CTA 0 publishes it for the
  //      merge kernel), or read from the plan kernel's output when there are many units ----
  const int32_t* pfx = a.pfx;
  if (a.plan_in_kernel) {
    int32_t* pfx_s = reinterpret_cast<int32_t*>(cb_smem + a.cb_smem_bytes + kWarps * smem_priv_bytes());
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
  const int TPP = N >> 4;  // 16-token tiles per page: 1, 2, 4 or 8
  const int tpp_shift = 31 - __clz(TPP);
  const float qscale = p.sm_scale * kLog2e;
  const int fmt = p.radius_fmt;
  const int rb = fmt == SPHKV_RADIUS_F16 ? 2 : 1;
  int cb_head_loaded = -1;
  // per tier slot: b_theta | log2(g) << 8 | duplicated << 12 | codebook offset in shared
  // memory << 13, held by lanes 0..3 and read with a shuffle
  uint32_t tier_word = 0;
  if (lane < SPHKV_MAX_TIER_SLOTS && lane < p.tiers.n_slots) {
    int g_l = 16, b_l = 1, off_l = 0, dup_l = 0;
#pragma unroll
    for (int s = 0; s < SPHKV_MAX_TIER_SLOTS; ++s)
      if (s == lane) { g_l = p.tiers.g[s]; b_l = p.tiers.bits[s]; off_l = a.cb_smem_off[s]; dup_l = a.cb_dup[s]; }
    tier_word = (uint32_t)b_l | ((uint32_t)(g_l == 32 ? 5 : 4) << 8) | ((uint32_t)dup_l << 12) |
                ((uint32_t)off_l << 13);
  }
  auto tier_of = [&](int slot) { return __shfl_sync(0xffffffffu, tier_word, slot); };
  // chunk order of this lane: loop index i reads chunk (i + j) mod NCH of its centroid rows
  uint32_t coff[NCH];
#pragma unroll
  for (int i = 0; i < NCH; ++i) coff[i] = (uint32_t)(((i + j) & (NCH - 1)) * 16);

  while (start < end) {
    while ((int64_t)pfx[u + 1] <= start) ++u;  // skip units without blocks
    const int64_t seg_end = end < (int64_t)pfx[u + 1] ? end : (int64_t)pfx[u + 1];
    const int lb0 = (int)(start - pfx[u]);
    const int seg_tiles = (int)(seg_end - start) * TPP;
    // units are walked KV head major (u = hkv * B + b) so that neighbouring segments share
    // their codebooks; tables are indexed by the external unit id b * Hkv + hkv
    const int hkv = u / p.B, b = u - hkv * p.B;
    const int u_ext = b * p.Hkv + hkv;
    const int nt = (!dead && seg_tiles > warp) ? (seg_tiles - warp + kWarps - 1) / kWarps : 0;
    const int32_t* bt_row = p.block_table + (int64_t)u_ext * p.max_blocks;
    const int32_t* st_row = p.bits_table + (int64_t)u_ext * p.max_blocks;

    auto tile_lb = [&](int kk) { return lb0 + ((warp + kWarps * kk) >> tpp_shift); };
    auto tile_sub = [&](int kk) { return (warp + kWarps * kk) & (TPP - 1); };
    // per-tile statistics of this segment: tile kk of head n lands at ml_seg[n * ml_head + 2 * (warp + kWarps kk)]
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

    // V tile kk into the next ring stage: one lane, one or two boxes of 16 rows x 128 bytes
    // through the tensor map, hardware swizzle = chunk ^ (row & 7)
    auto issue_v = [&](int kk) {
      if (kk >= nt) return;
      const TileMeta m = get_meta(kk);
      if (lane == 0) {
        const uint32_t bar = bar_v + 8 * vi_stage;
        if (m.phys >= 0) {
          mbar_expect_tx(bar, V_TILE);
          const uint32_t dst = smem_u32(v_ring) + vi_stage * V_TILE;
          const int y = m.phys * N + 16 * tile_sub(kk);
#pragma unroll
          for (int h = 0; h < DH / 64; ++h) tma_load_2d(dst + h * 2048, &a.v_map, 64 * h, y, bar);
        } else {
          mbar_arrive(bar);
        }
      }
      vi_stage = vi_stage + 1 == kVStages ? 0 : vi_stage + 1;
    };
    // waits for the oldest tile in flight; returns its stage through `stage`
    auto wait_v = [&](uint32_t& stage) -> bool {
      const bool ok = mbar_wait(bar_v + 8 * vw_stage, vw_phase);
      stage = vw_stage;
      if (++vw_stage == kVStages) { vw_stage = 0; vw_phase ^= 1u; }
      return ok;
    };

    // geometry of this lane's two groups for a tier word
    auto lane_groups = [&](uint32_t tw, int& G, int& glo, int& ghi, int& sub_off) {
      const int lg = (tw >> 8) & 0xF;
      G = DH >> lg;
      glo = (W * j) >> lg;
      ghi = glo + (G >> 1);
      sub_off = (W * j) & ((1 << lg) - 1);
    };

    auto load_kraw = [&](int kk, KRaw& w) {
#pragma unroll
      for (int i = 0; i < 4; ++i) w.tw0[i] = w.tw1[i] = w.rw0[i] = w.rw1[i] = 0u;
      w.sc[0] = w.sc[1] = 0.f;
      w.pos[0] = w.pos[1] = -1;
      if (kk >= nt) return;
      const TileMeta m = get_meta(kk);
      if (m.phys < 0) return;
      if (ROT) {  // key positions of rows r and r + 8 (-1: no token)
        const int32_t* pp = p.positions + (int64_t)m.phys * N + 16 * tile_sub(kk);
        w.pos[0] = pp[r];
        w.pos[1] = pp[r + 8];
      }
      const uint32_t tw = tier_of(meta_slot(m));
      const int bits = tw & 0xFF;
      int G, glo, ghi, sub_off;
      lane_groups(tw, G, glo, ghi, sub_off);
      const int roff = meta_roff(m);
#pragma unroll
      for (int tk = 0; tk < 2; ++tk) {
        const int tp = 16 * tile_sub(kk) + r + 8 * tk;
        if (tp >= meta_count(m)) continue;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int idx = tp * G + (hf ? ghi : glo);
          const int bit = idx * bits;
          const int ba = m.toff + (bit >> 3);
          const uint32_t* wp = reinterpret_cast<const uint32_t*>(p.k_pages + (ba & ~3));
          w.tw0[2 * tk + hf] = wp[0];
          if ((ba & 3) * 8 + (bit & 7) + bits > 32) w.tw1[2 * tk + hf] = wp[1];
          const int ra = roff + idx * rb;
          const uint32_t* rp = reinterpret_cast<const uint32_t*>(p.k_pages + (ra & ~3));
          w.rw0[2 * tk + hf] = rp[0];
          if (rb == 2 && (ra & 3) == 3) w.rw1[2 * tk + hf] = rp[1];
        }
      }
      if (rb == 1) {
        const float* sp = reinterpret_cast<const float*>(p.k_pages + m.poff + 8);
        w.sc[0] = sp[glo];
        w.sc[1] = sp[ghi];
      }
    };
    auto clamp_pos = [&](int pos) -> int {
      if (pos >= p.max_pos) {
        if (p.status) atomicOr(p.status, SPHKV_ST_BAD_POSITION);
        pos = 0;
      }
      return pos < 0 ? 0 : pos;
    };

    // cos/sin of the tile's key positions.  Staged: half h of the row (loop indices
    // h * NH .. h * NH + NH - 1) of every token goes to shared memory by one bulk copy per
    // token, lanes with j = 0 for rows r, j = 1 for rows r + 8.  Register path: this lane's
    // 32-byte pieces by 128-bit loads through L1.
    float4 cs[STAGED ? 1 : 2][STAGED ? 1 : NCH][2];
    auto issue_cs_half = [&](int h, const int (&ps)[2]) {
      if constexpr (STAGED) {
        const int pos = j == 0 ? ps[0] : ps[1];
        const bool mine = j < 2 && pos >= 0;
        const uint32_t n_rows = __popc(__ballot_sync(0xffffffffu, mine));
        const uint32_t bar = bar_cs + 8 * h;
        if (lane == 0) mbar_expect_tx(bar, n_rows * (DH * 2));
        __syncwarp();
        if (mine) {
          const int row = r + 8 * j;
          bulk_copy_g2s(smem_u32(cs_warp) + h * CS_HALF + row * CS_PITCH,
                        p.rope_table + (int64_t)clamp_pos(pos) * DH + h * (DH / 2), DH * 2, bar);
        }
      }
    };
    auto issue_cs_regs = [&](const int (&ps)[2]) {
      if constexpr (ROT && !STAGED) {
#pragma unroll
        for (int tk = 0; tk < 2; ++tk) {
          const float4* rp = reinterpret_cast<const float4*>(p.rope_table + (int64_t)clamp_pos(ps[tk]) * DH) + j * 2;
#pragma unroll
          for (int i = 0; i < NCH; ++i) {
            cs[tk][i][0] = __ldg(rp + i * 8);
            cs[tk][i][1] = __ldg(rp + i * 8 + 1);
          }
        }
      }
    };
    auto wait_cs_half = [&](int h) -> bool {
      bool ok = true;
      if constexpr (STAGED) {
        ok = mbar_wait(bar_cs + 8 * h, cs_waited[h] & 1u);
        ++cs_waited[h];
      }
      return ok;
    };

    auto stage_codebooks = [&]() {
      if (hkv == cb_head_loaded) return;
      const sphkv_tiers& tg = p.tiers;
      for (int s = 0; s < tg.n_slots; ++s) {
        // natural order [group][centroid][g floats]; a duplicated slot (g = 16) keeps two
        // copies of every 64-byte row in one 128-byte slot, the second for odd token rows
        const int g = tg.g[s], bits = tg.bits[s], G = DH / g, cpr = g >> 2;
        const int dup = a.cb_dup[s];
        const float* src = p.codebooks + ((int64_t)(hkv * tg.n_slots + s) * tg.G_max) * tg.C_max * tg.g_max;
        float4* dst = reinterpret_cast<float4*>(cb_smem + a.cb_smem_off[s]);
        const int chunks = (G << bits) * cpr;
        for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
          const int c4 = i % cpr, row = i / cpr;
          const int c = row & ((1 << bits) - 1), gam = row >> bits;
          const float4 v = __ldg(reinterpret_cast<const float4*>(src + ((int64_t)gam * tg.C_max + c) * tg.g_max) + c4);
          if (dup) {
            dst[row * 8 + c4] = v;
            dst[row * 8 + 4 + c4] = v;
          } else {
            dst[i] = v;
          }
        }
      }
      cb_head_loaded = hkv;
    };

    // query fragments (B operand [k = dim][n = column]) in registers, pre-scaled by
    // sm_scale * log2(e).  Column n of a packed tile: head n & 3, hi part for n < 4, lo part
    // otherwise; unpacked: qh = hi parts, ql = lo parts of head n.
    uint32_t qh[2 * NCH][QR], ql[PACK ? 1 : 2 * NCH][PACK ? 1 : QR];
    auto load_q = [&]() {
      const int n = r;  // B-fragment column of this lane
      const int head = PACK ? (n & 3) : n;
      const bool real = head < a.grp;
      const int64_t qbase = ((int64_t)b * p.Hq + (int64_t)hkv * a.grp + head) * DH;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          float v[4], hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int d = hf * (DH / 2) + lane_freq(DH, i, j, e);
            v[e] = real ? load_as_float(p.q, p.q_dtype, qbase + d) * qscale : 0.f;
            const uint32_t msk = kSplit == 2 ? 0xFFFFE000u : 0xFFFF0000u;
            hi[e] = __uint_as_float(__float_as_uint(v[e]) & msk);
            lo[e] = v[e] - hi[e];
          }
          const int s = hf * NCH + i;
          if (kSplit == 2) {
            // k8 step t: b0 = value 2t (k = j), b1 = value 2t + 1 (k = j + 4)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (PACK) {
                qh[s][e] = __float_as_uint(n < 4 ? hi[e] : lo[e]);
              } else {
                qh[s][e] = __float_as_uint(hi[e]);
                ql[PACK ? 0 : s][PACK ? 0 : e] = __float_as_uint(lo[e]);
              }
            }
          } else {
#pragma unroll
            for (int e2 = 0; e2 < 2; ++e2) {
              const uint32_t h2 = __byte_perm(__float_as_uint(hi[2 * e2]), __float_as_uint(hi[2 * e2 + 1]), 0x7632);
              __nv_bfloat162 lb = __floats2bfloat162_rn(lo[2 * e2], lo[2 * e2 + 1]);
              const uint32_t l2 = *reinterpret_cast<uint32_t*>(&lb);
              if (PACK) {
                qh[s][e2] = n < 4 ? h2 : l2;
              } else {
                qh[s][e2] = h2;
                ql[PACK ? 0 : s][PACK ? 0 : e2] = l2;
              }
            }
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
    fence_async_smem();  // this thread's plain shared-memory writes before the next async copies
    __syncthreads();     // the previous segment is done with shared memory
    meta_stage0(0);
    stage_codebooks();
    meta_stage1();
    load_q();
    meta_stage2(0);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kVStages - 1; ++i) issue_v(i);
    KRaw kw_a, kw_b, kw_c;  // page words of tiles k, k+1, k+2 (rotating)
    load_kraw(0, kw_a);
    load_kraw(1, kw_b);
    if (nt > 0) {
      issue_cs_half(0, kw_a.pos);
      issue_cs_half(1, kw_a.pos);
      issue_cs_regs(kw_a.pos);
    }

    // one tile: `cur` holds tile k, `nx1` tile k + 1 (its positions start the next cos/sin
    // copies), `nx2` receives the loads of tile k + 2.  Returns false when a wait gave up.
    auto tile_step = [&](const int k, KRaw& cur, KRaw& nx1, KRaw& nx2) -> bool {
      {  // fetch the next 16 tiles' metadata into the idle half of the ring, in three steps
        const int ph = k & 15, kb = (k & ~15) + 16;
        if (ph == 0) meta_stage0(kb);
        else if (ph == 5) meta_stage1();
        else if (ph == 10) { meta_stage2(kb); __syncwarp(); }
      }
      issue_v(k + kVStages - 1);  // into the stage tile k - 1 has just released
      load_kraw(k + 2, nx2);
      const TileMeta m = get_meta(k);
      const int sub = tile_sub(k);
      const int cnt_tile = m.phys < 0 ? 0 : min(16, max(0, meta_count(m) - 16 * sub));
      const bool live = cnt_tile > 0;
      bool ok_wait = true;

      // ---- this lane's centroid rows and radii for tokens r, r + 8 ------------------------
      uint32_t row_lo[2] = {cb_u32, cb_u32}, row_hi[2] = {cb_u32, cb_u32};
      float rad_lo[2] = {0.f, 0.f}, rad_hi[2] = {0.f, 0.f};
      if (live) {
        const uint32_t tw = tier_of(meta_slot(m));
        const int bits = tw & 0xFF;
        const uint32_t cmask = (1u << bits) - 1u;
        const int dup = (tw >> 12) & 1;
        const int row_shift = (int)((tw >> 8) & 0xF) + 2 + dup;
        int G, glo, ghi, sub_off;
        lane_groups(tw, G, glo, ghi, sub_off);
        const uint32_t base = cb_u32 + (tw >> 13) + sub_off * 4 + (dup ? (r & 1) * 64 : 0);
        const int roff = meta_roff(m);
#pragma unroll
        for (int tk = 0; tk < 2; ++tk) {
          const int tp = 16 * sub + r + 8 * tk;
          const bool tok_ok = tp < meta_count(m);
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int grp = hf ? ghi : glo;
            const int idx = tp * G + grp;
            const int bit = idx * bits;
            const int ba = m.toff + (bit >> 3);
            const uint32_t code =
                __funnelshift_r(cur.tw0[2 * tk + hf], cur.tw1[2 * tk + hf], (ba & 3) * 8 + (bit & 7)) & cmask;
            const uint32_t row = base + ((((uint32_t)grp << bits) + code) << row_shift);
            const int ra = roff + idx * rb;
            float rad;
            if (fmt == SPHKV_RADIUS_F16) {
              const uint32_t hv = __funnelshift_r(cur.rw0[2 * tk + hf], cur.rw1[2 * tk + hf], (ra & 3) * 8);
              rad = __half2float(__ushort_as_half((unsigned short)(hv & 0xFFFFu)));
            } else {
              const int c8 = (int)(int8_t)((cur.rw0[2 * tk + hf] >> ((ra & 3) * 8)) & 0xFFu);
              rad = (cur.sc[hf] * (float)c8) * (1.0f / 127.0f);
            }
            if (!tok_ok) rad = 0.f;
            if (hf) { row_hi[tk] = row; rad_hi[tk] = rad; } else { row_lo[tk] = row; rad_lo[tk] = rad; }
          }
        }
      }

      // ---- rebuild the rotated key tile chunk by chunk, QK^T on tensor cores ---------------
      float s_h[4] = {0.f, 0.f, 0.f, 0.f}, s_l[4] = {0.f, 0.f, 0.f, 0.f}, s_x[4] = {0.f, 0.f, 0.f, 0.f};
      auto qk_chunk = [&](int s, const float2 (&v)[2][2]) {
        // v[token][pair]: the four values of chunk s for rows r and r + 8
        if constexpr (kSplit == 2) {
          uint32_t ah[2][4], al[2][4];
#pragma unroll
          for (int tk = 0; tk < 2; ++tk)
#pragma unroll
            for (int e2 = 0; e2 < 2; ++e2) {
              const uint32_t x0 = __float_as_uint(v[tk][e2].x), x1 = __float_as_uint(v[tk][e2].y);
              const uint32_t h0 = x0 & 0xFFFFE000u, h1 = x1 & 0xFFFFE000u;
              const float2 l = __ffma2_rn(f2(__uint_as_float(h0), __uint_as_float(h1)), f2(-1.f, -1.f), v[tk][e2]);
              ah[tk][2 * e2] = h0; ah[tk][2 * e2 + 1] = h1;
              al[tk][2 * e2] = __float_as_uint(l.x); al[tk][2 * e2 + 1] = __float_as_uint(l.y);
            }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t b0 = qh[s][2 * t], b1 = qh[s][2 * t + 1];
            mma_tf32_1688(s_h, ah[0][2 * t], ah[1][2 * t], ah[0][2 * t + 1], ah[1][2 * t + 1], b0, b1);
            mma_tf32_1688(s_l, al[0][2 * t], al[1][2 * t], al[0][2 * t + 1], al[1][2 * t + 1], b0, b1);
            if (!PACK)
              mma_tf32_1688(s_x, ah[0][2 * t], ah[1][2 * t], ah[0][2 * t + 1], ah[1][2 * t + 1],
                            ql[PACK ? 0 : s][PACK ? 0 : 2 * t], ql[PACK ? 0 : s][PACK ? 0 : 2 * t + 1]);
          }
        } else {
          uint32_t ah[4], al[4];
#pragma unroll
          for (int tk = 0; tk < 2; ++tk)
#pragma unroll
            for (int e2 = 0; e2 < 2; ++e2) {
              const uint32_t x0 = __float_as_uint(v[tk][e2].x), x1 = __float_as_uint(v[tk][e2].y);
              const uint32_t h0 = x0 & 0xFFFF0000u, h1 = x1 & 0xFFFF0000u;
              const float2 l = __ffma2_rn(f2(__uint_as_float(h0), __uint_as_float(h1)), f2(-1.f, -1.f), v[tk][e2]);
              ah[tk + 2 * e2] = __byte_perm(x0, x1, 0x7632);
              al[tk + 2 * e2] = __byte_perm(__float_as_uint(l.x), __float_as_uint(l.y), 0x7632);
            }
          mma_bf16_16816(s_h, ah, qh[s][0], qh[s][1]);
          mma_bf16_16816(s_l, al, qh[s][0], qh[s][1]);
          if (!PACK) mma_bf16_16816(s_x, ah, ql[PACK ? 0 : s][0], ql[PACK ? 0 : s][PACK ? 0 : 1]);
        }
      };
      auto do_chunk = [&](int i) {
        float2 lo[2][2], hi[2][2];
#pragma unroll
        for (int tk = 0; tk < 2; ++tk) {
          const float4 x = lds128(row_lo[tk] + coff[i]);
          const float4 y = lds128(row_hi[tk] + coff[i]);
          const float2 rl = f2(rad_lo[tk], rad_lo[tk]), rh = f2(rad_hi[tk], rad_hi[tk]);
          const float2 x0 = __fmul2_rn(f2(x.x, x.y), rl), x1 = __fmul2_rn(f2(x.z, x.w), rl);
          const float2 y0 = __fmul2_rn(f2(y.x, y.y), rh), y1 = __fmul2_rn(f2(y.z, y.w), rh);
          if constexpr (ROT) {
            float4 c, sn;
            if constexpr (STAGED) {
              const uint32_t ad = cs_lane + tk * 8 * CS_PITCH + (i / NH) * CS_HALF + (i % NH) * 128;
              c = lds128(ad);
              sn = lds128(ad + 16);
            } else {
              c = cs[STAGED ? 0 : tk][STAGED ? 0 : i][0];
              sn = cs[STAGED ? 0 : tk][STAGED ? 0 : i][1];
            }
            const float2 c0 = f2(c.x, c.y), c1 = f2(c.z, c.w);
            const float2 s0 = f2(sn.x, sn.y), s1 = f2(sn.z, sn.w);
            const float2 n0 = f2(-sn.x, -sn.y), n1 = f2(-sn.z, -sn.w);
            lo[tk][0] = __ffma2_rn(y0, n0, __fmul2_rn(x0, c0));
            lo[tk][1] = __ffma2_rn(y1, n1, __fmul2_rn(x1, c1));
            hi[tk][0] = __ffma2_rn(x0, s0, __fmul2_rn(y0, c0));
            hi[tk][1] = __ffma2_rn(x1, s1, __fmul2_rn(y1, c1));
          } else {
            lo[tk][0] = x0; lo[tk][1] = x1; hi[tk][0] = y0; hi[tk][1] = y1;
          }
        }
        qk_chunk(i, lo);
        qk_chunk(NCH + i, hi);
      };

      ok_wait &= wait_cs_half(0);
      if (live) {
#pragma unroll
        for (int i = 0; i < NH; ++i) do_chunk(i);
      }
      __syncwarp();
      if (k + 1 < nt) issue_cs_half(0, nx1.pos);
      ok_wait &= wait_cs_half(1);
      if (live) {
#pragma unroll
        for (int i = NH; i < NCH; ++i) do_chunk(i);
      }
      __syncwarp();
      if (k + 1 < nt) { issue_cs_half(1, nx1.pos); issue_cs_regs(nx1.pos); }

      float pv[4] = {0.f, 0.f, 0.f, 0.f};
      if (live) {
        // ---- online softmax over the 16 token rows, per head column ------------------
        float sv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          sv[e] = s_h[e] + (s_l[e] + s_x[e]);
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
        const bool ok0 = r < cnt_tile && (!ROT || cur.pos[0] >= 0);
        const bool ok1 = (r + 8) < cnt_tile && (!ROT || cur.pos[1] >= 0);
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
      } else if (EXTRA && ml_seg != nullptr && lane < a.grp) {  // a tile without tokens: (-inf, 0)
        float* dst = ml_seg + lane * ml_head + 2 * kWarps * k;
        dst[0] = -INFINITY;
        dst[1] = 0.f;
      }
      uint32_t v_stage;
      ok_wait &= wait_v(v_stage);  // tile k's V has landed
      __syncwarp();
      if (live) {
        const uint32_t* ph32 = reinterpret_cast<const uint32_t*>(pbuf);
        const uint32_t b0 = ph32[(r * 16 + 2 * j) >> 1];
        const uint32_t b1 = ph32[(r * 16 + 2 * j + 8) >> 1];
        uint32_t c0 = 0, c1 = 0;
        if (kBf16 && !PACK) {
          c0 = ph32[(8 * 16 + r * 16 + 2 * j) >> 1];
          c1 = ph32[(8 * 16 + r * 16 + 2 * j + 8) >> 1];
        }
        // ---- acc^T[dh][head] += V^T[dh][token] P^T[token][head] ---------------------
        const uint32_t vbase = smem_u32(v_ring) + v_stage * V_TILE;
        const int mi = lane >> 3;
        const int tau = (lane & 7) + ((mi >> 1) << 3);
#pragma unroll
        for (int dt = 0; dt < KS; ++dt) {
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
      if (!__all_sync(0xffffffffu, ok_wait)) {
        // an async copy never completed: flag it and stop; the partial row of this segment is
        // not meaningful and the host sees the status bit
        if (lane == 0 && p.status) atomicOr(p.status, SPHKV_ST_TIMEOUT);
        dead = true;
        return false;
      }
      return true;
    };
    for (int k = 0; k < nt; k += 3) {
      if (!tile_step(k, kw_a, kw_b, kw_c)) break;
      if (k + 1 < nt && !tile_step(k + 1, kw_b, kw_c, kw_a)) break;
      if (k + 2 < nt && !tile_step(k + 2, kw_c, kw_a, kw_b)) break;
    }

    // ---- merge the warps of this CTA and write one partial row ---------------------
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
      l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
    }
    __syncthreads();  // every warp is done with its V ring
    if (!dead) {
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
    } else if (lane < 8) {
      reinterpret_cast<float*>(v_ring)[lane * (DH + 2)] = -INFINITY;  // contributes nothing
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

// Shared-memory layout of the codebooks: a g = 16 slot may be stored twice (row pitch 128
// bytes, second copy for odd token rows) when the policy asks for it and the space is there.
static int smem_cb_layout(const sphkv_tiers& t, int dh, int budget_bytes, int* offs, int* dup) {
  int plain = 0;
  for (int s = 0; s < t.n_slots; ++s) plain += dh * (1 << t.bits[s]) * 4;
  int extra_left = budget_bytes - plain;
  int off = 0;
  for (int s = 0; s < t.n_slots; ++s) {
    const int bytes = dh * (1 << t.bits[s]) * 4;
    const bool want = t.g[s] == 16 && (SPHKV_CB_DUP == 2 || (SPHKV_CB_DUP == 1 && t.bits[s] <= 4));
    dup[s] = (want && bytes <= extra_left) ? 1 : 0;
    if (dup[s]) extra_left -= bytes;
    offs[s] = off;
    off += bytes * (dup[s] ? 2 : 1);
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

// ---- tensor map of the V pool ------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    tried = true;
  }
  return fn;
}

// V pool viewed as a 2-D tensor [n_pages * page_size rows][dh] of 16-bit elements; a box is 16
// rows x 64 elements (128 bytes, the widest row the 128-byte swizzle takes).  Encoding is host
// arithmetic only (no device memory, no driver state).
static int make_v_map(CUtensorMap* map, const sphkv_decode_params& p) {
  EncodeTiledFn fn = encode_tiled_fn();
  SPHKV_REQUIRE(fn != nullptr, SPHKV_E_ARG, "decode: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)p.dh, (cuuint64_t)p.n_pages * (cuuint64_t)p.page_size};
  const cuuint64_t strides[1] = {(cuuint64_t)p.dh * 2};
  const cuuint32_t box[2] = {64, 16};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = fn(map, p.v_dtype == SPHKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         2, const_cast<void*>(p.v_pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SPHKV_REQUIRE(rc == CUDA_SUCCESS, SPHKV_E_ARG, "decode: cuTensorMapEncodeTiled failed (%d) for the V pool", (int)rc);
  return 0;
}

template <int DH, typename VT, bool ROT, bool EXTRA, bool PACK>
static int launch_decode_t(const DecodeArgs& a, int smem_bytes, cudaStream_t st) {
  static SmemOptIn opt_in;
  auto kern = decode_splitk_kernel<DH, VT, ROT, EXTRA, PACK>;
  if (int rc = ensure_dynamic_smem(opt_in, (const void*)kern, smem_bytes, "decode")) return rc;
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

static int resolve_ctas(int n_ctas) { return n_ctas > 0 ? n_ctas : sm_count_current_device(); }

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
  SPHKV_REQUIRE(p.rope_table == nullptr || p.max_pos > 0, SPHKV_E_ARG,
                "decode: rope_table given with max_pos=%d (rows of the table)", p.max_pos);
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
  a.plan_in_kernel = a.n_units <= kMaxUnitsInKernelPlan ? 1 : 0;
  const int fixed_bytes = smem_v_bytes(p.dh) + (p.rope_table ? smem_cs_bytes(p.dh) : smem_cs_bytes(p.dh)) +
                          kWarps * smem_priv_bytes() + (a.plan_in_kernel ? (a.n_units + 1) * 4 : 0);
  a.cb_smem_bytes = smem_cb_layout(p.tiers, p.dh, 227 * 1024 - fixed_bytes, a.cb_smem_off, a.cb_dup);
  const int smem_bytes = fixed_bytes + a.cb_smem_bytes;
  SPHKV_REQUIRE(smem_bytes <= 227 * 1024, SPHKV_E_LIMIT,
                "decode: codebooks need %d B of shared memory (limit %d)", smem_bytes, 227 * 1024);
  if (int rc = make_v_map(&a.v_map, p)) return rc;
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
