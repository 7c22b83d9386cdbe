// Angle-domain decode attention over bit-packed, paged, codebook-quantised keys.
//
// One persistent CTA per SM (8 warps) walks a contiguous range of (KV head, batch row) blocks.
// Each warp owns every 8th 16-token tile of the range and keeps an online-softmax state for
// all query heads of the KV head.
//
// Lane map of a tile (lane = 4 r + j): rows r and r + 8 are the lane's two tokens; in each
// rotary half the lane owns the contiguous block of W = dh / 8 dimensions  W j .. W j + W - 1
// and, in the other half, the same block shifted by dh / 2 -- the RoPE partner of every value
// a lane holds is in the same lane, and for g = 16, dh = 128 a lane needs exactly two centroid
// indices and two radii per token, which it extracts itself from the page bytes.
//
// Data movement, all asynchronous and issued tiles ahead of use:
//   * V tiles: tensor-map (TMA) copies into a per-warp ring, 128-byte swizzle = the pattern
//     ldmatrix wants, completion on an mbarrier per stage (bounded wait);
//   * page bytes + key positions: cp.async (16-byte chunks for 16-byte-aligned pages, 4-byte
//     words otherwise) into a per-warp ring of 512-byte stages, three tiles ahead, so the
//     page -> position -> cos/sin dependency never stalls a tile;
//   * cos/sin rows of the key positions: one 256-bit load per (token, 4-frequency chunk) from the
//     L2-resident table into registers, one tile ahead.
// Per tile a warp
//   1. extracts its centroid indices / radii from the staged page with constants that are
//      recomputed only when the tier changes,
//   2. gathers the selected centroid rows from shared memory (128-bit loads, chunk order
//      XOR-skewed by j so the four lanes of a token never meet in a bank; odd token rows read a
//      second copy of the codebook so the two tokens of a quarter-warp do not meet either),
//      scales by the radius and rotates by the key's RoPE angle with packed fp32 arithmetic,
//   3. feeds the rotated values to the tensor cores as bf16 hi + lo parts
//      (tokens x dh) * (dh x heads), fp32 accumulate, query fragments held in registers,
//   4. runs the online softmax and accumulates V^T P^T.
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
constexpr int kMetaRing = 32;  // tiles of metadata per warp, refilled 16 at a time
constexpr int kMaxUnitsInKernelPlan = 2048;
#ifndef SPHKV_VSTAGES
#define SPHKV_VSTAGES 3
#endif
constexpr int kVStages = SPHKV_VSTAGES;  // V tile buffers per warp: one being read, the others in flight

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
// per warp: P^T buffer, tile metadata ring, mbarriers (kVStages for V, two for cos/sin), four
// 512-byte stages of page pieces + positions
__host__ __device__ constexpr int smem_priv_bytes() { return 512 + kMetaRing * 16 + 64 + 4 * 512; }

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
// one box of a 2-D tensor map, global -> this CTA's shared memory
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// codebook rows only: they do not change while a segment is processed, so the load may be
// scheduled freely
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// ---- RoPE table ------------------------------------------------------------------------
// Row of one position: for loop index i (0 .. W/4 - 1) and lane quad member j (0 .. 3) the
// four frequencies  W j + 4 ((i xor j) mod (W/4)) + {0..3}  as {cos x 4, sin x 4}: 32 bytes per
// (i, j), so what the four lanes of a token read in one step is one 128-byte line, and the
// first half of the row is what the first half of the tile loop needs.
__host__ __device__ __forceinline__ int lane_freq(int dh, int i, int j, int e) {
  const int W = dh / 8, nch = W / 4;
  return W * j + 4 * ((i ^ j) & (nch - 1)) + e;
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

// ---- K stage: what a tile needs of its page, copied into a per-warp ring ---------------------
// A stage holds, at fixed offsets, the page header + group scales, the slice of the theta bit
// stream of the tile's 16 tokens, the slice of their radius bytes and their 16 positions.
// Every piece starts at the 4-byte word that holds its first byte, so the byte phase inside
// the first word is the phase the piece has in the pool.  The copies are 4-byte cp.async
// (the pool only promises 4-byte alignment), word w of the stage by lane w mod 32 in round
// w / 32; they are issued three tiles ahead and cost no registers while in flight.
constexpr int kKStages = 4;
constexpr int kKStageBytes = 512;
constexpr int kKHdr = 0;    // 12 words: 8 header bytes + up to 8 scales (+ slack)
constexpr int kKTh = 48;    // 28 words: 16 tokens x 8 groups x 6 bits = 96 bytes + phase
constexpr int kKRd = 160;   // 68 words: 16 tokens x 8 groups x 2 bytes = 256 bytes + phase
constexpr int kKPos = 448;  // 16 words
static_assert(kKPos + 64 <= kKStageBytes, "K stage layout");

__device__ __forceinline__ void cp_async_4(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ int lds_s8(uint32_t addr) {
  int v;
  asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// PACK (<= 4 query heads per KV head): the 8 mma columns carry [q_hi heads 0..3 | q_lo heads
// 0..3] (one product fewer per step) and later [P_hi | P_lo] (one product per V tile).
// MODE bit 0 clear: 16-token pages with int8 radii (the serving configuration: page size and
// radius format are compile-time constants and the page image is staged word for word); set: any
// page size / radius format.  MODE bit 1: the logits / per-tile statistics side outputs.
template <int DH, typename VT, bool ROT, int MODE, bool PACK>
__global__ void __launch_bounds__(kWarps * 32, 1) decode_splitk_kernel(const __grid_constant__ DecodeArgs a) {
  constexpr bool EXTRA = (MODE & 2) != 0, FAST = (MODE & 1) == 0;
  constexpr int KS = DH / 16;   // 16-dim output tiles of the V product
  constexpr int W = DH / 8;     // dims a lane owns in each rotary half
  constexpr int NCH = W / 4;    // 16-byte chunks of those dims
  constexpr int V_TILE = 16 * DH * 2;
  constexpr int V_WARP = kVStages * V_TILE;
  constexpr bool kBf16 = std::is_same<VT, __nv_bfloat16>::value;

  extern __shared__ __align__(1024) uint8_t smem[];
  const sphkv_decode_params& p = a.p;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, j = lane & 3;

  uint8_t* v_ring = smem + warp * V_WARP;
  uint8_t* cb_smem = smem + smem_v_bytes(DH);
  uint8_t* warp_priv = cb_smem + a.cb_smem_bytes + warp * smem_priv_bytes();
  uint16_t* pbuf = reinterpret_cast<uint16_t*>(warp_priv);  // [2][8][16]
  TileMeta* meta = reinterpret_cast<TileMeta*>(warp_priv + 512);
  const uint32_t bar_v = smem_u32(warp_priv + 512 + kMetaRing * 16);  // one per V stage
  static_assert(8 * kVStages <= 64, "mbarriers exceed their slot");
  const uint32_t k_ring = bar_v + 64;  // kKStages stages of kKStageBytes
  const uint32_t cb_u32 = smem_u32(cb_smem);

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kVStages; ++i) mbar_init(bar_v + 8 * i, 1);
    fence_async_smem();
  }
  __syncthreads();
  // everything above touched shared memory only: this grid's launch overlaps the tail of the kernel
  // before it in the stream (the previous step's merge kernel, which lets it in early)
  griddep_wait();
  // V ring position of the next tile to issue / to wait for: stage index and phase parity
  uint32_t vi_stage = 0, vw_stage = 0, vw_phase = 0;
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

  const int N = FAST ? 16 : p.page_size;
  const int TPP = N >> 4;  // 16-token tiles per page: 1, 2, 4 or 8
  const int tpp_shift = 31 - __clz(TPP);
  const float qscale = p.sm_scale * kLog2e;
  const int fmt = FAST ? SPHKV_RADIUS_I8 : p.radius_fmt;
  const uint32_t rb = fmt == SPHKV_RADIUS_F16 ? 2u : 1u;
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
  // chunk order of this lane: loop index i reads chunk (i xor j) mod NCH of its centroid rows,
  // i.e. byte (row ^ (j mod NCH) * 16) ^ (i * 16) of a 64-byte-aligned row
  const uint32_t cskew = (uint32_t)((j & (NCH - 1)) * 16);

  // ldmatrix row address of this lane for output tile dt: token row tau, 16-byte chunk
  // c = 2 dt + (lane / 8 & 1) of the 256-byte row, stored at chunk (c & 7) ^ (tau & 7) of the
  // 128-byte half-row (c >> 3).  (c & 7) ^ (tau & 7) = 2 (dt & 3) ^ ((lane / 8 & 1) ^ (tau & 7)).
  uint32_t ldsm_off[4];
  {
    const int mi = lane >> 3, tau = (lane & 7) + ((mi >> 1) << 3);
#pragma unroll
    for (int x = 0; x < 4; ++x) ldsm_off[x] = (uint32_t)(tau * 128 + (((2 * x) ^ ((mi & 1) ^ (tau & 7))) << 4));
  }
  // K-stage copy plan of this lane: in round q it copies stage word 32 q + lane.  Words 0..11
  // are the header piece, 12..39 the theta piece, 40..107 the radius piece, 108..123 the
  // positions; krel[q] is the byte offset of the lane's word inside its piece.
  const uint32_t krel[4] = {4u * (lane < 12 ? lane : lane - 12), 4u * (lane < 8 ? lane + 20 : lane - 8),
                            4u * (lane + 24), 4u * (lane < 12 ? lane + 56 : lane - 12)};
  uint32_t k_issue = 0;  // K stages issued so far (ring index = k_issue mod kKStages)
  uint32_t k_read = 0;   // K stages consumed so far

  // lane constants of the tier slot of the current tile, recomputed only when the slot changes
  // (block lists keep the pages of a tier together)
  int c_slot = -1;
  uint32_t c_bits = 1, c_mask = 1, c_rowb = 64, c_cb_lo = 0, c_cb_hi = 0;
  // bit offset of the centroid index of (token, half) and byte offset of its radius: relative to
  // the tile's theta / radius slice, or (FAST) to the page start and to the first radius byte
  uint32_t c_bit[4] = {0, 0, 0, 0};
  uint32_t c_wa[4] = {0, 0, 0, 0};    // FAST: byte offset in the stage of the word holding the index
  uint32_t c_rad[4] = {0, 0, 0, 0};
  uint32_t c_sc[2] = {0, 0};          // byte offset of its group's scale in the header piece
  auto load_slot_constants = [&](int slot) {
    const uint32_t tw = tier_of(slot);
    const int lg = (tw >> 8) & 0xF;
    const int G = DH >> lg;
    const int glo = (W * j) >> lg, ghi = glo + (G >> 1);
    const int sub_off = (W * j) & ((1 << lg) - 1);
    const int dup = (tw >> 12) & 1;
    c_bits = tw & 0xFF;
    c_mask = (1u << c_bits) - 1u;
    c_rowb = 4u << (lg + dup);  // bytes from one centroid row to the next
    const uint32_t base = cb_u32 + (tw >> 13) + sub_off * 4 + (dup ? (r & 1) * 64 : 0);
    c_cb_lo = base + ((uint32_t)glo << c_bits) * c_rowb;
    c_cb_hi = base + ((uint32_t)ghi << c_bits) * c_rowb;
#pragma unroll
    for (int tk = 0; tk < 2; ++tk)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const uint32_t idx = (uint32_t)((r + 8 * tk) * G + (hf ? ghi : glo));
        // 16-token pages: the theta stream starts 8 + 4 G bytes into the page (pagebuilder.py:8-33;
        // checked against the pointer table when the tile metadata is fetched)
        c_bit[2 * tk + hf] = idx * c_bits + (FAST ? (8 + 4 * G) * 8 : 0);
        c_wa[2 * tk + hf] = (c_bit[2 * tk + hf] >> 5) << 2;
        c_rad[2 * tk + hf] = idx * rb;
      }
    c_sc[0] = 8 + 4 * glo;
    c_sc[1] = 8 + 4 * ghi;
    c_slot = slot;
  };

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
        if (FAST && mf_toff - mf_poff != 8 + 4 * (DH / p.tiers.g[mf_slot])) {
          // the pointer table disagrees with the page format: not a page this path can read
          if (p.status) atomicOr(p.status, SPHKV_ST_BAD_BLOCK);
          m.phys = -1;
          count = 0;
        }
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

    // One K stage per tile, issued three tiles ahead.  16-token pages: the page image itself,
    // word for word from the page start (header at 0, theta at toff - poff, radii at
    // roff - poff).  Larger pages: the header piece at kKHdr, the tile's slice of the theta
    // stream at kKTh and of the radii at kKRd, each from the word that holds its first byte.
    // The positions go to kKPos.  One commit group per call, whether or not anything is
    // copied, so that the group of tile k is always the (kKStages - 1)-th newest when tile k
    // is consumed.
    auto issue_k = [&](int kk) {
      if (kk < nt) {
        const TileMeta m = get_meta(kk);
        const uint32_t dst = k_ring + (k_issue & (kKStages - 1)) * kKStageBytes + 4 * lane;
        if (m.phys >= 0) {
          const uint32_t tw = tier_of(meta_slot(m));
          const uint32_t bits = tw & 0xFF, G = (uint32_t)DH >> ((tw >> 8) & 0xF);
          const uint32_t poff = (uint32_t)m.poff;
          if (TPP == 1) {
            const uint32_t page_end = (uint32_t)meta_roff(m) + (uint32_t)meta_count(m) * G * rb;
            if ((poff & 15u) == 0) {
              // 16-byte copies for the chunks wholly inside the page (at most 24), 4-byte copies by
              // the next four lanes for the words of the last, partial chunk: nothing past the page
              const uint32_t full = (page_end - poff) >> 4;
              const uint32_t kb = dst - 4 * lane;
              if ((uint32_t)lane < full) {
                cp_async_16(kb + 16 * lane, p.k_pages + (poff + 16 * lane));
              } else {
                const uint32_t o = 16 * full + 4 * (lane - full);
                if (lane < full + 4 && poff + o < page_end) cp_async_4(kb + o, p.k_pages + (poff + o));
              }
            } else {
              const uint32_t off = poff + 4 * lane;
#pragma unroll
              for (int q = 0; q < 3; ++q)
                if (off + 128 * q < page_end) cp_async_4(dst + 128 * q, p.k_pages + (off + 128 * q));
              if (rb == 2 && off + 384 < page_end && lane < 16) cp_async_4(dst + 384, p.k_pages + (off + 384));
            }
          } else {
            const int sub = tile_sub(kk);
            const uint32_t t0 = 16u * sub, t1 = min((uint32_t)meta_count(m), t0 + 16u);
            const uint32_t th0 = (uint32_t)m.toff + ((t0 * G * bits) >> 3);
            const uint32_t th1 = (uint32_t)m.toff + ((t1 * G * bits + 7) >> 3);
            const uint32_t rd0 = (uint32_t)meta_roff(m) + t0 * G * rb, rd1 = (uint32_t)meta_roff(m) + t1 * G * rb;
            const uint32_t hdr1 = poff + 8 + 4 * G, thA = th0 & ~3u, rdA = rd0 & ~3u;
            {  // words 0..31: header | theta
              const bool hd = lane < 12;
              const uint32_t off = (hd ? poff : thA) + krel[0];
              if (off < (hd ? hdr1 : th1)) cp_async_4(dst, p.k_pages + off);
            }
            {  // words 32..63: theta | radius
              const bool th = lane < 8;
              const uint32_t off = (th ? thA : rdA) + krel[1];
              if (off < (th ? th1 : rd1)) cp_async_4(dst + 128, p.k_pages + off);
            }
            {  // words 64..95: radius
              const uint32_t off = rdA + krel[2];
              if (off < rd1) cp_async_4(dst + 256, p.k_pages + off);
            }
            if (lane < 12) {  // words 96..107: radius
              const uint32_t off = rdA + krel[3];
              if (off < rd1) cp_async_4(dst + 384, p.k_pages + off);
            }
          }
          if (ROT && lane >= 16)  // words 112..127: positions
            cp_async_4(dst + 384, p.positions + ((uint32_t)m.phys * (uint32_t)N + 16u * tile_sub(kk) + (lane - 16)));
        } else if (ROT && lane >= 16) {
          // a hole in the block list: no page; its positions read as "no token"
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst + 384), "r"(0xFFFFFFFFu) : "memory");
        }
      }
      cp_async_commit();
      ++k_issue;
    };

    // table row of a key position: "no token" (-1) and out-of-range positions read row 0; the
    // latter also raise a status bit
    auto clamp_pos = [&](int pos) -> uint32_t {
      if (pos >= p.max_pos && p.status) atomicOr(p.status, SPHKV_ST_BAD_POSITION);
      return (uint32_t)pos < (uint32_t)p.max_pos ? (uint32_t)pos : 0u;
    };
    // positions of this lane's two tokens in K stage `st` (-1: no token)
    auto stage_pos = [&](uint32_t st, int (&ps)[2]) {
      ps[0] = (int)lds32(st + kKPos + 4 * r);
      ps[1] = (int)lds32(st + kKPos + 4 * r + 32);
    };

    // cos/sin of this lane's two key positions: one 256-bit load per (token, chunk) brings the
    // chunk's {cos x 4, sin x 4} (the table is L2 resident), issued for tile k + 1 once tile k
    // has used its own
    float4 cs[2][NCH][2];
    const float4* cs_src[2] = {nullptr, nullptr};  // this lane's pieces of the two table rows
    auto cs_rows = [&](const int (&ps)[2]) {
      if constexpr (ROT) {
#pragma unroll
        for (int tk = 0; tk < 2; ++tk)
          cs_src[tk] = reinterpret_cast<const float4*>(p.rope_table) + (clamp_pos(ps[tk]) * (DH / 4) + j * 2);
      }
    };
    auto issue_cs_chunk = [&](int i) {
      if constexpr (ROT) {
#pragma unroll
        for (int tk = 0; tk < 2; ++tk)
          asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                       : "=f"(cs[tk][i][0].x), "=f"(cs[tk][i][0].y), "=f"(cs[tk][i][0].z), "=f"(cs[tk][i][0].w),
                         "=f"(cs[tk][i][1].x), "=f"(cs[tk][i][1].y), "=f"(cs[tk][i][1].z), "=f"(cs[tk][i][1].w)
                       : "l"(cs_src[tk] + i * 8));
      }
    };
    auto issue_cs = [&](const int (&ps)[2]) {
      cs_rows(ps);
#pragma unroll
      for (int i = 0; i < NCH; ++i) issue_cs_chunk(i);
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
        const uint32_t dst = cb_u32 + a.cb_smem_off[s];
        const int chunks = (G << bits) * cpr;
        // asynchronous 16-byte copies: every chunk of the codebook is in flight at once instead
        // of one load-store round trip per loop iteration (the caller waits for the group)
        for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
          const int c4 = i % cpr, row = i / cpr;
          const int c = row & ((1 << bits) - 1), gam = row >> bits;
          const float4* sp = reinterpret_cast<const float4*>(src + ((int64_t)gam * tg.C_max + c) * tg.g_max) + c4;
          if (dup) {
            cp_async_16(dst + (row * 8 + c4) * 16, sp);
            cp_async_16(dst + (row * 8 + 4 + c4) * 16, sp);
          } else {
            cp_async_16(dst + i * 16, sp);
          }
        }
      }
      cb_head_loaded = hkv;
    };

    // query fragments (B operand [k = dim][n = column]) in registers, pre-scaled by
    // sm_scale * log2(e) and split into bf16 hi (truncated) + bf16 lo.  Column n of a packed tile:
    // head n & 3, hi part for n < 4, lo part otherwise; unpacked: qh = hi parts, ql = lo parts of
    // head n.  Chunk s of rotary half hf: register 0 = values 0, 1 (k = 2j, 2j + 1), register 1 =
    // values 2, 3 (k = 2j + 8, 2j + 9).
    uint32_t qh[2 * NCH][2], ql[PACK ? 1 : 2 * NCH][2];
    auto load_q = [&]() {
      const int n = r;  // B-fragment column of this lane
      const int head = PACK ? (n & 3) : n;
      const bool real = head < a.grp;
      const int64_t qbase = ((int64_t)b * p.Hq + (int64_t)hkv * a.grp + head) * DH;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          float hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int d = hf * (DH / 2) + lane_freq(DH, i, j, e);
            const float v = real ? load_as_float(p.q, p.q_dtype, qbase + d) * qscale : 0.f;
            hi[e] = __uint_as_float(__float_as_uint(v) & 0xFFFF0000u);
            lo[e] = v - hi[e];
          }
          const int s = hf * NCH + i;
#pragma unroll
          for (int e2 = 0; e2 < 2; ++e2) {
            const uint32_t h2 = __byte_perm(__float_as_uint(hi[2 * e2]), __float_as_uint(hi[2 * e2 + 1]), 0x7632);
            __nv_bfloat162 lb = __floats2bfloat162_rn(lo[2 * e2], lo[2 * e2 + 1]);
            const uint32_t l2 = *reinterpret_cast<uint32_t*>(&lb);
            if (PACK) {
              qh[s][e2] = n < 4 ? h2 : l2;
            } else {
              qh[s][e2] = h2;
              ql[PACK ? 0 : s][e2] = l2;
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
    cp_async_commit();
    meta_stage1();
    load_q();
    meta_stage2(0);
    cp_async_wait<0>();  // the codebook copies of this thread; the barrier publishes everyone's
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kVStages - 1; ++i) issue_v(i);
#pragma unroll
    for (int i = 0; i < kKStages - 1; ++i) issue_k(i);
    if (nt > 0 && ROT) {
      // tile 0's positions start its cos/sin fetch
      cp_async_wait<kKStages - 2>();
      __syncwarp();
      int ps0[2];
      stage_pos(k_ring + (k_read & (kKStages - 1)) * kKStageBytes, ps0);
      issue_cs(ps0);
    }

    for (int k = 0; k < nt; ++k) {
      {  // fetch the next 16 tiles' metadata into the idle half of the ring, in three steps
        const int ph = k & 15, kb = (k & ~15) + 16;
        if (ph == 0) meta_stage0(kb);
        else if (ph == 5) meta_stage1();
        else if (ph == 10) { meta_stage2(kb); __syncwarp(); }
      }
      issue_v(k + kVStages - 1);  // into the stage tile k - 1 has just released
      issue_k(k + kKStages - 1);
      const TileMeta m = get_meta(k);
      const int sub = tile_sub(k);
      const int cnt_tile = m.phys < 0 ? 0 : min(16, max(0, meta_count(m) - 16 * sub));
      // K stages of tiles k and k + 1 have landed (the two newest groups may be in flight)
      cp_async_wait<kKStages - 2>();
      __syncwarp();
      const uint32_t kst = k_ring + (k_read & (kKStages - 1)) * kKStageBytes;
      const uint32_t kst1 = k_ring + ((k_read + 1) & (kKStages - 1)) * kKStageBytes;
      ++k_read;
      int pos_n[2] = {-1, -1};
      if (ROT && k + 1 < nt) stage_pos(kst1, pos_n);

      if (cnt_tile == 0) {
        // nothing stored here (a hole, or a tile past the page's count): keep the pipelines moving
        if (EXTRA && ml_seg != nullptr && lane < a.grp) {  // its statistics: (-inf, 0)
          float* dst = ml_seg + lane * ml_head + 2 * kWarps * k;
          dst[0] = -INFINITY;
          dst[1] = 0.f;
        }
        if (k + 1 < nt) issue_cs(pos_n);
        uint32_t v_stage;
        if (!__all_sync(0xffffffffu, wait_v(v_stage))) { dead = true; break; }
        continue;
      }

      // ---- this lane's centroid rows and radii for tokens r, r + 8 ------------------------
      int pos_c[2] = {0, 0};
      if (ROT) stage_pos(kst, pos_c);
      if (meta_slot(m) != c_slot) load_slot_constants(meta_slot(m));
      // stage-relative byte address of the first theta byte / radius byte of the tile
      uint32_t th_b0, rd_b0;
      if (FAST) {
        th_b0 = 0;  // folded into the slot constants
        rd_b0 = (uint32_t)(m.toff - m.poff) + (m.misc & 0xFFFFu);
      } else if (TPP == 1) {
        th_b0 = (uint32_t)(m.toff - m.poff);
        rd_b0 = th_b0 + (m.misc & 0xFFFFu);
      } else {
        const uint32_t G = (uint32_t)DH >> ((tier_of(meta_slot(m)) >> 8) & 0xF);
        th_b0 = kKTh + (((uint32_t)m.toff + ((16u * sub * G * c_bits) >> 3)) & 3u);
        rd_b0 = kKRd + (((uint32_t)meta_roff(m) + 16u * sub * G * rb) & 3u);
      }
      uint32_t row_lo[2], row_hi[2];
      float rad_lo[2], rad_hi[2];
      {
        const uint32_t th_bit = th_b0 << 3;
        const uint32_t rd_ad = kst + rd_b0;
        float scl[2] = {1.f, 1.f};
        if (fmt != SPHKV_RADIUS_F16) {
          scl[0] = __uint_as_float(lds32(kst + kKHdr + c_sc[0])) * (1.0f / 127.0f);
          scl[1] = __uint_as_float(lds32(kst + kKHdr + c_sc[1])) * (1.0f / 127.0f);
        }
#pragma unroll
        for (int tk = 0; tk < 2; ++tk)
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const uint32_t bit = th_bit + c_bit[2 * tk + hf];
            const uint32_t wa = kst + (FAST ? c_wa[2 * tk + hf] : ((bit >> 5) << 2));
            const uint32_t code = __funnelshift_r(lds32(wa), lds32(wa + 4), bit) & c_mask;
            const uint32_t row = ((hf ? c_cb_hi : c_cb_lo) + code * c_rowb) ^ cskew;
            float rad;
            if (fmt == SPHKV_RADIUS_F16) {
              const uint32_t ra = rd_ad + c_rad[2 * tk + hf];
              rad = __half2float(__ushort_as_half((unsigned short)(lds_u8(ra) | (lds_u8(ra + 1) << 8))));
            } else {
              rad = scl[hf] * (float)lds_s8(rd_ad + c_rad[2 * tk + hf]);
            }
            if (hf) { row_hi[tk] = row; rad_hi[tk] = rad; } else { row_lo[tk] = row; rad_lo[tk] = rad; }
          }
      }

      // ---- rebuild the rotated key tile chunk by chunk, QK^T on tensor cores ---------------
      float s_h[4] = {0.f, 0.f, 0.f, 0.f}, s_l[4] = {0.f, 0.f, 0.f, 0.f}, s_x[4] = {0.f, 0.f, 0.f, 0.f};
      auto qk_chunk = [&](int s, const float2 (&v)[2][2]) {
        // v[token][pair]: the four values of chunk s for rows r and r + 8.  Operand split: hi = the
        // upper 16 bits of the fp32 value (a bf16 number, by truncation: one byte permute packs two
        // of them), lo = the value minus hi, again truncated to bf16; hi + lo carries 16 mantissa
        // bits, and the three products hi*hi + lo*hi + hi*lo are accumulated in fp32.
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
        if (!PACK) mma_bf16_16816(s_x, ah, ql[PACK ? 0 : s][0], ql[PACK ? 0 : s][1]);
      };
      const bool more = k + 1 < nt;
      if (more) cs_rows(pos_n);
#pragma unroll
      for (int i = 0; i < NCH; ++i) {
        float2 lo[2][2], hi[2][2];
#pragma unroll
        for (int tk = 0; tk < 2; ++tk) {
          const float4 x = lds128(row_lo[tk] ^ (uint32_t)(i * 16));
          const float4 y = lds128(row_hi[tk] ^ (uint32_t)(i * 16));
          const float2 rl = f2(rad_lo[tk], rad_lo[tk]), rh = f2(rad_hi[tk], rad_hi[tk]);
          const float2 x0 = __fmul2_rn(f2(x.x, x.y), rl), x1 = __fmul2_rn(f2(x.z, x.w), rl);
          const float2 y0 = __fmul2_rn(f2(y.x, y.y), rh), y1 = __fmul2_rn(f2(y.z, y.w), rh);
          if constexpr (ROT) {
            const float4 c = cs[tk][i][0], sn = cs[tk][i][1];
            const float2 c0 = f2(c.x, c.y), c1 = f2(c.z, c.w);
            const float2 s0 = f2(sn.x, sn.y), s1 = f2(sn.z, sn.w);
            // x cos - y sin needs a negated operand and the packed fma has no negate modifier: the
            // negative radius gives -y for the price of two packed multiplies
            const float2 rn = f2(-rad_hi[tk], -rad_hi[tk]);
            const float2 m0 = __fmul2_rn(f2(y.x, y.y), rn), m1 = __fmul2_rn(f2(y.z, y.w), rn);
            lo[tk][0] = __ffma2_rn(m0, s0, __fmul2_rn(x0, c0));
            lo[tk][1] = __ffma2_rn(m1, s1, __fmul2_rn(x1, c1));
            hi[tk][0] = __ffma2_rn(x0, s0, __fmul2_rn(y0, c0));
            hi[tk][1] = __ffma2_rn(x1, s1, __fmul2_rn(y1, c1));
          } else {
            lo[tk][0] = x0; lo[tk][1] = x1; hi[tk][0] = y0; hi[tk][1] = y1;
          }
        }
        // this chunk's cos/sin registers are free: fetch the next tile's
        if (more) issue_cs_chunk(i);
        qk_chunk(i, lo);
        qk_chunk(NCH + i, hi);
      }

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
      // rows without a token (past the page's count, or position -1) take no part; whatever
      // their stale page bytes produced above is replaced here
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
      float alpha[2], msafe[2], pv[4];
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
      uint32_t v_stage;
      const bool v_ok = wait_v(v_stage);  // tile k's V has landed
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
        const uint32_t vbase = smem_u32(v_ring) + v_stage * V_TILE;
#pragma unroll
        for (int dt = 0; dt < KS; ++dt) {
          uint32_t af[4];
          ldmatrix_x4_trans(af, vbase + ldsm_off[dt & 3] + (dt >> 2) * 2048);
          if (kBf16) {
            mma_bf16_16816(acc[dt], af, b0, b1);
            if (!PACK) mma_bf16_16816(acc[dt], af, c0, c1);
          } else {
            mma_f16_16816(acc[dt], af, b0, b1);
          }
        }
      }
      __syncwarp();
      if (!__all_sync(0xffffffffu, v_ok)) { dead = true; break; }
    }
    if (dead && lane == 0 && p.status) {
      // an async copy never completed within the bounded wait: the partial row of this segment
      // is not meaningful and the host sees the status bit
      atomicOr(p.status, SPHKV_ST_TIMEOUT);
    }
    cp_async_wait<0>();  // the tail groups are empty; nothing of this segment stays in flight
    k_read = k_issue;

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
  __shared__ float s_M[8], s_L[8];
  __shared__ float s_w[8][kChunk];
  // The next kernel in the stream -- the next step's decode kernel -- may become resident now; it
  // waits for this grid to complete before it touches global memory.  (Launching THIS kernel the
  // same way measured 2 us slower per step, so it is launched plainly.)
  griddep_launch();
  const int32_t* pfx = a.pfx;
  const int64_t T = pfx[a.n_units];
  const int64_t ps = pfx[u], pe = pfx[u + 1];
  // the CTAs whose block ranges meet this unit's (every thread derives them: no barrier, no
  // shared-memory round trip between the prefix loads and the row loads)
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
  const int nrows = c_hi - c_lo + 1;
  auto row_exists = [&](int c) -> bool {
    return cta_range_start(c, a.n_ctas, T) != cta_range_start(c + 1, a.n_ctas, T);
  };
  auto row_m = [&](int n, int c) -> float {  // max of row (c, u) for head n; -inf if no such row
    if (!row_exists(c)) return -INFINITY;
    return a.rows[((int64_t)(c + u) * 8 + n) * (DH + 2)];
  };
  float o_acc[(8 * DH + 255) / 256];
#pragma unroll
  for (int q = 0; q < (8 * DH + 255) / 256; ++q) o_acc[q] = 0.f;
  const bool few_rows = nrows <= 32;
  if (few_rows) {
    // At most one row per lane (the usual case: units >= CTAs / 32).  A warp covers 32 dimensions
    // of one head: lane c fetches row c's (max, sum) while the accumulator loads of the first
    // rows are already in flight, the warp reduces, and every lane then folds the rows of its
    // dimension with the weights passed around by shuffles -- one memory latency instead of the
    // four of the general path below, and the same arithmetic in the same order.
#pragma unroll
    for (int q = 0; q < (8 * DH + 255) / 256; ++q) {
      const int i = threadIdx.x + q * 256;
      const int n = i / DH, d = i - n * DH;
      if (n >= a.grp) continue;  // warp-uniform: DH is a multiple of 32
      const float* col = a.rows + ((int64_t)(c_lo + u) * 8 + n) * (DH + 2);
      const bool mine = lane < nrows && row_exists(c_lo + lane);
      const float mr = mine ? col[(int64_t)lane * 8 * (DH + 2)] : -INFINITY;
      const float lr = mine ? col[(int64_t)lane * 8 * (DH + 2) + 1] : 0.f;
      float M = mr;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
      const float w = (mine && M != -INFINITY) ? exp2f(mr - M) : 0.f;
      float L = lr * w;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
      if (lane == 0 && d == 0) { s_M[n] = M; s_L[n] = L; }
      float o = 0.f;
      for (int ci = 0; ci < nrows; ci += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = ci + k < nrows ? col[(int64_t)(ci + k) * 8 * (DH + 2) + 2 + d] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float wk = __shfl_sync(0xffffffffu, w, (ci + k) & 31);
          o += (ci + k < nrows && wk != 0.f) ? wk * v[k] : 0.f;
        }
      }
      o_acc[q] = o;
    }
    __syncthreads();
  } else if (warp < a.grp) {
    // pass 1: warp n -> global max and sum of head n
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
  if (!few_rows) __syncthreads();
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
  // pass 2 of the general path: weights per chunk of rows, then threads over (head, dim)
  for (int c0 = 0; c0 < (few_rows ? 0 : nrows); c0 += kChunk) {
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
        // eight rows' loads in flight at a time (a unit cut over many CTAs has tens of rows: one
        // dependent load per row made this loop the whole kernel); a row that does not exist has
        // weight 0 and whatever the scratch holds there is discarded by the select
        float o = o_acc[q];
        const float* col = a.rows + ((int64_t)(c_lo + c0 + u) * 8 + n) * (DH + 2) + 2 + d;
        for (int ci = 0; ci < nc; ci += 8) {
          float v[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = ci + k < nc ? col[(int64_t)(ci + k) * 8 * (DH + 2)] : 0.f;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float w = ci + k < nc ? s_w[n][ci + k] : 0.f;
            o += w != 0.f ? w * v[k] : 0.f;
          }
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
    if (p.out != nullptr && p.xchg_world <= 1)
      store_from_float(p.out, p.out_dtype, hq * DH + d, l > 0.f ? o / l : 0.f);
  }
  if (p.xchg_world <= 1) return;

  // ---- split-KV exchange: this rank's rows of the unit go to every rank, then the unit is
  //      combined over the ranks here.  Every 64-bit word a rank stores carries the step number
  //      beside the value ((seq << 32) | f32 bits, one single-copy-atomic store), so a word
  //      validates itself: no fence, no separate flag, one NVLink crossing per value.  Peer
  //      memory is touched by plain stores only; the words a rank reads are in its own memory.
  __shared__ int s_seq, s_ok;
  __shared__ float s_rm[SPHKV_MAX_XCHG_RANKS][8], s_rl[SPHKV_MAX_XCHG_RANKS][8];
  const int unit = b * p.Hkv + hkv;
  const int64_t n_rows = (int64_t)p.B * p.Hq;
  if (threadIdx.x == 0) {
    s_seq = p.xchg_seq[unit] + 1;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t seq = (uint32_t)s_seq;
  const int64_t slot_base = (int64_t)(seq & 1) * p.xchg_world * n_rows;  // rows; the two slots alternate by step
  auto put = [&](unsigned long long* dst, float v) {
    const unsigned long long w = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
  };
#pragma unroll
  for (int q = 0; q < (8 * DH + 255) / 256; ++q) {
    const int i = threadIdx.x + q * 256;
    const int n = i / DH, d = i - n * DH;
    if (n >= a.grp) continue;
    const int64_t hq = (int64_t)b * p.Hq + (int64_t)hkv * a.grp + n;
    const int64_t off = (slot_base + (int64_t)p.xchg_rank * n_rows + hq) * (DH + 2);
    for (int peer = 0; peer < p.xchg_world; ++peer) {
      unsigned long long* dst = p.xchg_recv[peer] + off;
      if (d == 0) {
        put(dst, s_M[n] * kLn2);
        put(dst + 1, s_L[n]);
      }
      put(dst + 2 + d, o_acc[q]);
    }
  }
  // Bounded wait, word by word: a word of this step's slot is in when it carries exactly this
  // step's number (a later step of a peer goes to the other slot; a peer cannot be two steps
  // ahead because it needs this rank's next step to finish its own).  The wait also runs when
  // no output is wanted: it is what keeps the ranks within one step of each other.
  const unsigned long long* mine = p.xchg_recv[p.xchg_rank] + slot_base * (DH + 2);
  const long long limit = p.xchg_timeout_cycles > 0 ? p.xchg_timeout_cycles : 2000000000LL;
  const long long t0 = clock64();
  auto get = [&](const unsigned long long* src) -> float {
    for (;;) {
      unsigned long long w;
      asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
      if ((uint32_t)(w >> 32) == seq) return __uint_as_float((uint32_t)w);
      if (clock64() - t0 > limit) {
        s_ok = 0;  // every thread that gives up writes the same value
        return 0.f;
      }
    }
  };
  for (int i = threadIdx.x; i < p.xchg_world * a.grp; i += blockDim.x) {
    const int rr = i / a.grp, n = i - rr * a.grp;
    const int64_t hq = (int64_t)b * p.Hq + (int64_t)hkv * a.grp + n;
    const unsigned long long* pr = mine + ((int64_t)rr * n_rows + hq) * (DH + 2);
    const float pm = get(pr), pl = get(pr + 1);
    s_rm[rr][n] = pl > 0.f ? pm : -INFINITY;
    s_rl[rr][n] = pl;
  }
  __syncthreads();
  float res[(8 * DH + 255) / 256];
#pragma unroll
  for (int q = 0; q < (8 * DH + 255) / 256; ++q) {
    const int i = threadIdx.x + q * 256;
    const int n = i / DH, d = i - n * DH;
    res[q] = 0.f;
    if (n >= a.grp) continue;
    const int64_t hq = (int64_t)b * p.Hq + (int64_t)hkv * a.grp + n;
    float M = -INFINITY;
    for (int rr = 0; rr < p.xchg_world; ++rr) M = fmaxf(M, s_rm[rr][n]);
    float l = 0.f, o = 0.f;
    for (int rr = 0; rr < p.xchg_world; ++rr) {
      const float v = get(mine + ((int64_t)rr * n_rows + hq) * (DH + 2) + 2 + d);  // every word is awaited
      if (M == -INFINITY || s_rm[rr][n] == -INFINITY) continue;
      const float w = __expf(s_rm[rr][n] - M);
      l += s_rl[rr][n] * w;
      o += v * w;
    }
    res[q] = l > 0.f ? o / l : 0.f;
  }
  __syncthreads();  // every wait has ended, one way or the other
  if (threadIdx.x == 0) p.xchg_seq[unit] = (int32_t)seq;
  const bool ok = s_ok != 0;
  if (!ok && threadIdx.x == 0 && p.status) atomicOr(p.status, SPHKV_ST_TIMEOUT);  // a rank never published this step
  if (p.out == nullptr) return;
#pragma unroll
  for (int q = 0; q < (8 * DH + 255) / 256; ++q) {
    const int i = threadIdx.x + q * 256;
    const int n = i / DH, d = i - n * DH;
    if (n >= a.grp) continue;
    const int64_t hq = (int64_t)b * p.Hq + (int64_t)hkv * a.grp + n;
    store_from_float(p.out, p.out_dtype, hq * DH + d, ok ? res[q] : 0.f);  // defined output either way
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
    const bool want = t.g[s] == 16;
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

// Launch with programmatic stream serialization: the grid may become resident while the kernel
// before it in the stream is still running.  Only for kernels that call griddep_wait() before
// their first global-memory access.
template <typename Arg>
static cudaError_t launch_after_predecessor_starts(void (*kern)(Arg), dim3 grid, dim3 block, size_t smem_bytes,
                                                   cudaStream_t st, const DecodeArgs& a) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, a);
}

template <int DH, typename VT, bool ROT, int MODE, bool PACK>
static int launch_decode_t(const DecodeArgs& a, int smem_bytes, cudaStream_t st) {
  static SmemOptIn opt_in;
  auto kern = decode_splitk_kernel<DH, VT, ROT, MODE, PACK>;
  if (int rc = ensure_dynamic_smem(opt_in, (const void*)kern, smem_bytes, "decode")) return rc;
  (void)launch_after_predecessor_starts(kern, dim3(a.n_ctas), dim3(kWarps * 32), smem_bytes, st, a);  // check_launch reports
  return check_launch("decode_splitk_kernel");
}

template <int DH, typename VT, bool ROT>
static int launch_decode_r(const DecodeArgs& a, int smem_bytes, cudaStream_t st) {
  const bool extra = a.p.logits_out != nullptr || a.p.page_ml != nullptr;
  const bool pack = a.grp <= 4;
  const bool fast = a.p.page_size == 16 && a.p.radius_fmt == SPHKV_RADIUS_I8;
  if (extra && fast)
    return pack ? launch_decode_t<DH, VT, ROT, 2, true>(a, smem_bytes, st)
                : launch_decode_t<DH, VT, ROT, 2, false>(a, smem_bytes, st);
  if (extra)
    return pack ? launch_decode_t<DH, VT, ROT, 3, true>(a, smem_bytes, st)
                : launch_decode_t<DH, VT, ROT, 3, false>(a, smem_bytes, st);
  if (fast)
    return pack ? launch_decode_t<DH, VT, ROT, 0, true>(a, smem_bytes, st)
                : launch_decode_t<DH, VT, ROT, 0, false>(a, smem_bytes, st);
  return pack ? launch_decode_t<DH, VT, ROT, 1, true>(a, smem_bytes, st)
              : launch_decode_t<DH, VT, ROT, 1, false>(a, smem_bytes, st);
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
  SPHKV_REQUIRE(((uintptr_t)table & 31) == 0, SPHKV_E_ALIGN, "rope_table: table needs 32-byte alignment");
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
                    (p.rope_table == nullptr || ((uintptr_t)p.rope_table & 31) == 0) &&
                    ((uintptr_t)p.scratch & 255) == 0,
                SPHKV_E_ALIGN, "decode: v_pool/codebooks need 16 B, rope_table 32 B, k_pages 4 B, scratch 256 B");
  if (int rc = validate_tiers(p.tiers, p.dh)) return rc;
  if (p.xchg_world > 1) {
    SPHKV_REQUIRE(p.xchg_world <= SPHKV_MAX_XCHG_RANKS, SPHKV_E_LIMIT, "decode: xchg_world=%d (max %d)",
                  p.xchg_world, SPHKV_MAX_XCHG_RANKS);
    SPHKV_REQUIRE(p.xchg_rank >= 0 && p.xchg_rank < p.xchg_world, SPHKV_E_ARG, "decode: xchg_rank=%d of %d",
                  p.xchg_rank, p.xchg_world);
    SPHKV_REQUIRE(p.xchg_recv && p.xchg_seq, SPHKV_E_ARG, "decode: the exchange needs xchg_recv and xchg_seq");
    SPHKV_REQUIRE(p.omega == nullptr, SPHKV_E_ARG,
                  "decode: the page-importance update is per rank; run it without the exchange");
  }

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
  const int fixed_bytes = smem_v_bytes(p.dh) + 
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
