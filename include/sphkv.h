/*
 * sphkv.h -- C ABI of libsphkv_b200.so
 *
 * B200 (sm_100a) kernels for the Spherical-KV hot path: the spherical encode that
 * writes codebook-quantised, bit-packed KV pages, and angle-domain decode attention
 * over those pages.  Every entry point takes plain device pointers, sizes and a CUDA
 * stream handle (a cudaStream_t passed as void*; NULL = legacy default stream).
 * Nothing here allocates device memory except where a function says so; all
 * buffers are caller-owned.
 *
 * Return value of every int function: 0 on success, a negative SPHKV_E_* code for a
 * rejected argument, or a positive cudaError_t value if a launch failed.
 * sphkv_last_error() returns a human-readable string for the last failure on the
 * calling thread.
 *
 * Each declaration cites the reference interface (file:line in the Spherical-KV
 * source tree) that it replaces or extends.
 */
#ifndef SPHKV_H_
#define SPHKV_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPHKV_ABI_VERSION 4

/* error codes */
#define SPHKV_OK 0
#define SPHKV_E_ARG (-1)      /* null pointer / bad size / unsupported shape        */
#define SPHKV_E_DTYPE (-2)    /* unsupported dtype tag                               */
#define SPHKV_E_ALIGN (-3)    /* pointer or offset alignment not satisfied           */
#define SPHKV_E_SCRATCH (-4)  /* scratch buffer too small                            */
#define SPHKV_E_LIMIT (-5)    /* size beyond a documented fixed maximum              */

/* dtype tags */
#define SPHKV_F32 0
#define SPHKV_BF16 1
#define SPHKV_F16 2

/* radius storage formats inside a K page (page header byte 2) */
#define SPHKV_RADIUS_I8 0  /* int8 code * scale_g / 127, the reference page format   */
#define SPHKV_RADIUS_F16 1 /* IEEE half per (token, group); header scales still set  */

#define SPHKV_MAX_TIER_SLOTS 4
#define SPHKV_MAX_GQA 8 /* query heads per KV head handled by one kernel pass        */
#define SPHKV_MAX_XCHG_RANKS 16 /* GPUs one split-KV exchange can span                  */

/* Geometry of the codebook tensor and of the tiers stored in it.  The codebook
 * tensor has the layout of LayerPool.cb_flat (sphkv_lut.py:108-111):
 * f32 [Hkv][n_slots][G_max][C_max][g_max], zero padded.  A "slot" is the tier rank
 * of make_tier_idx_map (sphkv_lut.py:7-14). */
typedef struct sphkv_tiers {
  int32_t n_slots;
  int32_t G_max, C_max, g_max;
  int32_t g[SPHKV_MAX_TIER_SLOTS];       /* group size per slot: 16 or 32            */
  int32_t bits[SPHKV_MAX_TIER_SLOTS];    /* b_theta per slot (1..6), C = 2^bits      */
  int32_t tier_id[SPHKV_MAX_TIER_SLOTS]; /* value written to page header byte 0      */
} sphkv_tiers;

/* ---- RoPE table ----------------------------------------------------------------
 * Builds the cos/sin table the decode kernel gathers per key position.  Values are
 * cos/sin of the fp32 product float(pos) * inv_freq[i], the same arguments the HF
 * rotary module produces for the reference's tables
 * (spherical_kv_pipeline.py:1591-1610).  Layout: f32 [max_pos][dh], 32-byte aligned; a row
 * holds, for i = 0 .. dh/32 - 1 and j = 0 .. 3, {cos f0..f3, sin f0..f3} of the frequencies
 * f = (dh/8) j + 4 ((i xor j) mod dh/32) + {0..3} (the order in which the decode kernel's
 * lanes consume them).  inv_freq: device f32 [dh/2]. */
int sphkv_rope_table_build(float* table, int32_t max_pos, int32_t dh, const float* inv_freq,
                           void* stream);

/* ---- Encode ----------------------------------------------------------------------
 * Bulk spherical encode + page build.  Replaces _encode_keys_with_codebooks
 * (spherical_kv_pipeline.py:1130-1144) + build_page (pagebuilder.py:8-33) +
 * PageHeader.to_tensor (paging.py:20-31) + pack_bits (bitpacking.py:5-29) for whole
 * page lists, and the V/position page writes of _build_per_head_pages
 * (spherical_kv_pipeline.py:1146-1228).
 *
 * Work is described per bundle: 128 token slots = 128/page_size pages that share one
 * (KV head, tier slot). */
typedef struct sphkv_encode_params {
  const void* k_src;        /* [rows][Hkv][dh], k_dtype; pre-RoPE keys                */
  const void* v_src;        /* same indexing, v_src_dtype; may be NULL (skip V)       */
  const int32_t* src_index; /* [P][page_size] source row per page slot, -1 = empty    */
  const int32_t* bundles;   /* [n_bundles][8] physical page ids, -1 = unused          */
  const int32_t* page_head; /* [P] KV head of each page (codebook selector)           */
  const int32_t* page_slot; /* [P] tier slot of each page                             */
  const int32_t* ptable;    /* [P][3] (page_off, theta_off, radius_off) byte offsets,
                               pointer_table.py:10-21                                 */
  const float* codebooks;   /* see sphkv_tiers                                        */
  uint8_t* k_pages;         /* out: byte pool                                         */
  void* v_pool;             /* out: [P][page_size][dh], v_pool_dtype (F16 or BF16)    */
  void* scratch;            /* optional, sphkv_encode_scratch_bytes() bytes, 16-aligned:
                               with it the search and the page assembly run as two
                               launches (faster); NULL = one fused launch              */
  int64_t scratch_bytes;
  int64_t k_row_stride;     /* elements between consecutive source rows               */
  int64_t k_head_stride;    /* elements between consecutive heads of a row            */
  int64_t v_row_stride, v_head_stride;
  /* code cache written by sphkv_encode_codes, read by sphkv_pages_from_codes only: per
     tier slot s, radii f32 and centroid indices u8 laid out [Hkv][code_rows][dh / g_s]   */
  const float* code_r[SPHKV_MAX_TIER_SLOTS];
  const uint8_t* code_theta[SPHKV_MAX_TIER_SLOTS];
  int64_t code_rows;
  int32_t n_bundles, n_pages, page_size, dh, Hkv;
  int32_t k_dtype, v_src_dtype, v_pool_dtype;
  int32_t radius_fmt;
  sphkv_tiers tiers;
} sphkv_encode_params;

int64_t sphkv_encode_scratch_bytes(int32_t n_pages, int32_t page_size, int32_t dh);
int sphkv_encode_pages(const sphkv_encode_params* p, void* stream);

/* All-tier pre-encode: radius and nearest centroid of every (row, KV head, group) for every
 * tier slot in ONE pass over the keys.  Replaces the per-tier loop of
 * spherical_kv_pipeline.py:1535-1553 (three _encode_keys_with_codebooks calls per (layer,
 * head), each re-reading K and recomputing the norms).  k_src as in sphkv_encode_params;
 * r_out / theta_out are HOST arrays of tiers->n_slots device pointers, slot s receiving f32
 * / u8 [Hkv][rows][dh / g_s] (a NULL pair skips that slot).  Values equal what
 * sphkv_encode_pages computes for the same tier (same fixed fp32 order). */
int sphkv_encode_codes(const void* k_src, int32_t k_dtype, int64_t k_row_stride,
                       int64_t k_head_stride, int64_t rows, int32_t Hkv, int32_t dh,
                       const float* codebooks, const sphkv_tiers* tiers, float* const* r_out,
                       uint8_t* const* theta_out, void* stream);

/* Re-paging without re-encoding: builds the byte pages (and V pages, when v_src is given) of
 * the page lists in p from the code cache (p->code_r, p->code_theta, p->code_rows) instead of
 * the keys; k_src, codebooks and scratch are ignored.  Replaces _rebuild_pages_for
 * (spherical_kv_pipeline.py:2579-2660): index-select of cached codes + build_page_from_codes
 * per page.  The pages are byte-identical to what sphkv_encode_pages writes from the keys. */
int sphkv_pages_from_codes(const sphkv_encode_params* p, void* stream);

/* ---- Decode ----------------------------------------------------------------------
 * Angle-domain decode attention over bit-packed pages with in-kernel back-rotation
 * by each key's RoPE position, batch, split-K and log-sum-exp merge.  Numerics follow
 * SphericalKVPipeline._compressed_head_attention_batched
 * (spherical_kv_pipeline.py:2136-2177, 2348, 2364-2367); the table layout extends
 * LayerPool (sphkv_lut.py:77-103) with a batch dimension; the call supersedes
 * sphkv_logit_launcher (fused_decode.cpp:3-8) and the undefined fused_decode_ragged
 * (call sites spherical_kv_pipeline.py:1109-1125). */
typedef struct sphkv_decode_params {
  const void* q;              /* [B][Hq][dh] q_dtype, post-RoPE at the query position */
  const uint8_t* k_pages;     /* byte pool, readable up to the next multiple of 4 bytes
                                 past the end of its last page                        */
  const int32_t* ptable;      /* [P][3]                                               */
  const void* v_pool;         /* [P][page_size][dh] v_dtype (F16/BF16); slots past a
                                 page's count must hold finite values (zero-filled)   */
  const int32_t* positions;   /* [P][page_size] key positions, -1 = empty             */
  const int32_t* block_table; /* [B*Hkv][max_blocks] physical page id, -1 = hole      */
  const int32_t* bits_table;  /* [B*Hkv][max_blocks] tier slot of each block          */
  const int32_t* num_blocks;  /* [B*Hkv] blocks in use per (batch row, KV head)       */
  const float* codebooks;     /* see sphkv_tiers                                      */
  const float* rope_table;    /* from sphkv_rope_table_build; NULL = no rotation      */
  void* out;                  /* [B][Hq][dh] out_dtype; may be NULL with out_partial  */
  float* out_partial;         /* optional [B][Hq][dh+2]: (max, sum, acc) un-normalised,
                                 natural-log max, the triple of decode_kernel.cu:212-217
                                 taken over the whole local context                   */
  float* page_ml;             /* optional [B][Hq][max_blocks][page_size/16][2]: (max, sum)
                                 of every 16-token tile of every block in use, natural-
                                 log domain ((-inf, 0) for a tile without tokens); with
                                 page_size 16 this is the per-block side output read at
                                 spherical_kv_pipeline.py:1690-1693                   */
  float* logits_out;          /* optional [B][Hq][max_blocks*page_size] f32: the scaled
                                 logit of every stored token (slot order of the block
                                 table); slots without a token are left untouched       */
  void* scratch;              /* sphkv_decode_scratch_bytes() bytes, 256-aligned      */
  int64_t scratch_bytes;
  int32_t* status;            /* optional device int, OR-ed with SPHKV_ST_* bits      */
  float* omega;               /* optional [B*Hkv][max_blocks] page importance, updated in
                                 place by the merge kernel: omega*ema_beta + (mean over
                                 the KV head's query heads of the block's softmax mass)
                                 *(1-ema_beta), the update of _omega_ema_eager
                                 (spherical_kv_pipeline.py:952-987); needs page_ml      */
  int32_t B, Hq, Hkv, dh, page_size, max_blocks, n_pages, max_pos;
  int32_t q_dtype, v_dtype, out_dtype, radius_fmt;
  int32_t n_ctas;             /* 0 = one per SM of the current device                 */
  float sm_scale;
  float ema_beta;             /* EMA factor for omega (the reference uses 0.9)        */
  sphkv_tiers tiers;
  /* Cross-GPU split-KV exchange inside the merge kernel (xchg_world <= 1: off).  The block
   * tables of this call cover this rank's share of every sequence; the un-normalised
   * (max, sum, acc) rows of every (batch row, query head) are stored straight into every
   * rank's receive buffer (plain peer stores over NVLink) as 64-bit words that carry the step
   * number beside the value, (seq << 32) | f32 bits, so every word validates itself: no fence,
   * no flag, no collective library call, no extra launch.  The same kernel then waits --
   * bounded -- until the words of all ranks carry this step's number, combines the `xchg_world`
   * partial sets by log-sum-exp (math of decode_kernel.cu:230-245) and writes `out`.
   *   xchg_recv[q]  : rank q's receive buffer in rank q's memory, u64
   *                   [2][xchg_world][B*Hq][dh+2] (two slots alternate by step),
   *                   zero-initialised once
   *   xchg_seq      : this rank's step counters, i32 [B*Hkv], zero-initialised once; every
   *                   call advances them by one, so calls replay from a CUDA graph
   * The pointer array lives in device memory of this rank and holds xchg_world entries (entry
   * xchg_rank = this rank's own buffer).  All ranks must issue the same sequence of calls.  A
   * wait that exceeds xchg_timeout_cycles SM clocks (0 = 2e9, about a second) gives up: the
   * kernel raises SPHKV_ST_TIMEOUT in `status`, writes zeros to the rows of that unit and
   * returns. */
  unsigned long long* const* xchg_recv;
  int32_t* xchg_seq;
  int64_t xchg_timeout_cycles;
  int32_t xchg_rank, xchg_world;
} sphkv_decode_params;

#define SPHKV_ST_BAD_POSITION 1 /* a key position was outside [0, max_pos)            */
#define SPHKV_ST_BAD_BLOCK 2    /* a block-table entry was >= n_pages                 */
#define SPHKV_ST_BAD_SLOT 4     /* a bits-table entry was outside [0, n_slots)        */
#define SPHKV_ST_TIMEOUT 8      /* an asynchronous copy, or another rank's part of a split-KV
                                   exchange, did not arrive within the kernel's bounded
                                   wait; the output is not valid                      */
#define SPHKV_ST_INTERNAL 16    /* the kernel found its shared memory misaligned      */

int64_t sphkv_decode_scratch_bytes(int32_t B, int32_t Hkv, int32_t dh, int32_t n_ctas);
/* Two launches on `stream`: the split-K decode kernel and the merge kernel.  The decode kernel is
 * launched with programmatic stream serialization: its CTAs may become resident while the kernel
 * before it in the stream is still running, but it reads and writes no global memory before that
 * kernel has completed, so stream order is what the caller observes (and what a CUDA graph
 * captured from the stream replays). */
int sphkv_decode_paged(const sphkv_decode_params* p, void* stream);

/* Has no counterpart in the reference.  Same operation, arguments and results as
 * sphkv_decode_paged, for callers that cannot provide scratch memory and must not cause an
 * allocation: a serving process that committed all of its HBM to the KV pools at start-up,
 * or a plug-in inside one, gets nothing back from cudaMalloc.  p->scratch and
 * p->scratch_bytes are ignored; the split-K scratch is a fixed array inside the library
 * image (about 1.7 MB on every GPU that loads the library, for the life of the process).
 * Limits: B * Hkv <= 256, dh <= 128, at most 160 CTAs (p->n_ctas, or the SM count when 0);
 * anything larger returns SPHKV_E_LIMIT.  The call performs no cudaMalloc / cudaFree and
 * uses no allocating library routine.  Its first call on a device looks the array's device
 * address up (cudaGetSymbolAddress, that device current): make that call before any stream
 * capture begins.  All calls on a device share the one array, which keeps whatever the last
 * call left in it (the kernels overwrite every word they later read, nothing needs
 * clearing): two calls whose kernels may overlap on the GPU -- different streams, or two
 * host threads -- race on it and must be serialised by the caller. */
int sphkv_decode_paged_static(const sphkv_decode_params* p, void* stream);

/* Buffers of the split-KV peer exchange (xchg_recv of sphkv_decode_params); no
 * counterpart in the reference, which has no multi-GPU path.  They are written by kernels of
 * other GPUs, each driven by its own process, so they travel as CUDA IPC handles:
 *   sphkv_xchg_alloc  cudaMalloc + zero fill on the current device; returns the pointer and the
 *                     64-byte IPC handle to hand to the other ranks (this call ALLOCATES);
 *   sphkv_xchg_open   maps another rank's buffer into the current device's address space
 *                     (peer access is enabled as a side effect); call with the device current
 *                     whose kernels will store into it, once per handle and process;
 *   sphkv_xchg_close / sphkv_xchg_free   undo the two. */
int sphkv_xchg_alloc(int64_t bytes, void** dev_ptr, unsigned char* handle64);
int sphkv_xchg_open(const unsigned char* handle64, void** dev_ptr);
int sphkv_xchg_close(void* opened_ptr);
int sphkv_xchg_free(void* dev_ptr);

/* Log-sum-exp combine of R partial sets, each f32 [n_rows][dh+2] = (max, sum, acc),
 * natural-log max.  Same math as sphkv_reduce_kernel (decode_kernel.cu:221-246) with a
 * plain division (no +1e-8); rows whose total sum is 0 produce zeros.  Used after the
 * all-gather of per-GPU partials in split-KV decode.  parts: [R][n_rows][dh+2]. */
int sphkv_merge_partials(const float* parts, int32_t R, int32_t n_rows, int32_t dh, void* out,
                         int32_t out_dtype, void* stream);

/* ---- Reference-signature operators over the LayerPool layout ----------------------
 * Pools as built by LayerPool.__init__ (sphkv_lut.py:77-103): theta_codes, radius_codes
 * u8 [P][page_size][G_max]; r_scales f32 [P][G_max]; v_pool f16 [P][page_size][dh];
 * block_table, bits_table i32 [Hkv][max_blocks]; cb_flat f32
 * [Hkv][num_tiers][G_max][cb_max][g_max]; single sequence, post-RoPE keys. */

/* Replaces sphkv_logit_launcher (fused_decode.cpp:3-8; kernels decode_kernel.cu:108-246),
 * argument for argument, plus the stream.  out f32 [Hq][dh]; partial_scratch f32
 * [Hq][max_blocks][dh+2] receives the per-page (m, l, acc) that
 * spherical_kv_pipeline.py:1690-1693 reads back.  ctx_lens and max_ctx are accepted and
 * unused, as in the reference. */
int sphkv_pool_decode(const float* q_all, const float* cb_flat, const int32_t* tier_G,
                      const int32_t* tier_g, const uint8_t* theta_codes,
                      const uint8_t* radius_codes, const float* r_scales, const void* v_pool,
                      const int32_t* block_table, const int32_t* bits_table,
                      const int32_t* ctx_lens, float* out, float* partial_scratch,
                      int32_t num_q_heads, int32_t num_kv_heads, int32_t kv_groups,
                      int32_t num_tiers, int32_t max_blocks, int32_t page_size, int32_t dh,
                      int32_t G_max, int32_t cb_max, int32_t g_max, float sm_scale, int32_t max_ctx,
                      void* stream);

/* Replaces sphkv_encode_append_launcher (fused_decode.cpp:10-14; kernel
 * decode_kernel.cu:10-84).  num_kv is k_post.size(0) of the reference call.  pids: i64. */
int sphkv_pool_encode_append(const float* k_post, const float* v_new, const float* decode_cb,
                             uint8_t* theta_codes, uint8_t* radius_codes, float* r_scales,
                             void* v_pool, const int64_t* pids, int32_t slot, int32_t G, int32_t g,
                             int32_t C, int32_t G_max, int32_t dh, int32_t page_size,
                             int32_t is_new_page, int32_t num_kv, void* stream);

/* ---- Device-resident LayerPool management -------------------------------------------
 * Bookkeeping that the reference does on the host each decode step, done by the GPU so a
 * step needs no host reads, no uploads and can be recorded into a CUDA graph. */

/* Bulk construction of pool pages from encode output; replaces the per-page Python loop of
 * LayerPool.__init__ (sphkv_lut.py:37-68, arithmetic of :50-60).  r f32 and theta u8 are
 * [rows][code_stride], v_src [rows][v_stride] of v_dtype.  page_desc i32 [n_pages][4] =
 * {src_row, n_rows, G_t, dst_pid} (16-byte aligned): rows src_row .. src_row+n_rows fill the
 * first n_rows slots and G_t groups of page dst_pid; the rest of that page is zeroed.
 * Per page and group: scale = max(max_t r, 1e-8), code = clamp(rint(r / scale * 255)). */
int sphkv_pool_build_pages(const float* r, const uint8_t* theta, const void* v_src, int32_t v_dtype,
                           int64_t code_stride, int64_t v_stride, const int32_t* page_desc,
                           int32_t n_pages, uint8_t* theta_codes, uint8_t* radius_codes,
                           float* r_scales, void* v_pool, int32_t page_size, int32_t G_max,
                           int32_t dh, void* stream);

/* One decode-step append with the bookkeeping of LayerPool.append_and_compute
 * (sphkv_lut.py:150-186) on the device: state i32 [4] = {uniform context length, pages in
 * use, internal ticket (0 between calls), error flag}.  slot = ctx % page_size; when slot is 0
 * head h claims page used+h, writes block_table[h][ctx / page_size] and
 * bits_table[..] = dec_tier_idx and pids[h]; then the token is encoded and appended exactly as
 * sphkv_pool_encode_append does, ctx_lens[h] += 1, and the state advances.  A step that
 * would exceed n_pool_pages or max_blocks changes nothing except state[3] = 1, after which
 * every later step is a no-op; the caller reads state[3] whenever it next synchronises. */
int sphkv_pool_append_step(const float* k_post, const float* v_new, const float* decode_cb,
                           uint8_t* theta_codes, uint8_t* radius_codes, float* r_scales,
                           void* v_pool, int32_t* block_table, int32_t* bits_table,
                           int32_t* ctx_lens, int64_t* pids, int32_t* state, int32_t dec_tier_idx,
                           int32_t G, int32_t g, int32_t C, int32_t G_max, int32_t dh,
                           int32_t page_size, int32_t num_kv, int32_t max_blocks,
                           int32_t n_pool_pages, void* stream);

/* ---- Codebook training inner loop ----------------------------------------------------
 * Assignment + accumulation step of spherical_kmeans_gpu (codebooks/generate.py:47-58):
 * sims = U @ centers^T, assigns = argmax (first maximum), sums = index_add of U by assigns,
 * counts = bincount.  U f32 [N][d] (16-byte aligned), centers f32 [K][d], d in {8, 16, 32},
 * K * d * 8 + 12 * K + 2052 <= 49152.  assigns i32 [N]; best_sim f32 [N] optional (the similarity of
 * each point to its centre: sims.gather(1, assigns), used for the score at :71 and for
 * re-seeding empty clusters at :61-64); sums f32 [K][d] and counts i32 [K] are zeroed and
 * filled by the call.  Similarities use the encoder's fixed fp32 fma order; the order of
 * the float additions into sums is not fixed, as with index_add_ on a GPU. */
int sphkv_kmeans_assign(const float* U, int64_t N, int32_t d, const float* centers, int32_t K,
                        int32_t* assigns, float* best_sim, float* sums, int32_t* counts,
                        void* stream);

/* Implements the launcher new_fused_decode.cpp:3-22 declares and the reference never
 * defines: logits from a q.centroid table.  q_lut f32 [Hq][num_tiers][G_max][cb_size_max];
 * logits_out f32 [Hq][max_blocks*page_size]; holes, slots past ctx_lens and exact-zero
 * logits get -1e9. */
int sphkv_qlut_logits(const float* q_lut, const uint8_t* theta_codes, const uint8_t* radius_codes,
                      const float* r_scales, const int32_t* block_table, const int32_t* bits_table,
                      const int32_t* ctx_lens, float* logits_out, int32_t num_q_heads,
                      int32_t num_kv_heads, int32_t kv_groups, int32_t num_tiers,
                      int32_t max_blocks, int32_t page_size, int32_t G_max, int32_t cb_size_max,
                      float sm_scale, int32_t max_ctx, void* stream);

/* Implements fused_decode_ragged, which the reference calls
 * (spherical_kv_pipeline.py:1109-1125, 1866-1870, 1907-1910) and never defines: logits
 * over bit-packed byte pages of one tier with per-token back-rotation from the caller's
 * HF-layout cos/sin tables f32 [table_rows][dh].  codebooks f32 [num_kv*G][2^b_theta][g];
 * logits_out f32 [Hq][n_pages*page_size]. */
int sphkv_ragged_logits(const uint8_t* pages, const int32_t* ptable, const int32_t* head_ids,
                        const int32_t* positions, const float* cos_tbl, const float* sin_tbl,
                        const float* q, const float* codebooks, float* logits_out, int32_t grp,
                        int32_t num_kv, int32_t dh, int32_t G, int32_t g, int32_t b_theta,
                        int32_t page_size, int32_t n_pages, int32_t Hq, int32_t table_rows,
                        int32_t radius_fmt, int32_t reserved, void* stream);

/* Replaces _omega_ema_eager / _update_omega_gpu (spherical_kv_pipeline.py:952-987,
 * 1669-1701): page-level importance EMA from the per-block (m, l) the decode kernels emit.
 * ml: element (query head hq, block blk) at ml[(hq*max_blocks + blk)*stride + {0,1}] (stride =
 * dh+2 for partial_scratch of sphkv_pool_decode, 2 for page_ml of sphkv_decode_paged); omega
 * f32 [n_units][max_blocks] is updated in place: omega*beta + mean_group(mass)*(1-beta). */
int sphkv_omega_ema(const float* ml, float* omega, int32_t n_units, int32_t kv_groups,
                    int32_t max_blocks, int32_t stride, float beta, void* stream);

/* ---- Library ---------------------------------------------------------------------*/
int sphkv_abi_version(void);
const char* sphkv_last_error(void);
/* sizeof() of sphkv_tiers (0), sphkv_encode_params (1), sphkv_decode_params (2) as this
 * library was compiled; foreign-language bindings compare it with their own layout. */
int sphkv_struct_size(int which);
/* Number of SMs of the current device (grid sizing), or a negative error. */
int sphkv_sm_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SPHKV_H_ */
