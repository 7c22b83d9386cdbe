// Assignment + accumulation step of spherical k-means, the inner loop of codebook training
// (codebooks/generate.py:47-58): sims = U @ centers^T, assigns = argmax, per-cluster vector
// sums and counts.  The similarity search is the one of the page encoder: the dot product
// of a point with a centroid is an fp32 fma chain over d = 0..g-1 starting from 0, centroids
// are visited in ascending order and the first maximum wins (torch.argmax convention).
//
// One thread holds kPts points in registers and walks the centroids out of shared memory
// (one broadcast 16-byte load feeds 16 or 8 FMAs).  The accumulation uses no float atomics:
// per pass of 1024 (512) points a CTA counting-sorts the point ids by cluster in shared memory
// (integer atomics give each point its rank), then every (cluster, dimension) pair is summed
// by one thread walking its cluster's id list and re-reading the rows (L1/L2 hits).  The
// rank order inside a cluster is not fixed, so -- as with index_add_ on a GPU -- sums agree to
// rounding while assignments and counts are exact.  Per-CTA sums go to global memory once.
#include "common.cuh"

namespace sphkv {

constexpr int kKmThreads = 256;
// points per thread: 4 (2 for 32-dim points) keeps the kernel at two CTAs per SM
__host__ __device__ constexpr int pts_for(int d) { return d >= 32 ? 2 : 4; }

template <int D>
__global__ void __launch_bounds__(kKmThreads, 2) kmeans_assign_kernel(
    const float* __restrict__ U, int64_t N, const float* __restrict__ centers, int K,
    int32_t* __restrict__ assigns, float* __restrict__ best_sim, float* __restrict__ sums,
    int32_t* __restrict__ counts, int64_t pts_per_cta) {
  constexpr int kPts = pts_for(D);
  constexpr int P = kKmThreads * kPts;  // points per pass
  extern __shared__ __align__(16) float sm[];
  float* c_s = sm;                                      // [K][D] centres
  float* sum_s = sm + K * D;                            // [K][D] this CTA's sums
  int* cnt_s = reinterpret_cast<int*>(sum_s + K * D);   // [K] counts of the current pass
  int* tot_s = cnt_s + K;                               // [K] counts of all passes
  int* off_s = tot_s + K;                               // [K + 1] start of each cluster's id list
  uint16_t* order_s = reinterpret_cast<uint16_t*>(off_s + K + 1);  // [P] point ids sorted by cluster
  for (int i = threadIdx.x; i < K * D; i += blockDim.x) {
    c_s[i] = centers[i];
    sum_s[i] = 0.f;
  }
  for (int i = threadIdx.x; i < K; i += blockDim.x) cnt_s[i] = tot_s[i] = 0;
  __syncthreads();

  const int64_t first = (int64_t)blockIdx.x * pts_per_cta;
  const int64_t last = first + pts_per_cta < N ? first + pts_per_cta : N;
  for (int64_t base = first; base < last; base += P) {
    float u[kPts][D];
    bool live[kPts];
#pragma unroll
    for (int h = 0; h < kPts; ++h) {
      const int64_t idx = base + threadIdx.x + h * kKmThreads;  // coalesced across the CTA
      live[h] = idx < last;
      if (live[h]) {
        const float4* src = reinterpret_cast<const float4*>(U + idx * D);
#pragma unroll
        for (int q = 0; q < D / 4; ++q) {
          const float4 v = __ldg(src + q);
          u[h][4 * q] = v.x; u[h][4 * q + 1] = v.y; u[h][4 * q + 2] = v.z; u[h][4 * q + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < D; ++i) u[h][i] = 0.f;
      }
    }
    float best[kPts];
    int code[kPts];
#pragma unroll
    for (int h = 0; h < kPts; ++h) { best[h] = -INFINITY; code[h] = 0; }
    SPHKV_UNROLL_SEARCH
    for (int c = 0; c < K; ++c) {
      const float4* row = reinterpret_cast<const float4*>(c_s + c * D);
      float acc[kPts];
#pragma unroll
      for (int h = 0; h < kPts; ++h) acc[h] = 0.f;
#pragma unroll
      for (int q = 0; q < D / 4; ++q) {
        const float4 v = row[q];
#pragma unroll
        for (int h = 0; h < kPts; ++h) {
          acc[h] = __fmaf_rn(u[h][4 * q], v.x, acc[h]);
          acc[h] = __fmaf_rn(u[h][4 * q + 1], v.y, acc[h]);
          acc[h] = __fmaf_rn(u[h][4 * q + 2], v.z, acc[h]);
          acc[h] = __fmaf_rn(u[h][4 * q + 3], v.w, acc[h]);
        }
      }
#pragma unroll
      for (int h = 0; h < kPts; ++h)
        if (acc[h] > best[h]) { best[h] = acc[h]; code[h] = c; }
    }
    // rank of each point inside its cluster, results out
    int rank[kPts];
#pragma unroll
    for (int h = 0; h < kPts; ++h) {
      rank[h] = 0;
      if (live[h]) {
        const int64_t idx = base + threadIdx.x + h * kKmThreads;
        assigns[idx] = code[h];
        if (best_sim != nullptr) best_sim[idx] = best[h];
        rank[h] = atomicAdd(&cnt_s[code[h]], 1);
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {  // exclusive prefix of the K counts by one warp
      int carry = 0;
      for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + threadIdx.x;
        const int v = k < K ? cnt_s[k] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, incl, o);
          if ((int)threadIdx.x >= o) incl += t;
        }
        if (k < K) off_s[k] = carry + incl - v;
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (threadIdx.x == 0) off_s[K] = carry;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < kPts; ++h)
      if (live[h]) order_s[off_s[code[h]] + rank[h]] = (uint16_t)(threadIdx.x + h * kKmThreads);
    __syncthreads();
    for (int q = threadIdx.x; q < K * D; q += blockDim.x) {
      const int k = q / D, i = q - k * D;
      float acc = 0.f;
      for (int jj = off_s[k]; jj < off_s[k + 1]; ++jj) acc += __ldg(U + (base + order_s[jj]) * D + i);
      sum_s[q] += acc;
    }
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      tot_s[k] += cnt_s[k];
      cnt_s[k] = 0;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < K * D; i += blockDim.x)
    if (sum_s[i] != 0.f) atomicAdd(sums + i, sum_s[i]);
  for (int i = threadIdx.x; i < K; i += blockDim.x)
    if (tot_s[i] != 0) atomicAdd(counts + i, tot_s[i]);
}

}  // namespace sphkv

using namespace sphkv;

extern "C" int sphkv_kmeans_assign(const float* U, int64_t N, int32_t d, const float* centers, int32_t K,
                                   int32_t* assigns, float* best_sim, float* sums, int32_t* counts,
                                   void* stream) {
  SPHKV_REQUIRE(U && centers && assigns && sums && counts, SPHKV_E_ARG, "kmeans_assign: NULL pointer");
  SPHKV_REQUIRE(N >= 0 && (d == 8 || d == 16 || d == 32) && K >= 1 && K <= 256, SPHKV_E_ARG,
                "kmeans_assign: N=%lld d=%d (8, 16 or 32) K=%d (1..256)", (long long)N, d, K);
  SPHKV_REQUIRE((reinterpret_cast<uintptr_t>(U) & 15) == 0, SPHKV_E_ARG, "kmeans_assign: U must be 16-byte aligned");
  const int sms = sphkv_sm_count();
  SPHKV_REQUIRE(sms > 0, SPHKV_E_ARG, "kmeans_assign: cannot resolve the SM count");
  // a few CTAs per SM, each over a contiguous run of points that is a multiple of one pass
  const int64_t pass = (int64_t)kKmThreads * pts_for(d);
  int64_t ctas = (N + pass - 1) / pass;
  if (ctas < 1) ctas = 1;  // N == 0 returns after the memsets below
  if (ctas > (int64_t)sms * 8) ctas = (int64_t)sms * 8;
  const int64_t per = ((N + ctas - 1) / ctas + pass - 1) / pass * pass;
  ctas = (N + per - 1) / per;
  const size_t smem = (size_t)K * d * 8 + (size_t)(3 * K + 1) * 4 + (size_t)kKmThreads * pts_for(d) * 2;
  SPHKV_REQUIRE(smem <= 48 * 1024, SPHKV_E_LIMIT, "kmeans_assign: K=%d x d=%d needs %zu B of shared memory (limit 49152)",
                K, d, smem);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(float) * K * d, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(counts, 0, sizeof(int32_t) * K, st);
  if (e != cudaSuccess) {
    set_error("kmeans_assign: cudaMemsetAsync: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (N == 0) return SPHKV_OK;
  if (d == 8)
    kmeans_assign_kernel<8><<<(unsigned)ctas, kKmThreads, smem, st>>>(U, N, centers, K, assigns, best_sim, sums, counts, per);
  else if (d == 16)
    kmeans_assign_kernel<16><<<(unsigned)ctas, kKmThreads, smem, st>>>(U, N, centers, K, assigns, best_sim, sums, counts, per);
  else
    kmeans_assign_kernel<32><<<(unsigned)ctas, kKmThreads, smem, st>>>(U, N, centers, K, assigns, best_sim, sums, counts, per);
  return check_launch("kmeans_assign_kernel");
}
