// Inclusive prefix sum along the last axis of an [m, n] matrix (aten.cumsum over dim -1), fp32 and
// int64.  The reference only lists cumsum as backlog (KERNELS.md:68-90) and has no kernel.
//
// Reduce-then-scan over a cluster: a row is cut into one contiguous part per CTA of its cluster.
// Every CTA first sums its part with strided, coalesced loads, the parts' sums are exchanged through
// distributed shared memory, and each CTA then scans its part chunk by chunk (8 consecutive elements
// per thread) starting from the sum of the parts before it.  The second read of a part is served by
// L2 when the matrix fits there.  Rows are independent, so many short rows use clusters of one CTA
// and skip the first phase.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace kuiops {

constexpr int kScanThreads = 512;
constexpr int kScanPer = 8;                                   // consecutive elements per thread per chunk
constexpr uint32_t kScanChunk = kScanThreads * kScanPer;      // elements one CTA scans per round
constexpr int kScanMaxCluster = 8;

template <typename T> struct ScanAcc;
template <> struct ScanAcc<float> { using type = float; };
template <> struct ScanAcc<int64_t> { using type = unsigned long long; };   // wraps like the eager sum

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
cumsum_rows_kernel(uint32_t m, uint32_t n, const T* __restrict__ X, T* __restrict__ Y, uint32_t cluster_ctas) {
  using A = typename ScanAcc<T>::type;
  constexpr int VEC = 16 / sizeof(T);                         // elements per 16-byte access
  __shared__ A warp_tot[2][kScanThreads / 32];
  __shared__ A part_tot[kScanMaxCluster];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t part = cluster_ctas > 1 ? cluster.block_rank() : 0;
  const uint32_t row = blockIdx.x / cluster_ctas;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  (void)m;
  const T* x = X + size_t(row) * n;
  T* y = Y + size_t(row) * n;
  // parts are whole chunks, so that every chunk of a part starts on a 16-byte boundary of an aligned row
  const uint32_t chunks = (n + kScanChunk - 1) / kScanChunk;
  const uint32_t chunks_per = (chunks + cluster_ctas - 1) / cluster_ctas;
  const uint32_t lo = min(uint64_t(part) * chunks_per * kScanChunk, uint64_t(n));
  const uint32_t hi = min(uint64_t(lo) + uint64_t(chunks_per) * kScanChunk, uint64_t(n));
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
  pdl_wait();
  pdl_trigger();

  A carry = 0;
  if (cluster_ctas > 1) {
    // A CTA's shared memory may only be touched by its cluster peers once that CTA has started: every
    // CTA arrives here at entry and waits just before its first remote store, so the wait is covered
    // by the streaming of phase 1.
    cluster.barrier_arrive();
    // ---- phase 1: the sum of this part ----------------------------------------------------------
    A s = 0;
    const uint32_t nvec = vec_ok ? (hi - lo) / VEC : 0;
    for (uint32_t v = tid; v < nvec; v += kScanThreads) {
      const Vec16<T> q = ld16(x + lo + size_t(v) * VEC);
#pragma unroll
      for (int j = 0; j < VEC; ++j) s += A(q.v[j]);
    }
    for (uint32_t i = lo + nvec * VEC + tid; i < hi; i += kScanThreads) s += A(x[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) warp_tot[0][warp] = s;
    __syncthreads();
    cluster.barrier_wait();                // all peers are running: their shared memory exists
    if (tid == 0) {
      A t = 0;
      for (int w = 0; w < kScanThreads / 32; ++w) t += warp_tot[0][w];
      for (uint32_t r = 0; r < cluster_ctas; ++r) cluster.map_shared_rank(part_tot, r)[part] = t;
    }
    cluster.sync();                        // every part's sum has landed in every CTA
    for (uint32_t r = 0; r < part; ++r) carry += part_tot[r];
  }

  // ---- phase 2: scan the part chunk by chunk --------------------------------------------------
  uint32_t round = 0;
  for (uint32_t c0 = lo; c0 < hi; c0 += kScanChunk, ++round) {
    const uint32_t i0 = c0 + uint32_t(tid) * kScanPer;
    A e[kScanPer];
    if (vec_ok && i0 + kScanPer <= hi) {
#pragma unroll
      for (int q = 0; q < kScanPer / VEC; ++q) {
        const Vec16<T> v = ld16(x + i0 + q * VEC);
#pragma unroll
        for (int j = 0; j < VEC; ++j) e[q * VEC + j] = A(v.v[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < kScanPer; ++j) e[j] = (i0 + j < hi) ? A(x[i0 + j]) : A(0);
    }
#pragma unroll
    for (int j = 1; j < kScanPer; ++j) e[j] += e[j - 1];
    // exclusive offset of this thread inside the chunk
    A incl = e[kScanPer - 1];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const A up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    A excl = __shfl_up_sync(0xffffffffu, incl, 1);            // sum of the lanes before this one
    if (lane == 0) excl = 0;
    A (&wt)[kScanThreads / 32] = warp_tot[(round + 1) & 1];   // phase 1 used buffer 0 last
    if (lane == 31) wt[warp] = incl;
    __syncthreads();
    A before = carry, total = 0;
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; ++w) {
      const A t = wt[w];
      if (w < warp) before += t;
      total += t;
    }
    before += excl;
    carry += total;
    if (vec_ok && i0 + kScanPer <= hi) {
#pragma unroll
      for (int q = 0; q < kScanPer / VEC; ++q) {
        Vec16<T> v;
#pragma unroll
        for (int j = 0; j < VEC; ++j) v.v[j] = T(before + e[q * VEC + j]);
        st16(y + i0 + q * VEC, v);
      }
    } else {
#pragma unroll
      for (int j = 0; j < kScanPer; ++j)
        if (i0 + j < hi) y[i0 + j] = T(before + e[j]);
    }
  }
}

template <typename T>
static int cumsum_launch(uint32_t m, uint32_t n, const void* X, void* Y, cudaStream_t st) {
  if (m == 0 || n == 0 || !X || !Y) return KUIOPS_EINVAL;
  if (uint64_t(m) * n > (1ull << 31)) return KUIOPS_ELIMIT;
  // few long rows: a cluster per row, as long as the whole grid is resident (two CTAs per SM)
  uint32_t c = 1;
  while (c < uint32_t(kScanMaxCluster) && uint64_t(m) * c * 2 <= 2ull * num_sms() && n / (c * 2) >= kScanChunk) c *= 2;
  if (uint64_t(m) * c > 0x7FFFFFFFull) return KUIOPS_ELIMIT;   // one CTA per row part
  return launch_cluster_pdl(cumsum_rows_kernel<T>, dim3(m * c), dim3(kScanThreads), 0, st, c, m, n,
                            static_cast<const T*>(X), static_cast<T*>(Y), c);
}

}  // namespace kuiops

using namespace kuiops;

extern "C" {

int kuiops_cumsum_f32(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t s) {
  return cumsum_launch<float>(m, n, X, Y, as_stream(s));
}
int kuiops_cumsum_i64(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t s) {
  return cumsum_launch<int64_t>(m, n, X, Y, as_stream(s));
}

}  // extern "C"
