// Row-wise top-k by radix select (aten.topk, largest, sorted).
//
// Keys are the order-preserving unsigned image of the fp32 value (NaN above +inf, as torch
// orders them).  One thread-block cluster handles a row: every CTA histograms the top 11 key
// bits of its slice, the histograms are merged into the leader CTA through distributed shared
// memory, and the leader finds the bin holding the k-th largest key.  A second pass over the
// slices sends every element above that bin straight to the result list and the elements of
// the bin to a small candidate list, both in the leader's shared memory.  The leader sorts the
// candidates, takes what is still missing, sorts the result (value descending, index ascending
// among equal values) and writes it.  HBM sees the row once; the second pass is served by L2.
// When the threshold bin holds more than kCandMax elements (for example a constant row) the
// leader finishes the row alone with two more radix passes and an index-ordered tie pick.
//
// Small k (the sampling case, k = 50 of 128256) takes a cheaper first pass, topk_sel_kernel:
// the histogram is built from one key per thread, the largest of the elements the thread read.
// The k-th largest of those thread maxima is a lower bound of the k-th largest element (they are
// k distinct elements), so every element of the answer lies in a bin at or above the bin of that
// bound; the second pass collects exactly those elements (a few more than k) and the leader sorts
// them.  This keeps the radix-select structure but takes the shared-memory atomics, which
// serialise when most keys fall into a handful of exponent bins, out of the streaming pass.
#include "common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;
namespace kuiops {

constexpr int kTopkThreads = 1024;
constexpr int kBins = 2048;
constexpr int kCandMax = 2048;
constexpr int kTopkMaxK = 2048;

__device__ __forceinline__ uint32_t key_of(float v) {
  if (v != v) return 0xFFFFFFFFu;
  uint32_t u = __float_as_uint(v + 0.f);       // -0 and +0 compare equal: both take the key of +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
// (key, index) packed so that a descending sort yields value-descending, index-ascending
__device__ __forceinline__ unsigned long long pack(uint32_t key, uint32_t idx) {
  return (static_cast<unsigned long long>(key) << 32) | uint32_t(~idx);
}

// One histogram increment per key.  (Electing one lane per distinct bin with match.any was
// measured 2.7x slower than letting the shared-memory atomic unit serialise the duplicates.)
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t bin, bool valid) {
  if (valid) atomicAdd(&hist[bin], 1u);
}

struct TopkShared {
  uint32_t hist[kBins];
  unsigned long long cand[kCandMax];
  unsigned long long sel[kTopkMaxK];
  uint32_t warp_tot[32];
  uint32_t sel_cnt, cand_cnt;
  uint32_t bin, need, bin_cnt;     // threshold bin, how many of it are needed, how many it holds
  uint32_t scan_base;
};

// Suffix scan of hist (2 bins per thread, 1024 threads): find the bin b with
// count(bins > b) < need <= count(bins >= b).  Writes sh.bin / sh.need / sh.bin_cnt.
__device__ void find_threshold_bin(TopkShared& sh, uint32_t need) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const uint32_t h0 = sh.hist[2 * tid], h1 = sh.hist[2 * tid + 1];
  const uint32_t local = h0 + h1;
  // inclusive suffix sum over threads (thread t covers bins 2t, 2t+1; higher t = larger keys)
  uint32_t v = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_down_sync(0xffffffffu, v, o);
    if (lane + o < 32) v += t;
  }
  if (lane == 0) sh.warp_tot[w] = v;
  __syncthreads();
  uint32_t above_warps = 0;
  for (int ww = w + 1; ww < 32; ++ww) above_warps += sh.warp_tot[ww];
  const uint32_t incl = v + above_warps;       // elements in bins >= 2*tid
  const uint32_t above = incl - local;         // elements in bins >= 2*tid + 2
  if (above < need && need <= above + h1) {
    sh.bin = 2 * tid + 1; sh.need = need - above; sh.bin_cnt = h1;
  } else if (above + h1 < need && need <= incl) {
    sh.bin = 2 * tid; sh.need = need - above - h1; sh.bin_cnt = h0;
  }
  __syncthreads();
}

// In-place descending bitonic sort of the first pow2 entries (entries beyond cnt are 0).
__device__ void sort_desc(unsigned long long* a, uint32_t cnt) {
  uint32_t pow2 = 1;
  while (pow2 < cnt) pow2 <<= 1;
  for (uint32_t i = cnt + threadIdx.x; i < pow2; i += blockDim.x) a[i] = 0ull;
  __syncthreads();
  for (uint32_t k = 2; k <= pow2; k <<= 1) {
    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
      for (uint32_t i = threadIdx.x; i < pow2; i += blockDim.x) {
        const uint32_t l = i ^ j;
        if (l > i) {
          const unsigned long long x = a[i], y = a[l];
          const bool desc = (i & k) == 0;
          if ((x < y) == desc) { a[i] = y; a[l] = x; }
        }
      }
      __syncthreads();
    }
  }
}

// Leader-only slow path over the whole row: the 11-bit bin is known (sh.bin / sh.need) and
// holds too many elements.  Two more radix passes over global memory pin the exact key, then
// elements above it are appended and ties are taken in index order.
__device__ void finish_row_slow(TopkShared& sh, const float* __restrict__ x, uint32_t n, uint32_t k) {
  const int tid = threadIdx.x;
  uint32_t prefix = sh.bin << 21, mask = 0xFFE00000u;
  uint32_t need = sh.need;
  const int shifts[2] = {10, 0};
  const int widths[2] = {11, 10};
  for (int p = 0; p < 2; ++p) {
    for (int i = tid; i < kBins; i += blockDim.x) sh.hist[i] = 0;
    __syncthreads();
    const uint32_t dm = (1u << widths[p]) - 1u;
    for (uint32_t i = tid; i < n; i += blockDim.x) {
      const uint32_t key = key_of(x[i]);
      if ((key & mask) == prefix) atomicAdd(&sh.hist[(key >> shifts[p]) & dm], 1u);
    }
    __syncthreads();
    find_threshold_bin(sh, need);
    prefix |= sh.bin << shifts[p];
    mask |= dm << shifts[p];
    need = sh.need;
    __syncthreads();
  }
  const uint32_t T = prefix;              // exact key of the k-th largest element
  const uint32_t ties_total = sh.bin_cnt; // elements equal to it
  // everything strictly above T (the first pass already took the bins above the 11-bit bin)
  const uint32_t coarse = T >> 21;
  for (uint32_t i = tid; i < n; i += blockDim.x) {
    const uint32_t key = key_of(x[i]);
    if (key > T && (key >> 21) == coarse) {
      const uint32_t pos = atomicAdd(&sh.sel_cnt, 1u);
      if (pos < k) sh.sel[pos] = pack(key, i);
    }
  }
  __syncthreads();
  if (ties_total == need) {
    for (uint32_t i = tid; i < n; i += blockDim.x) {
      if (key_of(x[i]) == T) {
        const uint32_t pos = atomicAdd(&sh.sel_cnt, 1u);
        if (pos < k) sh.sel[pos] = pack(T, i);
      }
    }
    __syncthreads();
    return;
  }
  // more ties than needed: take the `need` lowest indices, chunk by chunk in index order
  if (tid == 0) sh.scan_base = 0;
  __syncthreads();
  const int lane = tid & 31, w = tid >> 5;
  for (uint32_t base = 0; base < n; base += blockDim.x) {
    const uint32_t i = base + tid;
    const bool hit = i < n && key_of(x[i]) == T;
    const uint32_t ballot = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) sh.warp_tot[w] = __popc(ballot);
    __syncthreads();
    uint32_t before = sh.scan_base;
    for (int ww = 0; ww < w; ++ww) before += sh.warp_tot[ww];
    const uint32_t rank = before + __popc(ballot & ((1u << lane) - 1u));
    if (hit && rank < need) {
      const uint32_t pos = atomicAdd(&sh.sel_cnt, 1u);
      if (pos < k) sh.sel[pos] = pack(T, i);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t tot = 0;
      for (int ww = 0; ww < 32; ++ww) tot += sh.warp_tot[ww];
      sh.scan_base += tot;
    }
    __syncthreads();
    if (sh.scan_base >= need) break;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kTopkThreads)
topk_rows_kernel(uint32_t m, uint32_t n, uint32_t k, const float* __restrict__ X, float* __restrict__ values,
                 int64_t* __restrict__ indices, uint32_t cluster_ctas) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TopkShared& sh = *reinterpret_cast<TopkShared*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t part = cluster_ctas > 1 ? cluster.block_rank() : 0;
  const uint32_t row = blockIdx.x / cluster_ctas;
  const bool leader = part == 0;
  TopkShared* lead = cluster_ctas > 1 ? cluster.map_shared_rank(&sh, 0) : &sh;
  const int tid = threadIdx.x;
  const float* x = X + size_t(row) * n;

  // slice of this CTA, in whole float4s so vector loads stay aligned when the row is
  const uint32_t nv_total = (n + 3) / 4;
  const uint32_t nv_per = (nv_total + cluster_ctas - 1) / cluster_ctas;
  const uint32_t lo = min(part * nv_per * 4, n), hi = min(lo + nv_per * 4, n);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;

  for (int i = tid; i < kBins; i += blockDim.x) sh.hist[i] = 0;
  if (tid == 0) { sh.sel_cnt = 0; sh.cand_cnt = 0; sh.bin = 0; sh.need = 0; sh.bin_cnt = 0; }
  __syncthreads();
  pdl_wait();
  pdl_trigger();

  // ---- pass 1: histogram of the top 11 key bits over the slice -------------------------
  // (uniform trip counts: hist_add is warp-collective; four 16-byte loads in flight per thread)
  if (vec_ok) {
    const uint32_t nvec = (hi - lo) / 4;
    const uint32_t nt = blockDim.x;
    for (uint32_t v0 = 0; v0 < nvec; v0 += 4 * nt) {
      float4 f[4];
      bool ok[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t v = v0 + u * nt + tid;
        ok[u] = v < nvec;
        f[u] = ok[u] ? __ldcs(reinterpret_cast<const float4*>(x + lo + size_t(v) * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        hist_add(sh.hist, key_of(f[u].x) >> 21, ok[u]);
        hist_add(sh.hist, key_of(f[u].y) >> 21, ok[u]);
        hist_add(sh.hist, key_of(f[u].z) >> 21, ok[u]);
        hist_add(sh.hist, key_of(f[u].w) >> 21, ok[u]);
      }
    }
    for (uint32_t i0 = lo + nvec * 4; i0 < hi; i0 += nt) {
      const uint32_t i = i0 + tid;
      const bool v = i < hi;
      hist_add(sh.hist, v ? key_of(x[i]) >> 21 : 0u, v);
    }
  } else {
    for (uint32_t i0 = lo; i0 < hi; i0 += blockDim.x) {
      const uint32_t i = i0 + tid;
      const bool v = i < hi;
      hist_add(sh.hist, v ? key_of(x[i]) >> 21 : 0u, v);
    }
  }
  __syncthreads();
  if (cluster_ctas > 1) {
    cluster.sync();                        // the leader's histogram is initialised and filled
    if (!leader) {
      for (int i = tid; i < kBins; i += blockDim.x) {
        const uint32_t c = sh.hist[i];
        if (c) atomicAdd(&lead->hist[i], c);
      }
    }
    cluster.sync();
  }
  if (leader) find_threshold_bin(sh, k);
  if (cluster_ctas > 1) cluster.sync();
  const uint32_t bin = lead->bin, bin_cnt = lead->bin_cnt;
  const bool fast = bin_cnt <= uint32_t(kCandMax);

  // ---- pass 2: scatter the slice into the leader's result / candidate lists ------------
  if (fast) {
    auto route = [&](float v, uint32_t i) {
      const uint32_t key = key_of(v), b = key >> 21;
      if (b > bin) {
        const uint32_t pos = atomicAdd(&lead->sel_cnt, 1u);
        if (pos < k) lead->sel[pos] = pack(key, i);
      } else if (b == bin) {
        const uint32_t pos = atomicAdd(&lead->cand_cnt, 1u);
        if (pos < uint32_t(kCandMax)) lead->cand[pos] = pack(key, i);
      }
    };
    if (vec_ok) {
      const uint32_t nvec = (hi - lo) / 4;
      const uint32_t nt = blockDim.x;
      for (uint32_t v0 = tid; v0 < nvec; v0 += 4 * nt) {
        float4 f[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * nt < nvec) f[u] = *reinterpret_cast<const float4*>(x + lo + size_t(v0 + u * nt) * 4);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * nt < nvec) {
            const uint32_t i0 = lo + (v0 + u * nt) * 4;
            route(f[u].x, i0); route(f[u].y, i0 + 1); route(f[u].z, i0 + 2); route(f[u].w, i0 + 3);
          }
      }
      for (uint32_t i = lo + nvec * 4 + tid; i < hi; i += blockDim.x) route(x[i], i);
    } else {
      for (uint32_t i = lo + tid; i < hi; i += blockDim.x) route(x[i], i);
    }
  }
  if (cluster_ctas > 1) cluster.sync();    // all remote writes landed; followers may leave
  if (!leader) return;
  __syncthreads();

  if (fast) {
    const uint32_t need = sh.need;
    const uint32_t ccnt = min(sh.cand_cnt, uint32_t(kCandMax));
    sort_desc(sh.cand, ccnt);
    const uint32_t base = sh.sel_cnt;      // == k - need
    for (uint32_t i = tid; i < need; i += blockDim.x)
      if (base + i < k) sh.sel[base + i] = sh.cand[i];
    __syncthreads();
  } else {
    // bins above the threshold bin first, then the slow exact finish
    for (uint32_t i = tid; i < n; i += blockDim.x) {
      const uint32_t key = key_of(x[i]);
      if ((key >> 21) > bin) {
        const uint32_t pos = atomicAdd(&sh.sel_cnt, 1u);
        if (pos < k) sh.sel[pos] = pack(key, i);
      }
    }
    __syncthreads();
    finish_row_slow(sh, x, n, k);
  }
  sort_desc(sh.sel, k);
  for (uint32_t i = tid; i < k; i += blockDim.x) {
    const uint32_t idx = ~uint32_t(sh.sel[i] & 0xFFFFFFFFull);
    values[size_t(row) * k + i] = x[idx];
    indices[size_t(row) * k + i] = int64_t(idx);
  }
}

// Exact top-k of a whole row by one CTA (1024 threads), reading global memory: the fall-back of
// topk_sel_kernel when its candidate list overflows.  Leaves the unsorted answer in sh.sel.
__device__ void topk_row_single_cta(TopkShared& sh, const float* __restrict__ x, uint32_t n, uint32_t k) {
  const int tid = threadIdx.x;
  for (int i = tid; i < kBins; i += blockDim.x) sh.hist[i] = 0;
  if (tid == 0) { sh.sel_cnt = 0; sh.cand_cnt = 0; sh.bin = 0; sh.need = 0; sh.bin_cnt = 0; }
  __syncthreads();
  for (uint32_t i = tid; i < n; i += blockDim.x) atomicAdd(&sh.hist[key_of(x[i]) >> 21], 1u);
  __syncthreads();
  find_threshold_bin(sh, k);
  const uint32_t bin = sh.bin;
  const bool fits = sh.bin_cnt <= uint32_t(kCandMax);
  for (uint32_t i = tid; i < n; i += blockDim.x) {
    const uint32_t key = key_of(x[i]), b = key >> 21;
    if (b > bin) {
      const uint32_t pos = atomicAdd(&sh.sel_cnt, 1u);
      if (pos < k) sh.sel[pos] = pack(key, i);
    } else if (fits && b == bin) {
      const uint32_t pos = atomicAdd(&sh.cand_cnt, 1u);
      if (pos < uint32_t(kCandMax)) sh.cand[pos] = pack(key, i);
    }
  }
  __syncthreads();
  if (fits) {
    const uint32_t need = sh.need, base = sh.sel_cnt;
    sort_desc(sh.cand, min(sh.cand_cnt, uint32_t(kCandMax)));
    for (uint32_t i = tid; i < need; i += blockDim.x)
      if (base + i < k) sh.sel[base + i] = sh.cand[i];
    __syncthreads();
  } else {
    finish_row_slow(sh, x, n, k);
  }
}

__global__ void __launch_bounds__(kTopkThreads)
topk_sel_kernel(uint32_t m, uint32_t n, uint32_t k, const float* __restrict__ X, float* __restrict__ values,
                int64_t* __restrict__ indices, uint32_t cluster_ctas) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TopkShared& sh = *reinterpret_cast<TopkShared*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t part = cluster_ctas > 1 ? cluster.block_rank() : 0;
  const uint32_t row = blockIdx.x / cluster_ctas;
  const bool leader = part == 0;
  TopkShared* lead = cluster_ctas > 1 ? cluster.map_shared_rank(&sh, 0) : &sh;
  const int tid = threadIdx.x;
  const float* x = X + size_t(row) * n;
  const uint32_t nv_total = (n + 3) / 4;
  const uint32_t nv_per = (nv_total + cluster_ctas - 1) / cluster_ctas;
  const uint32_t lo = min(part * nv_per * 4, n), hi = min(lo + nv_per * 4, n);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  const uint32_t nvec = vec_ok ? (hi - lo) / 4 : 0;
  const uint32_t nt = blockDim.x;

  for (int i = tid; i < kBins; i += blockDim.x) sh.hist[i] = 0;
  if (tid == 0) { sh.sel_cnt = 0; sh.cand_cnt = 0; sh.bin = 0; sh.need = 0; sh.bin_cnt = 0; }
  __syncthreads();
  pdl_wait();
  pdl_trigger();

  // ---- pass 1: the largest value each thread meets (no atomics in the stream) -----------------
  // fmaxf skips NaNs, so a thread that saw NaNs reports a smaller value than its true maximum;
  // the bound below only needs "some element of the thread is at least this large", which holds.
  float fm = -INFINITY;
  bool saw = false;
  for (uint32_t v0 = tid; v0 < nvec; v0 += 4 * nt) {
    float4 f[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      f[u] = (v0 + u * nt < nvec) ? __ldcs(reinterpret_cast<const float4*>(x + lo + size_t(v0 + u * nt) * 4))
                                  : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
    for (int u = 0; u < 4; ++u) fm = fmaxf(fmaxf(fm, fmaxf(f[u].x, f[u].y)), fmaxf(f[u].z, f[u].w));
    saw = true;
  }
  for (uint32_t i = lo + nvec * 4 + tid; i < hi; i += nt) { fm = fmaxf(fm, x[i]); saw = true; }
  const uint32_t kmax = saw ? key_of(fm) : 0u;      // 0 is the key of no value: "this thread saw nothing"
  {
    // one histogram entry per thread, duplicates inside a warp combined first
    const uint32_t b = kmax >> 21;
    const uint32_t peers = __match_any_sync(0xffffffffu, kmax ? b : 0xFFFFFFFFu);
    if (kmax && (tid & 31) == __ffs(peers) - 1) atomicAdd(&sh.hist[b], uint32_t(__popc(peers)));
  }
  __syncthreads();
  if (cluster_ctas > 1) {
    cluster.sync();                        // the leader's histogram is initialised and filled
    if (!leader) {
      for (int i = tid; i < kBins; i += blockDim.x) {
        const uint32_t c = sh.hist[i];
        if (c) atomicAdd(&lead->hist[i], c);
      }
    }
    cluster.sync();
  }
  if (leader) find_threshold_bin(sh, k);   // fewer than k thread maxima: bin stays 0, everything is a candidate
  if (cluster_ctas > 1) cluster.sync();
  const uint32_t bin = lead->bin;

  // ---- pass 2 (served by L2): every element at or above the bound's bin goes to the leader ----
  // The bin's lower edge as a float: keys are monotonic in the value, so "key >= edge" is one
  // float compare; NaNs (the top keys) always qualify.
  const uint32_t edge = bin << 21;
  const bool nan_only = edge > 0xFF800000u;                       // above the key of +inf
  const float thr = edge >= 0x80000000u ? __uint_as_float(edge & 0x7FFFFFFFu)
                  : (edge < 0x00800000u ? -INFINITY : __uint_as_float(~edge));
  auto route = [&](float v, uint32_t i) {
    if (v != v || (!nan_only && v >= thr)) {
      const uint32_t pos = atomicAdd(&lead->cand_cnt, 1u);
      if (pos < uint32_t(kCandMax)) lead->cand[pos] = pack(key_of(v), i);
    }
  };
  for (uint32_t v0 = tid; v0 < nvec; v0 += 4 * nt) {
    float4 f[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v0 + u * nt < nvec) f[u] = *reinterpret_cast<const float4*>(x + lo + size_t(v0 + u * nt) * 4);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v0 + u * nt < nvec) {
        const uint32_t i0 = lo + (v0 + u * nt) * 4;
        route(f[u].x, i0); route(f[u].y, i0 + 1); route(f[u].z, i0 + 2); route(f[u].w, i0 + 3);
      }
  }
  for (uint32_t i = lo + nvec * 4 + tid; i < hi; i += nt) route(x[i], i);
  if (cluster_ctas > 1) cluster.sync();    // all remote writes landed; followers may leave
  if (!leader) return;
  __syncthreads();

  const uint32_t cnt = sh.cand_cnt;
  const unsigned long long* res = sh.cand;
  if (cnt <= uint32_t(kCandMax) && cnt >= k) {
    sort_desc(sh.cand, cnt);               // key descending, index ascending among equal keys
  } else {
    topk_row_single_cta(sh, x, n, k);
    sort_desc(sh.sel, k);
    res = sh.sel;
  }
  for (uint32_t i = tid; i < k; i += blockDim.x) {
    const uint32_t idx = ~uint32_t(res[i] & 0xFFFFFFFFull);
    values[size_t(row) * k + i] = x[idx];
    indices[size_t(row) * k + i] = int64_t(idx);
  }
}

}  // namespace kuiops

using namespace kuiops;

extern "C" int kuiops_topk_f32(uint32_t m, uint32_t n, uint32_t k, const void* X, void* values, int64_t* indices,
                               kuiops_stream_t s) {
  if (m == 0 || n == 0 || k == 0 || !X || !values || !indices) return KUIOPS_EINVAL;
  if (k > n) return KUIOPS_EINVAL;
  if (k > uint32_t(kTopkMaxK)) return KUIOPS_ELIMIT;
  // a cluster per row when rows are few and long, so that every SM streams part of the input
  uint32_t c = 1;
  while (c < 4 && uint64_t(m) * c * 2 <= uint64_t(num_sms()) && n / (c * 2) >= 16384) c *= 2;
  const size_t smem = sizeof(TopkShared);   // ~41 KB, below the 48 KB that needs no opt-in
  // few results per row: the thread-maxima bound is tight (the row has 1024 c thread maxima)
  if (k * 8 <= 1024 * c)
    return launch_cluster_pdl(topk_sel_kernel, dim3(m * c), dim3(kTopkThreads), smem, as_stream(s), c, m, n, k,
                              static_cast<const float*>(X), static_cast<float*>(values), indices, c);
  return launch_cluster_pdl(topk_rows_kernel, dim3(m * c), dim3(kTopkThreads), smem, as_stream(s), c, m, n, k,
                            static_cast<const float*>(X), static_cast<float*>(values), indices, c);
}
