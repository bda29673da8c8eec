// Stable sort of every row of an [m, n] fp32 matrix with the permutation (aten.sort over the last
// axis: values + int64 indices), ascending or descending; equal values keep their original order,
// -0 equals +0, NaN is the largest value.  The reference only lists sort as backlog
// (KERNELS.md:68-90) and has no kernel.
//
// A cluster of 1..8 CTAs per row runs a least-significant-digit radix sort on order-preserving
// 32-bit keys, four passes of eight bits; every CTA owns one contiguous chunk of the row's
// positions.  The four digit histograms of the row are counted once up front (each CTA counts
// its chunk, the chunks' histograms are summed through distributed shared memory).  Before a
// pass every CTA counts the digits of its chunk in the current arrangement and reads the counts of
// the chunks before it from its peers: that gives the first output position of each digit for
// its chunk.  The pass then walks the chunk tile by tile; inside a tile the rank of an element
// among the equal digits before it is found per warp with lane votes plus a per-warp counter table
// in shared memory, the warps' tables are turned into offsets by one thread per digit, and the
// elements are scattered.  Keys and indices ping-pong between two caller-provided buffers; the
// first pass reads the input itself and the last pass writes the results.  Cluster barriers
// separate the passes (a pass reads what every CTA of the row wrote in the one before).
#include <atomic>
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace kuiops {

constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortItems = 8;                                  // elements per thread per tile
constexpr uint32_t kSortTile = kSortThreads * kSortItems;
constexpr int kSortDigits = 256;
constexpr int kSortPasses = 4;

struct SortShared {
  uint32_t hist[kSortPasses][kSortDigits];       // per pass: elements of the row with a smaller digit
  uint32_t warp_cnt[kSortWarps][kSortDigits];    // per tile: counts, then offsets inside the digit, per (warp, digit)
  uint32_t base[kSortDigits];                    // per pass: where the next element of a digit goes
  uint32_t tile_start[kSortDigits];              // per tile: first slot of a digit in the tile's sorted order
  int32_t delta[kSortDigits];                    // per tile: global position minus slot, per digit
  uint32_t warp_sum[kSortDigits / 32];
  uint32_t chunk_hist[kSortPasses][kSortDigits]; // this CTA's chunk: digit counts of the input, per pass (read by the peers once)
  uint32_t chunk_cnt[kSortDigits];               // this CTA's chunk: digit counts in the arrangement the current pass reads (read by the peers)
  uint2 slot[kSortTile];                         // the tile in sorted order: (key, index)
};

// Order-preserving key of a float: ascending keys are ascending values, -0 and +0 share a key and
// every NaN takes the largest one.  Descending order sorts the complemented key, which keeps
// equal values in their original order too.
__device__ __forceinline__ uint32_t sort_key(float v, bool descending) {
  uint32_t k;
  if (v != v) {
    k = 0xFFFFFFFFu;
  } else {
    const uint32_t u = __float_as_uint(v + 0.f);
    k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  }
  return descending ? ~k : k;
}

__global__ void __launch_bounds__(kSortThreads)
sort_rows_kernel(uint32_t n, int descending, const float* __restrict__ X, float* __restrict__ values,
                 int64_t* __restrict__ indices, uint2* buf_a, uint2* buf_b, uint32_t cluster_ctas) {
  extern __shared__ __align__(16) unsigned char sort_smem[];
  SortShared& sh = *reinterpret_cast<SortShared*>(sort_smem);
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t part = cluster_ctas > 1 ? cluster.block_rank() : 0;
  const uint32_t row = blockIdx.x / cluster_ctas;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t off = size_t(row) * n;
  const float* x = X + off;
  const bool desc = descending != 0;
  // this CTA's chunk of the row's positions
  const uint32_t chunk = (n + cluster_ctas - 1) / cluster_ctas;
  const uint32_t lo = min(uint64_t(part) * chunk, uint64_t(n)), hi = min(uint64_t(lo) + chunk, uint64_t(n));
  pdl_wait();
  pdl_trigger();

  // ---- the four digit histograms: of this chunk, then of the row --------------------------------
  static_assert(kSortPasses * kSortDigits == kSortThreads, "one histogram entry per thread");
  (&sh.chunk_hist[0][0])[tid] = 0;
  __syncthreads();
  for (uint32_t i0 = lo; i0 < hi; i0 += kSortTile) {
    // all loads of a tile in flight before the first shared-memory atomic
    float v[kSortItems];
#pragma unroll
    for (int j = 0; j < kSortItems; ++j) {
      const uint32_t i = i0 + uint32_t(j) * kSortThreads + tid;
      v[j] = i < hi ? x[i] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kSortItems; ++j) {
      if (i0 + uint32_t(j) * kSortThreads + tid < hi) {
        const uint32_t k = sort_key(v[j], desc);
#pragma unroll
        for (int p = 0; p < kSortPasses; ++p) atomicAdd(&sh.chunk_hist[p][(k >> (8 * p)) & 255u], 1u);
      }
    }
  }
  __syncthreads();
  if (tid < kSortDigits) sh.chunk_cnt[tid] = sh.chunk_hist[0][tid];      // pass 0 reads the input: its chunk counts are known already
  if (cluster_ctas > 1) {
    cluster.sync();                                                       // every chunk's histograms are complete (and every peer is running)
    uint32_t sum = 0;
    for (uint32_t r = 0; r < cluster_ctas; ++r) sum += (&cluster.map_shared_rank(&sh.chunk_hist[0][0], r)[0])[tid];
    (&sh.hist[0][0])[tid] = sum;
  } else {
    (&sh.hist[0][0])[tid] = (&sh.chunk_hist[0][0])[tid];
  }
  __syncthreads();
  if (warp < kSortPasses) {
    // exclusive prefix over the 256 digits of pass `warp`: eight digits per lane
    uint32_t c[8], s = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) { c[q] = sh.hist[warp][lane * 8 + q]; s += c[q]; }
    uint32_t incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    uint32_t run = incl - s;
#pragma unroll
    for (int q = 0; q < 8; ++q) { sh.hist[warp][lane * 8 + q] = run; run += c[q]; }
  }
  __syncthreads();

  // ---- four scatter passes ----------------------------------------------------------------------
  for (int pass = 0; pass < kSortPasses; ++pass) {
    const uint32_t shift = 8u * pass;
    const uint2* src = (pass == 2 ? buf_b : buf_a) + off;                // pass 0 reads x instead
    uint2* dst = (pass == 1 ? buf_b : buf_a) + off;                      // pass 3 writes the results instead
    if (pass > 0 && cluster_ctas > 1) {
      // digit counts of this chunk in the arrangement this pass reads (a row with one CTA needs none:
      // nothing comes before its only chunk)
      if (tid < kSortDigits) sh.chunk_cnt[tid] = 0;
      __syncthreads();
      for (uint32_t i0 = lo; i0 < hi; i0 += kSortTile) {
        uint32_t k[kSortItems];
#pragma unroll
        for (int j = 0; j < kSortItems; ++j) {
          const uint32_t i = i0 + uint32_t(j) * kSortThreads + tid;
          k[j] = i < hi ? src[i].x : 0u;
        }
#pragma unroll
        for (int j = 0; j < kSortItems; ++j)
          if (i0 + uint32_t(j) * kSortThreads + tid < hi) atomicAdd(&sh.chunk_cnt[(k[j] >> shift) & 255u], 1u);
      }
      __syncthreads();
    }
    if (cluster_ctas > 1) cluster.sync();                                 // the peers' counts for this pass are complete
    if (tid < kSortDigits) {
      // first output position of a digit for this chunk: the digit's start in the row plus what the chunks before hold
      uint32_t b = sh.hist[pass][tid];
      for (uint32_t r = 0; r < part; ++r) b += cluster.map_shared_rank(&sh.chunk_cnt[0], r)[tid];
      sh.base[tid] = b;                                                   // read again by the same thread only
    }
    for (uint32_t tile0 = lo; tile0 < hi; tile0 += kSortTile) {
#pragma unroll
      for (int q = 0; q < kSortDigits / 32; ++q) sh.warp_cnt[warp][lane + 32 * q] = 0;
      // element order inside the tile: warp, then j, then lane
      uint32_t key[kSortItems], idx[kSortItems], rank[kSortItems];
#pragma unroll
      for (int j = 0; j < kSortItems; ++j) {
        const uint32_t e = tile0 + uint32_t(warp) * (32 * kSortItems) + uint32_t(j) * 32 + lane;
        key[j] = 0; idx[j] = e;
        if (e < hi) {
          if (pass == 0) key[j] = sort_key(x[e], desc);
          else { const uint2 kv = src[e]; key[j] = kv.x; idx[j] = kv.y; }
        }
      }
      __syncwarp();                                   // the zeroed counters are visible to the warp
#pragma unroll
      for (int j = 0; j < kSortItems; ++j) {
        const uint32_t e = tile0 + uint32_t(warp) * (32 * kSortItems) + uint32_t(j) * 32 + lane;
        const bool valid = e < hi;
        const uint32_t d = (key[j] >> shift) & 255u;
        // the lanes that hold the same digit: nine votes instead of match.any, whose cost grows with
        // the number of distinct values in the warp (nearly 32 for random digits); lanes past the end
        // match only each other
        uint32_t peers = __ballot_sync(0xffffffffu, valid);
        if (!valid) peers = ~peers;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const bool bit = (d >> b) & 1u;
          const uint32_t vote = __ballot_sync(0xffffffffu, bit);
          peers &= bit ? vote : ~vote;
        }
        const int leader = __ffs(peers) - 1;
        uint32_t before = 0;
        if (lane == leader && valid) {
          before = sh.warp_cnt[warp][d];
          sh.warp_cnt[warp][d] = before + __popc(peers);
        }
        before = __shfl_sync(0xffffffffu, before, leader);
        rank[j] = before + __popc(peers & ((1u << lane) - 1u));
        __syncwarp();                                 // the next step reads the counter this one wrote
      }
      __syncthreads();                                // every warp's counts of this tile are final
      // One thread per digit: the warps' counts become offsets inside the digit, the digits' totals
      // become the tile's sorted layout (an exclusive scan over the 256 digits).
      uint32_t total = 0, incl = 0;
      if (tid < kSortDigits) {
        for (int w = 0; w < kSortWarps; ++w) {
          const uint32_t c = sh.warp_cnt[w][tid];
          sh.warp_cnt[w][tid] = total;
          total += c;
        }
        incl = total;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += up;
        }
        if (lane == 31) sh.warp_sum[warp] = incl;
      }
      __syncthreads();
      if (tid < kSortDigits) {
        uint32_t start = incl - total;
        for (int w = 0; w < warp; ++w) start += sh.warp_sum[w];
        sh.tile_start[tid] = start;
        const uint32_t b = sh.base[tid];
        sh.delta[tid] = int32_t(b - start);
        sh.base[tid] = b + total;
      }
      __syncthreads();
      // into the tile's sorted order in shared memory ...
#pragma unroll
      for (int j = 0; j < kSortItems; ++j) {
        const uint32_t e = tile0 + uint32_t(warp) * (32 * kSortItems) + uint32_t(j) * 32 + lane;
        if (e < hi) {
          const uint32_t d = (key[j] >> shift) & 255u;
          sh.slot[sh.tile_start[d] + sh.warp_cnt[warp][d] + rank[j]] = make_uint2(key[j], idx[j]);
        }
      }
      __syncthreads();
      // ... and out: neighbouring threads write neighbouring positions of a digit's run
      const uint32_t in_tile = min(kSortTile, hi - tile0);
#pragma unroll
      for (int q = 0; q < kSortItems; ++q) {
        const uint32_t l = uint32_t(q) * kSortThreads + tid;
        if (l < in_tile) {
          const uint2 kv = sh.slot[l];
          const uint32_t pos = uint32_t(int32_t(l) + sh.delta[(kv.x >> shift) & 255u]);
          if (pass == kSortPasses - 1) {
            values[off + pos] = x[kv.y];
            indices[off + pos] = int64_t(kv.y);
          } else {
            dst[pos] = kv;
          }
        }
      }
      __syncthreads();                                // tables and slots consumed before the next tile; stores ordered for the next pass
    }
    // the next pass reads what every CTA of the row wrote in this one, and overwrites the counts the
    // peers have just read
    if (cluster_ctas > 1) cluster.sync();
  }
}

}  // namespace kuiops

using namespace kuiops;

extern "C" {

size_t kuiops_sort_workspace_bytes(uint32_t m, uint32_t n) { return size_t(m) * n * 16; }

int kuiops_sort_f32(uint32_t m, uint32_t n, int descending, const void* X, void* values, int64_t* indices,
                    void* workspace, size_t workspace_bytes, kuiops_stream_t s) {
  if (m == 0 || n == 0 || !X || !values || !indices) return KUIOPS_EINVAL;
  if (uint64_t(m) * n > (1ull << 31) || m > 0x7FFFFFFFu) return KUIOPS_ELIMIT;
  if (!workspace || workspace_bytes < kuiops_sort_workspace_bytes(m, n)) return KUIOPS_EWORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 7u) return KUIOPS_EINVAL;
  {
    // the last pass gathers from X while it writes the values: the two must not overlap
    const uintptr_t a = reinterpret_cast<uintptr_t>(X), b = reinterpret_cast<uintptr_t>(values);
    const uintptr_t bytes = uintptr_t(m) * n * sizeof(float);
    if (a < b + bytes && b < a + bytes) return KUIOPS_EINVAL;
  }
  const size_t cells = size_t(m) * n;
  uint2* w = static_cast<uint2*>(workspace);
  static std::atomic<uint64_t> configured{0};      // the opt-in for large dynamic shared memory is per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return KUIOPS_ELAUNCH;
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(sort_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(SortShared))) != cudaSuccess)
      return KUIOPS_ELAUNCH;
    configured.fetch_or(bit, std::memory_order_release);
  }
  // few long rows: several CTAs per row, as long as the whole grid stays resident (two CTAs per SM) and
  // every CTA keeps at least two tiles of work
  uint32_t c = 1;
  while (c < 8 && uint64_t(m) * c * 2 <= 2ull * num_sms() && n / (c * 2) >= 2 * kSortTile) c *= 2;
  if (uint64_t(m) * c > 0x7FFFFFFFull) return KUIOPS_ELIMIT;
  return launch_cluster_pdl(sort_rows_kernel, dim3(m * c), dim3(kSortThreads), sizeof(SortShared), as_stream(s), c, n, descending,
                            static_cast<const float*>(X), static_cast<float*>(values), indices, w, w + cells, c);
}

}  // extern "C"
