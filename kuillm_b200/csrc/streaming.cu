// HBM-streaming reductions: row softmax, last-axis mean, whole-tensor folds, row arg-max.
// All are memory bound: 16-byte loads/stores, warp shuffles, fp32 statistics.
#include "common.cuh"
#include <cooperative_groups.h>
#include <climits>

namespace cg = cooperative_groups;
namespace kuiops {

// --------------------------------------------------------------------------------------
// Row softmax.
// A row is split over the CTAs of one thread-block cluster (1, 2, 4 or 8 CTAs) so that a
// handful of very long rows (64 x 128256 logits) still covers every SM.  Each CTA finds the max
// of its slice, then the sum of exp(x - max); every CTA pushes its (max, sum) pair into the shared
// memory of all its peers (distributed shared memory), one cluster barrier later each CTA combines
// the pairs locally and writes exp(x - M) / S.  A short slice is held in registers between the
// passes (CACHE_VECS 16-byte vectors per thread), so HBM sees one read and one write; a long slice
// is streamed once with a running (max, sum) per thread and read again for the write pass (served
// by L2 when the matrix fits there).
// Replaces Klas.RowSoftmax.inst_gpu, one block per row, in place
// (kuiops/softmax/Kuiops.Softmax.Inst.fst.j2:10-11).
// --------------------------------------------------------------------------------------
constexpr float kLog2e = 1.4426950408889634f;

struct MaxSum { float m, s; };
constexpr int kSoftmaxInFlight = 8;      // 16-byte loads a thread of the streaming (uncached) form keeps in flight

// Every thread gets the block-wide max (or sum) of v; `red` is a 32-float shared scratch.
__device__ __forceinline__ float block_allreduce_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  t = warp_max(t);
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_allreduce_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// Running (max, sum of 2^((x - max) log2 e)) of one thread; merging a vector costs one extra ex2.
struct OnlineMaxSum {
  float m = -INFINITY, s = 0.f;
  template <int VN>
  __device__ __forceinline__ void add(const float (&v)[VN]) {
    float vm = v[0];
#pragma unroll
    for (int e = 1; e < VN; ++e) vm = fmaxf(vm, v[e]);
    const float mn = fmaxf(m, vm);
    const float nb = (mn == -INFINITY) ? 0.f : -mn * kLog2e;
    float acc = s * fast_ex2(fmaf(m, kLog2e, nb));        // m = -inf: s is 0 and stays 0
#pragma unroll
    for (int e = 0; e < VN; ++e) acc += fast_ex2(fmaf(v[e], kLog2e, nb));
    s = acc;
    m = mn;
  }
  __device__ __forceinline__ void add1(float v) {
    const float one[1] = {v};
    add<1>(one);
  }
};

template <typename T, int CACHE_VECS>
__global__ void __launch_bounds__(256)
softmax_rows_kernel(uint32_t m, uint32_t n, const T* X, T* Y,   // Y may alias X
                    uint32_t cluster_ctas, int vec_ok) {
  constexpr int VN = Vec16<T>::N;
  __shared__ float red[32];
  __shared__ MaxSum pairs[8];        // (max, sum of exp) of every CTA of the cluster, pushed by its owner

  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t part = cluster_ctas > 1 ? cluster.block_rank() : 0;
  const uint32_t row = blockIdx.x / cluster_ctas;
  // peers must be running before their shared memory is written; arrive now, wait just before the push
  if (cluster_ctas > 1) cluster.barrier_arrive();
  pdl_wait();
  pdl_trigger();
  // slice boundaries in elements, multiples of VN so vector accesses stay aligned
  const uint32_t nv_total = (n + VN - 1) / VN;
  const uint32_t nv_per = (nv_total + cluster_ctas - 1) / cluster_ctas;
  const uint32_t lo = min(part * nv_per * VN, n);
  const uint32_t hi = min(lo + nv_per * VN, n);
  const T* x = X + size_t(row) * n;
  T* y = Y + size_t(row) * n;
  const uint32_t tid = threadIdx.x, nt = blockDim.x;
  const uint32_t nvec = (hi - lo) / VN;

  // ---- slice statistics: (max, sum of exp(x - max)) ------------------------------------------
  Vec16<T> cache[CACHE_VECS > 0 ? CACHE_VECS : 1];
  float bm, bs;
  if (CACHE_VECS > 0) {
    // short slice: it stays in registers, so the max and the sum are two passes over registers
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < CACHE_VECS; ++c)
      if (tid + c * nt < nvec) cache[c] = ld16_stream(x + lo + size_t(tid + c * nt) * VN);
#pragma unroll
    for (int c = 0; c < CACHE_VECS; ++c)
      if (tid + c * nt < nvec) {
#pragma unroll
        for (int e = 0; e < VN; ++e) mx = fmaxf(mx, ElemTraits<T>::to_f(cache[c].v[e]));
      }
    bm = block_allreduce_max(mx, red);
    const float nb = (bm == -INFINITY) ? 0.f : -bm * kLog2e;
    float sm = 0.f;
#pragma unroll
    for (int c = 0; c < CACHE_VECS; ++c)
      if (tid + c * nt < nvec) {
#pragma unroll
        for (int e = 0; e < VN; ++e) sm += fast_ex2(fmaf(ElemTraits<T>::to_f(cache[c].v[e]), kLog2e, nb));
      }
    bs = block_allreduce_sum(sm, red);
  } else {
    // long slice: one streaming pass with a running (max, sum) per thread; the write pass below
    // reads the slice again (from L2 when the matrix fits there)
    OnlineMaxSum st;
    if (vec_ok) {
      for (uint32_t v0 = tid; v0 < nvec; v0 += kSoftmaxInFlight * nt) {      // eight loads in flight per thread
        Vec16<T> t[kSoftmaxInFlight];
#pragma unroll
        for (int u = 0; u < kSoftmaxInFlight; ++u) if (v0 + u * nt < nvec) t[u] = ld16(x + lo + size_t(v0 + u * nt) * VN);
#pragma unroll
        for (int u = 0; u < kSoftmaxInFlight; ++u)
          if (v0 + u * nt < nvec) {
            float f[VN];
#pragma unroll
            for (int e = 0; e < VN; ++e) f[e] = ElemTraits<T>::to_f(t[u].v[e]);
            st.add<VN>(f);
          }
      }
      for (uint32_t i = lo + nvec * VN + tid; i < hi; i += nt) st.add1(ElemTraits<T>::to_f(x[i]));
    } else {
      for (uint32_t i = lo + tid; i < hi; i += nt) st.add1(ElemTraits<T>::to_f(x[i]));
    }
    bm = block_allreduce_max(st.m, red);
    const float nb = (bm == -INFINITY) ? 0.f : -bm * kLog2e;
    bs = block_allreduce_sum(st.s * fast_ex2(fmaf(st.m, kLog2e, nb)), red);
  }
  // ---- exchange: push this CTA's pair into every peer, one cluster barrier, read locally ------
  float M = bm, S = bs;
  if (cluster_ctas > 1) {
    cluster.barrier_wait();
    if (tid < cluster_ctas) {
      MaxSum* dst = cluster.map_shared_rank(pairs, tid);
      dst[part] = MaxSum{bm, bs};
    }
    cluster.sync();
    M = -INFINITY;
    for (uint32_t r = 0; r < cluster_ctas; ++r) M = fmaxf(M, pairs[r].m);
    S = 0.f;
    for (uint32_t r = 0; r < cluster_ctas; ++r)
      if (pairs[r].m != -INFINITY) S += pairs[r].s * exp2f((pairs[r].m - M) * kLog2e);
  }
  // ---- write exp(x - M) / S -------------------------------------------------------------------
  const float inv = 1.f / S;
  const float mb = -M * kLog2e;
  if (CACHE_VECS > 0) {
#pragma unroll
    for (int c = 0; c < CACHE_VECS; ++c)
      if (tid + c * nt < nvec) {
        Vec16<T> o;
#pragma unroll
        for (int e = 0; e < VN; ++e)
          o.v[e] = ElemTraits<T>::from_f(fast_ex2(fmaf(ElemTraits<T>::to_f(cache[c].v[e]), kLog2e, mb)) * inv);
        st16(y + lo + size_t(tid + c * nt) * VN, o);
      }
  } else if (vec_ok) {
    for (uint32_t v0 = tid; v0 < nvec; v0 += kSoftmaxInFlight * nt) {
      Vec16<T> t[kSoftmaxInFlight];
#pragma unroll
      for (int u = 0; u < kSoftmaxInFlight; ++u) if (v0 + u * nt < nvec) t[u] = ld16(x + lo + size_t(v0 + u * nt) * VN);
#pragma unroll
      for (int u = 0; u < kSoftmaxInFlight; ++u)
        if (v0 + u * nt < nvec) {
          Vec16<T> o;
#pragma unroll
          for (int e = 0; e < VN; ++e) o.v[e] = ElemTraits<T>::from_f(fast_ex2(fmaf(ElemTraits<T>::to_f(t[u].v[e]), kLog2e, mb)) * inv);
          st16(y + lo + size_t(v0 + u * nt) * VN, o);
        }
    }
    for (uint32_t i = lo + nvec * VN + tid; i < hi; i += nt)
      y[i] = ElemTraits<T>::from_f(fast_ex2(fmaf(ElemTraits<T>::to_f(x[i]), kLog2e, mb)) * inv);
  } else {
    for (uint32_t i = lo + tid; i < hi; i += nt)
      y[i] = ElemTraits<T>::from_f(fast_ex2(fmaf(ElemTraits<T>::to_f(x[i]), kLog2e, mb)) * inv);
  }
}

template <typename T>
static int softmax_launch(uint32_t m, uint32_t n, const void* X, void* Y, cudaStream_t st) {
  if (m == 0 || n == 0) return KUIOPS_EINVAL;
  if (!X || !Y) return KUIOPS_EINVAL;
  constexpr int VN = Vec16<T>::N;
  // a row start is 16-byte aligned for every row only when n is a multiple of VN
  const int vec_ok = aligned16(X) && aligned16(Y) && (n % VN == 0);
  // cluster width: enough CTAs to cover the SMs when rows are few and long
  uint32_t c = 1;
  while (c < 8 && uint64_t(m) * c < 2 * num_sms() && n / (c * 2) >= 8192) c *= 2;
  const uint32_t nv_per = ((n + VN - 1) / VN + c - 1) / c;   // vectors per CTA slice
  // A slice of up to 4 vectors per thread of a 256-thread CTA is kept in registers.  Longer slices
  // are streamed twice by 256-thread CTAs: small CTAs with few registers are all resident at once
  // (a 64 x 128256 matrix is 512 CTAs, three or four per SM), where 1024-thread CTAs that cache
  // their slice would run in several waves.
  uint32_t threads = ((nv_per + 3) / 4 + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  const bool cached = vec_ok && threads <= 256;
  if (!cached) threads = 256;
  const T* x = static_cast<const T*>(X);
  T* y = static_cast<T*>(Y);
  return cached
      ? launch_cluster_pdl(softmax_rows_kernel<T, 4>, dim3(m * c), dim3(threads), 0, st, c, m, n, x, y, c, vec_ok)
      : launch_cluster_pdl(softmax_rows_kernel<T, 0>, dim3(m * c), dim3(threads), 0, st, c, m, n, x, y, c, vec_ok);
}

// --------------------------------------------------------------------------------------
// Last-axis mean.  One warp per row for short rows, one CTA per row for long ones.
// Replaces Kuiper.Kernel.HReduce.Block.reduce_batched_block (kuiops/mean/Kuiops.Mean.fst:47-50),
// whose pre-map divides every element by n before the tree sum (Kuiops.Mean.fsti:25-32);
// here the sum is accumulated in fp32 and scaled once.
// --------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float row_partial_sum(const T* x, uint64_t n, int lane_id, int lanes,
                                                 bool vec_ok) {
  constexpr int VN = Vec16<T>::N;
  float s0 = 0.f, s1 = 0.f;
  if (vec_ok) {
    const uint64_t nvec = n / VN;
    uint64_t v = lane_id;
    for (; v + lanes < nvec; v += 2 * uint64_t(lanes)) {
      Vec16<T> a = ld16_stream(x + v * VN), b = ld16_stream(x + (v + lanes) * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) { s0 += ElemTraits<T>::to_f(a.v[e]); s1 += ElemTraits<T>::to_f(b.v[e]); }
    }
    for (; v < nvec; v += lanes) {
      Vec16<T> a = ld16_stream(x + v * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) s0 += ElemTraits<T>::to_f(a.v[e]);
    }
    for (uint64_t i = nvec * VN + lane_id; i < n; i += lanes) s1 += ElemTraits<T>::to_f(x[i]);
  } else {
    for (uint64_t i = lane_id; i < n; i += lanes) s0 += ElemTraits<T>::to_f(x[i]);
  }
  return s0 + s1;
}

template <typename T>
__global__ void __launch_bounds__(256)
mean_warp_rows_kernel(uint64_t m, uint64_t n, const T* __restrict__ X, T* __restrict__ out, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const uint64_t warps_total = uint64_t(gridDim.x) * (blockDim.x >> 5);
  const float inv = 1.f / float(n);
  for (uint64_t row = uint64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < m;
       row += warps_total) {
    float s = row_partial_sum(X + row * n, n, lane, 32, vec_ok);
    s = warp_sum(s);
    if (lane == 0) out[row] = ElemTraits<T>::from_f(s * inv);
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
mean_block_rows_kernel(uint64_t m, uint64_t n, const T* __restrict__ X, T* __restrict__ out, int vec_ok) {
  __shared__ float red[32];
  const float inv = 1.f / float(n);
  for (uint64_t row = blockIdx.x; row < m; row += gridDim.x) {
    float s = row_partial_sum(X + row * n, n, threadIdx.x, blockDim.x, vec_ok);
    s = block_sum(s, red);
    if (threadIdx.x == 0) out[row] = ElemTraits<T>::from_f(s * inv);
  }
}

template <typename T>
static int mean_launch(uint64_t m, uint64_t n, const void* in, void* out, cudaStream_t st) {
  if (m == 0 || n == 0 || !in || !out) return KUIOPS_EINVAL;
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = aligned16(in) && (n % VN == 0);
  const T* x = static_cast<const T*>(in);
  T* o = static_cast<T*>(out);
  if (n <= 16384 && m >= 8) {
    unsigned grid = stream_grid(m, 8, 16);
    mean_warp_rows_kernel<T><<<grid, 256, 0, st>>>(m, n, x, o, vec_ok);
  } else {
    unsigned threads = n >= 8192 ? 1024 : 256;
    unsigned grid = unsigned(m < uint64_t(num_sms()) * 8 ? m : uint64_t(num_sms()) * 8);
    mean_block_rows_kernel<T><<<grid, threads, 0, st>>>(m, n, x, o, vec_ok);
  }
  return check_launch();
}

// --------------------------------------------------------------------------------------
// Whole-tensor folds (all / any over bool bytes, max over int64 / fp32).
// Every CTA folds a grid-strided part, stores its partial and takes a ticket; the CTA that
// draws the last ticket folds the partials in index order and resets the ticket.  The folds
// are associative and commutative on these types, so the result equals the left-to-right
// fold of Kuiops.HReducePoly.Exact.reduce (kuiops/reduce/Kuiops.HReducePoly.Exact.fsti:26-46)
// bit for bit.
// --------------------------------------------------------------------------------------
template <typename T, int OP> struct Fold;
template <> struct Fold<uint8_t, KUIOPS_REDUCE_ALL> {
  using Acc = unsigned;
  static __device__ Acc init() { return 1u; }
  static __device__ Acc pre(uint8_t v) { return v != 0; }
  static __device__ Acc f(Acc a, Acc b) { return a & b; }
  static __device__ uint8_t fin(Acc a) { return uint8_t(a); }
};
template <> struct Fold<uint8_t, KUIOPS_REDUCE_ANY> {
  using Acc = unsigned;
  static __device__ Acc init() { return 0u; }
  static __device__ Acc pre(uint8_t v) { return v != 0; }
  static __device__ Acc f(Acc a, Acc b) { return a | b; }
  static __device__ uint8_t fin(Acc a) { return uint8_t(a); }
};
template <> struct Fold<int64_t, KUIOPS_REDUCE_MAX> {
  using Acc = long long;
  static __device__ Acc init() { return LLONG_MIN; }
  static __device__ Acc pre(int64_t v) { return v; }
  static __device__ Acc f(Acc a, Acc b) { return a > b ? a : b; }
  static __device__ int64_t fin(Acc a) { return a; }
};
template <> struct Fold<float, KUIOPS_REDUCE_MAX> {
  using Acc = float;
  static __device__ Acc init() { return -INFINITY; }
  static __device__ Acc pre(float v) { return v; }
  // NaN propagates, as torch.max does
  static __device__ Acc f(Acc a, Acc b) { return (a != a) ? a : ((b != b) ? b : (a > b ? a : b)); }
  static __device__ float fin(Acc a) { return a; }
};

template <typename Acc, typename F>
__device__ __forceinline__ Acc block_fold(Acc v, Acc* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = F::f(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  Acc t = lane < nw ? sh[lane] : F::init();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = F::f(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}

template <typename T, int OP>
__global__ void __launch_bounds__(512)
fold_kernel(uint64_t n, const T* __restrict__ in, T* __restrict__ out, unsigned long long* ticket,
            typename Fold<T, OP>::Acc* partials, int vec_ok) {
  using F = Fold<T, OP>;
  using Acc = typename F::Acc;
  __shared__ Acc sh[32];
  __shared__ bool is_last;
  constexpr int VN = Vec16<T>::N;
  Acc a = F::init();
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  if (vec_ok) {
    const uint64_t nvec = n / VN;
    for (uint64_t v = gt; v < nvec; v += gs) {
      Vec16<T> t = ld16_stream(in + v * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) a = F::f(a, F::pre(t.v[e]));
    }
    for (uint64_t i = nvec * VN + gt; i < n; i += gs) a = F::f(a, F::pre(in[i]));
  } else {
    for (uint64_t i = gt; i < n; i += gs) a = F::f(a, F::pre(in[i]));
  }
  a = block_fold<Acc, F>(a, sh);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = a;
    __threadfence();
    unsigned long long t = atomicAdd(ticket, 1ull);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  Acc b = F::init();
  for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) b = F::f(b, __ldcg(&partials[i]));
  b = block_fold<Acc, F>(b, sh);
  if (threadIdx.x == 0) {
    *out = F::fin(b);
    *ticket = 0ull;   // leave the workspace ready for the next call
  }
}

template <typename T, int OP>
static int fold_launch(uint64_t n, const void* in, void* out, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (n == 0 || !in || !out) return KUIOPS_EINVAL;
  if (!ws || ws_bytes < KUIOPS_REDUCE_WORKSPACE_BYTES) return KUIOPS_EWORKSPACE;
  using Acc = typename Fold<T, OP>::Acc;
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = aligned16(in);
  unsigned grid = stream_grid((n + VN - 1) / VN, 512 * 4, 4);
  const unsigned max_partials = (KUIOPS_REDUCE_WORKSPACE_BYTES - 64) / sizeof(Acc);
  if (grid > max_partials) grid = max_partials;
  auto* ticket = static_cast<unsigned long long*>(ws);
  auto* partials = reinterpret_cast<Acc*>(static_cast<char*>(ws) + 64);
  fold_kernel<T, OP><<<grid, 512, 0, st>>>(n, static_cast<const T*>(in), static_cast<T*>(out), ticket,
                                           partials, vec_ok);
  return check_launch();
}

// --------------------------------------------------------------------------------------
// Row arg-max (greedy sampling over the vocabulary), ties to the lowest index.
// --------------------------------------------------------------------------------------
// Candidate of one thread / warp / CTA: the value and its index inside the row.
struct ArgBest {
  float v;
  long long i;     // LLONG_MAX: nothing seen yet
};
// NaN counts as the maximum, as in torch.argmax; equal values (and -0 / +0) keep the lowest index.
__device__ __forceinline__ void arg_consider(ArgBest& b, float v, long long i) {
  if (i == LLONG_MAX) return;
  const bool vnan = v != v, bnan = b.v != b.v;
  bool better;
  if (b.i == LLONG_MAX) better = true;
  else if (vnan != bnan) better = vnan;
  else if (vnan) better = i < b.i;
  else better = v > b.v || (v == b.v && i < b.i);
  if (better) { b.v = v; b.i = i; }
}

// A row is split over the CTAs of a cluster (1..8) so that a few long rows still cover the SMs;
// every CTA pushes its candidate into the leader's shared memory and the leader picks.
template <typename T>
__global__ void __launch_bounds__(256)
argmax_rows_kernel(uint64_t m, uint64_t n, const T* __restrict__ X, int64_t* __restrict__ out, int vec_ok,
                   uint32_t cluster_ctas) {
  __shared__ float sv[32];
  __shared__ long long si[32];
  __shared__ ArgBest parts[8];
  constexpr int VN = Vec16<T>::N;
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t part = cluster_ctas > 1 ? cluster.block_rank() : 0;
  if (cluster_ctas > 1) cluster.barrier_arrive();      // peers are running before their memory is written
  pdl_wait();
  pdl_trigger();
  const uint64_t row = blockIdx.x / cluster_ctas;      // grid = m * cluster_ctas
  const T* x = X + row * n;
  // slice of this CTA in whole vectors
  const uint64_t nv_total = (n + VN - 1) / VN;
  const uint64_t nv_per = (nv_total + cluster_ctas - 1) / cluster_ctas;
  const uint64_t lo = min(uint64_t(part) * nv_per * VN, n), hi = min(lo + nv_per * VN, n);
  ArgBest best{-INFINITY, LLONG_MAX};
  if (vec_ok) {
    const uint64_t nvec = (hi - lo) / VN;
    const uint64_t nt = blockDim.x;
    // Hot loop, per 16-byte vector: its largest value (max tree), "is it above the thread's running
    // maximum" (strict, so the first vector that holds the maximum wins) and a NaN detector (the
    // sum is NaN when an element is; inf - inf also trips it, which only costs the exact path).
    // Which element of the winning vector it was is settled after the loop by reading that one
    // vector again.
    float bm = -INFINITY, nan_acc = 0.f;
    uint64_t bvec = ~0ull;
    for (uint64_t v0 = threadIdx.x; v0 < nvec; v0 += 4 * nt) {      // four loads in flight per thread
      Vec16<T> t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) if (v0 + u * nt < nvec) t[u] = ld16_stream(x + lo + (v0 + u * nt) * VN);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * nt < nvec) {
          float vm = ElemTraits<T>::to_f(t[u].v[0]), vs = vm;
#pragma unroll
          for (int e = 1; e < VN; ++e) { const float f = ElemTraits<T>::to_f(t[u].v[e]); vm = fmaxf(vm, f); vs += f; }
          nan_acc += vs * 0.f;                            // stays 0 unless vs is NaN or infinite
          const bool take = vm > bm || bvec == ~0ull;
          bm = take ? vm : bm;
          bvec = take ? v0 + u * nt : bvec;
        }
    }
    if (nan_acc != nan_acc) {
      // a NaN (or an infinity) somewhere in this thread's vectors: redo them with the exact rule
      for (uint64_t v = threadIdx.x; v < nvec; v += nt) {
        const Vec16<T> t = ld16(x + lo + v * VN);
#pragma unroll
        for (int e = 0; e < VN; ++e) arg_consider(best, ElemTraits<T>::to_f(t.v[e]), (long long)(lo + v * VN + e));
      }
    } else if (bvec != ~0ull) {
      const Vec16<T> t = ld16(x + lo + bvec * VN);
#pragma unroll
      for (int e = VN - 1; e >= 0; --e)
        if (ElemTraits<T>::to_f(t.v[e]) == bm) { best.v = bm; best.i = (long long)(lo + bvec * VN + e); }
    }
    for (uint64_t i = lo + nvec * VN + threadIdx.x; i < hi; i += blockDim.x)
      arg_consider(best, ElemTraits<T>::to_f(x[i]), (long long)i);
  } else {
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) arg_consider(best, ElemTraits<T>::to_f(x[i]), (long long)i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
    const long long oi = __shfl_xor_sync(0xffffffffu, best.i, o);
    arg_consider(best, ov, oi);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) { sv[w] = best.v; si[w] = best.i; }
  __syncthreads();
  if (w == 0) {
    best.v = lane < nw ? sv[lane] : -INFINITY;
    best.i = lane < nw ? si[lane] : LLONG_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, best.i, o);
      arg_consider(best, ov, oi);
    }
  }
  if (cluster_ctas == 1) {
    if (threadIdx.x == 0) out[row] = best.i;
    return;
  }
  cluster.barrier_wait();
  if (threadIdx.x == 0) cluster.map_shared_rank(parts, 0)[part] = best;
  cluster.sync();
  if (part == 0 && threadIdx.x == 0) {
    ArgBest b = parts[0];
    for (uint32_t r = 1; r < cluster_ctas; ++r) arg_consider(b, parts[r].v, parts[r].i);
    out[row] = b.i;
  }
}

template <typename T>
static int argmax_launch(uint64_t m, uint64_t n, const void* X, int64_t* out, cudaStream_t st) {
  if (m == 0 || n == 0 || !X || !out) return KUIOPS_EINVAL;
  if (m > 0x7FFFFFFFull / 8) return KUIOPS_ELIMIT;
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = aligned16(X) && (n % VN == 0);
  // small CTAs: with a cluster per row all of them must be resident at once to finish in one wave
  unsigned threads = n >= 2048 ? 256 : 64;
  // cluster width: enough CTAs to give every SM two when rows are few and long
  uint32_t c = 1;
  while (c < 8 && m * c < 2 * uint64_t(num_sms()) && n / (c * 2) >= 8192) c *= 2;
  return launch_cluster_pdl(argmax_rows_kernel<T>, dim3(unsigned(m * c)), dim3(threads), 0, st, c, m, n,
                            static_cast<const T*>(X), out, vec_ok, c);
}

}  // namespace kuiops

using namespace kuiops;

extern "C" {

int kuiops_softmax_f32(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t s) {
  return softmax_launch<float>(m, n, X, Y, as_stream(s));
}
int kuiops_softmax_bf16(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t s) {
  return softmax_launch<__nv_bfloat16>(m, n, X, Y, as_stream(s));
}
int kuiops_softmax_f16(uint32_t m, uint32_t n, const void* X, void* Y, kuiops_stream_t s) {
  return softmax_launch<__half>(m, n, X, Y, as_stream(s));
}

int kuiops_mean_f32(uint64_t m, uint64_t n, const void* in, void* out, kuiops_stream_t s) {
  return mean_launch<float>(m, n, in, out, as_stream(s));
}
int kuiops_mean_bf16(uint64_t m, uint64_t n, const void* in, void* out, kuiops_stream_t s) {
  return mean_launch<__nv_bfloat16>(m, n, in, out, as_stream(s));
}
int kuiops_mean_f16(uint64_t m, uint64_t n, const void* in, void* out, kuiops_stream_t s) {
  return mean_launch<__half>(m, n, in, out, as_stream(s));
}

int kuiops_reduce_u8(int op, uint64_t n, const void* in, void* out, void* ws, size_t wsb, kuiops_stream_t s) {
  if (op == KUIOPS_REDUCE_ALL) return fold_launch<uint8_t, KUIOPS_REDUCE_ALL>(n, in, out, ws, wsb, as_stream(s));
  if (op == KUIOPS_REDUCE_ANY) return fold_launch<uint8_t, KUIOPS_REDUCE_ANY>(n, in, out, ws, wsb, as_stream(s));
  return KUIOPS_EUNSUPPORTED;
}
int kuiops_reduce_i64(int op, uint64_t n, const void* in, void* out, void* ws, size_t wsb, kuiops_stream_t s) {
  if (op == KUIOPS_REDUCE_MAX) return fold_launch<int64_t, KUIOPS_REDUCE_MAX>(n, in, out, ws, wsb, as_stream(s));
  return KUIOPS_EUNSUPPORTED;
}
int kuiops_reduce_f32(int op, uint64_t n, const void* in, void* out, void* ws, size_t wsb, kuiops_stream_t s) {
  if (op == KUIOPS_REDUCE_MAX) return fold_launch<float, KUIOPS_REDUCE_MAX>(n, in, out, ws, wsb, as_stream(s));
  return KUIOPS_EUNSUPPORTED;
}

int kuiops_argmax(int dtype, uint64_t m, uint64_t n, const void* X, int64_t* out, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_F32: return argmax_launch<float>(m, n, X, out, as_stream(s));
    case KUIOPS_BF16: return argmax_launch<__nv_bfloat16>(m, n, X, out, as_stream(s));
    case KUIOPS_F16: return argmax_launch<__half>(m, n, X, out, as_stream(s));
  }
  return KUIOPS_EINVAL;
}

}  // extern "C"
