// Indexed data movement: gather, scatter, cat (binary and n-ary), index, isin.
// Payload-only kernels: elements are moved as opaque 1/2/4/8-byte words (or 16-byte vectors
// where chunks allow), so one instantiation per word size serves every dtype.  The int64
// index tensors are read directly.
#include "common.cuh"
#include <climits>

namespace kuiops {

template <int BYTES> struct Word;
template <> struct Word<1> { using type = uint8_t; };
template <> struct Word<2> { using type = uint16_t; };
template <> struct Word<4> { using type = uint32_t; };
template <> struct Word<8> { using type = uint64_t; };
template <> struct Word<16> { using type = int4; };

struct CoordMap {
  // Walk of a dense row-major `shape` whose cells map to offsets in another dense tensor
  // through `stride` (0 on the indexed axis, which is resolved through the index value).
  uint32_t rank;
  uint64_t shape[KUIOPS_MAX_RANK];
  uint64_t stride[KUIOPS_MAX_RANK];
  uint64_t dim_size;     // extent of the indexed axis in the addressed tensor
  uint64_t dim_stride;   // its element stride there
};

// Build the walk for gather/scatter.  `walk` is the shape that is enumerated (index/src
// shape), `full` the shape of the tensor addressed through the index (input/self).  Adjacent
// axes are merged when the addressed tensor is dense across them, which turns the usual
// (rows, dim) and (outer, dim, inner) cases into rank <= 3.
static bool build_coord_map(uint32_t rank, uint32_t dim, const uint64_t* walk, const uint64_t* full, CoordMap& cm) {
  uint64_t fstride[KUIOPS_MAX_RANK];
  uint64_t s = 1;
  for (int d = int(rank) - 1; d >= 0; --d) { fstride[d] = s; s *= full[d]; }
  cm.dim_size = full[dim];
  cm.dim_stride = fstride[dim];
  uint32_t r = 0;
  for (uint32_t d = 0; d < rank; ++d) {
    const uint64_t st = (d == dim) ? 0 : fstride[d];
    const bool mergeable = r > 0 && d != dim && (d - 1) != dim && walk[d] == full[d];
    if (mergeable) {
      // previous axis stride in `full` equals full[d] * fstride[d]: the two axes form one dense run
      cm.shape[r - 1] *= walk[d];
      cm.stride[r - 1] = st;
    } else {
      cm.shape[r] = walk[d];
      cm.stride[r] = st;
      ++r;
    }
  }
  cm.rank = r;
  return true;
}

template <typename I>
__device__ __forceinline__ uint64_t walk_offset(const CoordMap& cm, I linear) {
  uint64_t off = 0;
  I rem = linear;
#pragma unroll 1
  for (int d = int(cm.rank) - 1; d >= 0; --d) {
    const I ext = I(cm.shape[d]);
    const I c = rem % ext;
    rem /= ext;
    off += uint64_t(c) * cm.stride[d];
  }
  return off;
}

// out[x] = inp[x with x_dim := idx[x]]  (kuiops/gather/Kuiops.Gather.fst:93-99: one thread per output cell)
template <typename W, typename I>
__global__ void __launch_bounds__(256)
gather_kernel(const __grid_constant__ CoordMap cm, const W* __restrict__ inp, const int64_t* __restrict__ idx,
              W* __restrict__ out, uint64_t n, int32_t* status) {
  const uint64_t gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += gs) {
    const int64_t j = idx[i];
    if (j < 0 || uint64_t(j) >= cm.dim_size) {
      if (status) atomicExch(status, 1);
      continue;
    }
    out[i] = inp[walk_offset<I>(cm, I(i)) + uint64_t(j) * cm.dim_stride];
  }
}

// out[i with i_dim := idx[i]] = src[i]  (kuiops/scatter/Kuiops.Scatter.fst:363-400: one thread per src cell)
template <typename W, typename I>
__global__ void __launch_bounds__(256)
scatter_kernel(const __grid_constant__ CoordMap cm, const W* __restrict__ src, const int64_t* __restrict__ idx,
               W* __restrict__ out, uint64_t n, int32_t* status) {
  const uint64_t gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += gs) {
    const int64_t j = idx[i];
    if (j < 0 || uint64_t(j) >= cm.dim_size) {
      if (status) atomicExch(status, 1);
      continue;
    }
    out[walk_offset<I>(cm, I(i)) + uint64_t(j) * cm.dim_stride] = src[i];
  }
}

// ---- row-local gather / scatter ---------------------------------------------------------
// When the indexed axis is the innermost one, every cell that one row of the index addresses
// lies in one dense row of the addressed tensor.  A CTA stages that row in shared memory, so the
// random accesses never leave the SM and global memory only sees coalesced 16-byte traffic:
// gather reads input row + index row and writes the output row; scatter reads self row + src row
// + index row and writes the output row once (the separate clone of self disappears).
// The staging buffer is shifted by the row's misalignment so that global and shared addresses
// agree modulo 16 and the body of the row moves as 16-byte vectors.
template <typename W>
__device__ __forceinline__ W* stage_row_in(unsigned char* raw, const W* g, uint64_t count) {
  const uint32_t shift = uint32_t(reinterpret_cast<uintptr_t>(g) & 15u);      // multiple of sizeof(W)
  W* stage = reinterpret_cast<W*>(raw + shift);
  constexpr uint32_t PER = 16 / sizeof(W);
  const uint64_t head = shift ? min(uint64_t((16 - shift) / sizeof(W)), count) : 0;
  const uint64_t nvec = (count - head) / PER;
  for (uint64_t i = threadIdx.x; i < head; i += blockDim.x) stage[i] = g[i];
  const int4* gv = reinterpret_cast<const int4*>(g + head);
  int4* sv = reinterpret_cast<int4*>(stage + head);
  for (uint64_t v = threadIdx.x; v < nvec; v += blockDim.x) sv[v] = __ldcs(gv + v);
  for (uint64_t i = head + nvec * PER + threadIdx.x; i < count; i += blockDim.x) stage[i] = g[i];
  return stage;
}
template <typename W>
__device__ __forceinline__ void stage_row_out(const W* stage, W* g, uint64_t count) {
  // `stage` carries the misalignment of the row it was loaded from; vectors need the same one here
  const uint32_t shift_g = uint32_t(reinterpret_cast<uintptr_t>(g) & 15u);
  const uint32_t shift_s = uint32_t(__cvta_generic_to_shared(stage) & 15u);
  if (shift_g != shift_s) {
    for (uint64_t i = threadIdx.x; i < count; i += blockDim.x) g[i] = stage[i];
    return;
  }
  constexpr uint32_t PER = 16 / sizeof(W);
  const uint64_t head = shift_g ? min(uint64_t((16 - shift_g) / sizeof(W)), count) : 0;
  const uint64_t nvec = (count - head) / PER;
  for (uint64_t i = threadIdx.x; i < head; i += blockDim.x) g[i] = stage[i];
  const int4* sv = reinterpret_cast<const int4*>(stage + head);
  int4* gv = reinterpret_cast<int4*>(g + head);
  for (uint64_t v = threadIdx.x; v < nvec; v += blockDim.x) gv[v] = sv[v];
  for (uint64_t i = head + nvec * PER + threadIdx.x; i < count; i += blockDim.x) g[i] = stage[i];
}

template <typename W>
__global__ void __launch_bounds__(1024)
gather_rows_kernel(uint64_t rows_w, uint64_t cols_w, uint64_t cols_f, const W* __restrict__ inp,
                   const int64_t* __restrict__ idx, W* __restrict__ out, int32_t* status) {
  extern __shared__ __align__(16) unsigned char stage_raw[];
  for (uint64_t row = blockIdx.x; row < rows_w; row += gridDim.x) {
    __syncthreads();                                   // the previous row's readers are done
    const W* stage = stage_row_in(stage_raw, inp + row * cols_f, cols_f);
    const int64_t* irow = idx + row * cols_w;
    W* orow = out + row * cols_w;
    __syncthreads();
    const bool pairs = (reinterpret_cast<uintptr_t>(irow) & 15u) == 0;
    const uint64_t npair = pairs ? cols_w / 2 : 0;
    for (uint64_t q0 = threadIdx.x; q0 < npair; q0 += 4ull * blockDim.x) {       // four index loads in flight
      int4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (q0 + u * blockDim.x < npair) raw[u] = __ldcs(reinterpret_cast<const int4*>(irow) + q0 + u * blockDim.x);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint64_t q = q0 + u * blockDim.x;
        if (q < npair) {
          const long long* jj = reinterpret_cast<const long long*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const long long j = jj[e];
            if (j < 0 || uint64_t(j) >= cols_f) { if (status) atomicExch(status, 1); continue; }
            orow[2 * q + e] = stage[j];
          }
        }
      }
    }
    for (uint64_t c = npair * 2 + threadIdx.x; c < cols_w; c += blockDim.x) {
      const int64_t j = irow[c];
      if (j < 0 || uint64_t(j) >= cols_f) { if (status) atomicExch(status, 1); continue; }
      orow[c] = stage[j];
    }
  }
}

template <typename W>
__global__ void __launch_bounds__(1024)
scatter_rows_kernel(uint64_t rows_f, uint64_t rows_w, uint64_t cols_w, uint64_t cols_f, const W* self_,
                    const W* __restrict__ src, const int64_t* __restrict__ idx, W* out, int32_t* status) {
  extern __shared__ __align__(16) unsigned char stage_raw[];
  for (uint64_t row = blockIdx.x; row < rows_f; row += gridDim.x) {
    __syncthreads();                                   // the previous row has been written out
    W* stage = stage_row_in(stage_raw, self_ + row * cols_f, cols_f);
    __syncthreads();
    if (row < rows_w) {
      const int64_t* irow = idx + row * cols_w;
      const W* srow = src + row * cols_w;
      for (uint64_t c0 = threadIdx.x; c0 < cols_w; c0 += 4ull * blockDim.x) {    // four loads of each in flight
        int64_t j[4];
        W v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint64_t c = c0 + u * blockDim.x;
          if (c < cols_w) { j[u] = __ldcs(irow + c); v[u] = __ldcs(srow + c); }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint64_t c = c0 + u * blockDim.x;
          if (c < cols_w) {
            if (j[u] < 0 || uint64_t(j[u]) >= cols_f) { if (status) atomicExch(status, 1); continue; }
            stage[j[u]] = v[u];
          }
        }
      }
      __syncthreads();
    }
    stage_row_out(stage, out + row * cols_f, cols_f);
  }
}

// Launch geometry of the row-local kernels: as many CTAs per SM as shared memory and threads allow.
struct RowsLaunch { unsigned grid, threads; size_t smem; bool ok; };
static RowsLaunch rows_launch(uint64_t rows, uint64_t cols_f, uint32_t word) {
  RowsLaunch r = {};
  const uint64_t bytes = cols_f * word + 16;
  r.ok = bytes <= 200 * 1024;
  if (!r.ok) return r;
  r.smem = size_t(bytes);
  r.threads = bytes >= 64 * 1024 ? 1024 : (bytes >= 16 * 1024 ? 512 : 256);
  uint64_t per_sm = (220 * 1024) / (bytes + 1024);
  if (per_sm > 2048 / r.threads) per_sm = 2048 / r.threads;
  if (per_sm < 1) per_sm = 1;
  const uint64_t cap = uint64_t(num_sms()) * per_sm;
  r.grid = unsigned(rows < cap ? rows : cap);
  return r;
}
// Dynamic shared memory above 48 KB needs an opt-in per kernel and device.
template <typename K>
static bool allow_smem(K kern, size_t bytes) {
  static std::atomic<uint64_t> done{0};               // one per kernel type
  if (bytes <= 48 * 1024) return true;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  const uint64_t bit = 1ull << (dev & 63);
  if (done.load(std::memory_order_acquire) & bit) return true;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024 + 16) != cudaSuccess) return false;
  done.fetch_or(bit, std::memory_order_release);
  return true;
}

__global__ void __launch_bounds__(256)
copy_bytes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t bytes, int vec_ok) {
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  uint64_t start = 0;
  if (vec_ok) {
    const uint64_t nvec = bytes / 16;
    for (uint64_t v = gt; v < nvec; v += gs)
      reinterpret_cast<int4*>(dst)[v] = __ldcs(reinterpret_cast<const int4*>(src) + v);
    start = nvec * 16;
  }
  for (uint64_t i = start + gt; i < bytes; i += gs) dst[i] = src[i];
}

static int copy_bytes(const void* src, void* dst, uint64_t bytes, cudaStream_t st) {
  const int vec_ok = aligned16(src) && aligned16(dst);
  unsigned grid = stream_grid((bytes + 15) / 16, 256 * 4, 8);
  copy_bytes_kernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), bytes, vec_ok);
  return check_launch();
}

// ---- cat --------------------------------------------------------------------------------
// A cat along `dim` of dense tensors is, per outer index, the concatenation of one contiguous
// chunk from each input (kuiops/cat/Kuiops.Cat.fst:180-186 maps over output cells).  Up to
// kCatMax inputs per launch; chunks move as 16-byte vectors when sizes and pointers allow.
constexpr int kCatMax = 16;
struct CatParams {
  uint32_t count;
  const void* src[kCatMax];
  uint64_t chunk[kCatMax];      // words per outer index contributed by input t
  uint64_t offset[kCatMax + 1]; // prefix sums of chunk
  uint64_t out_row;             // words per outer index in the output (all inputs of the whole cat)
  uint64_t out_base;            // word offset of this launch's first input inside an output row
  uint64_t outer;
};

template <typename W>
__global__ void __launch_bounds__(256)
cat_kernel(const __grid_constant__ CatParams p, W* __restrict__ out) {
  const uint64_t row = p.offset[p.count];
  const uint64_t total = p.outer * row;
  const uint64_t gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += gs) {
    const uint64_t o = i / row, r = i % row;
    uint32_t t = 0;
#pragma unroll 1
    while (t + 1 < p.count && r >= p.offset[t + 1]) ++t;
    const W* s = static_cast<const W*>(p.src[t]);
    out[o * p.out_row + p.out_base + r] = s[o * p.chunk[t] + (r - p.offset[t])];
  }
}

static int cat_impl(uint32_t elem_bytes, uint32_t rank, uint32_t dim, uint32_t count, const uint64_t* shape,
                    const uint64_t* dim_sizes, const void* const* ptrs, void* out, cudaStream_t st) {
  if (rank == 0 || rank > KUIOPS_MAX_RANK || dim >= rank || count == 0 || !shape || !dim_sizes || !ptrs || !out)
    return KUIOPS_EINVAL;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) return KUIOPS_EINVAL;
  uint64_t outer = 1, inner = 1, dim_total = 0;
  for (uint32_t d = 0; d < dim; ++d) outer *= shape[d];
  for (uint32_t d = dim + 1; d < rank; ++d) inner *= shape[d];
  for (uint32_t t = 0; t < count; ++t) { if (!ptrs[t] && dim_sizes[t]) return KUIOPS_EINVAL; dim_total += dim_sizes[t]; }
  if (outer == 0 || inner == 0 || dim_total == 0) return KUIOPS_EINVAL;
  // widest word that divides every chunk (in bytes) and every pointer
  uint32_t word = 16;
  auto fits = [&](uint32_t w) {
    if (reinterpret_cast<uintptr_t>(out) % w) return false;
    for (uint32_t t = 0; t < count; ++t) {
      if ((dim_sizes[t] * inner * elem_bytes) % w) return false;
      if (dim_sizes[t] && reinterpret_cast<uintptr_t>(ptrs[t]) % w) return false;
    }
    return true;
  };
  while (word > elem_bytes && !fits(word)) word >>= 1;
  const uint64_t out_row = dim_total * inner * elem_bytes / word;
  uint64_t base = 0;
  int rc = KUIOPS_OK;
  for (uint32_t t0 = 0; t0 < count && rc == KUIOPS_OK; t0 += kCatMax) {
    CatParams p = {};
    p.count = (count - t0 < uint32_t(kCatMax)) ? count - t0 : uint32_t(kCatMax);
    p.out_row = out_row; p.out_base = base; p.outer = outer;
    p.offset[0] = 0;
    for (uint32_t t = 0; t < p.count; ++t) {
      p.src[t] = ptrs[t0 + t];
      p.chunk[t] = dim_sizes[t0 + t] * inner * elem_bytes / word;
      p.offset[t + 1] = p.offset[t] + p.chunk[t];
    }
    base += p.offset[p.count];
    const uint64_t total = outer * p.offset[p.count];
    if (total == 0) continue;
    unsigned grid = stream_grid(total, 256 * 2, 16);
    switch (word) {
      case 16: cat_kernel<int4><<<grid, 256, 0, st>>>(p, static_cast<int4*>(out)); break;
      case 8: cat_kernel<uint64_t><<<grid, 256, 0, st>>>(p, static_cast<uint64_t*>(out)); break;
      case 4: cat_kernel<uint32_t><<<grid, 256, 0, st>>>(p, static_cast<uint32_t*>(out)); break;
      case 2: cat_kernel<uint16_t><<<grid, 256, 0, st>>>(p, static_cast<uint16_t*>(out)); break;
      default: cat_kernel<uint8_t><<<grid, 256, 0, st>>>(p, static_cast<uint8_t*>(out)); break;
    }
    rc = check_launch();
  }
  return rc;
}

// ---- index ------------------------------------------------------------------------------
struct IndexParams {
  uint32_t n_idx, idx_rank;
  const int64_t* idx[4];
  uint64_t idx_shape[KUIOPS_MAX_RANK];
  int64_t idx_stride[4][KUIOPS_MAX_RANK];
  uint64_t dim_size[4];     // extents of the indexed axes of self
  uint64_t dim_stride[4];   // their strides in units of `inner` runs
  uint64_t pre, nb, inner;  // outer cells, broadcast index cells, dense trailing words
  uint64_t self_pre_stride; // words between consecutive outer cells of self
};

template <typename W>
__global__ void __launch_bounds__(256)
index_kernel(const __grid_constant__ IndexParams p, const W* __restrict__ self_, W* __restrict__ out, int32_t* status) {
  const uint64_t total = p.pre * p.nb * p.inner;
  const uint64_t gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += gs) {
    const uint64_t w = i % p.inner;
    const uint64_t b = (i / p.inner) % p.nb;
    const uint64_t o = i / (p.inner * p.nb);
    // coordinates of b in the broadcast index shape
    uint64_t c[KUIOPS_MAX_RANK];
    uint64_t rem = b;
#pragma unroll 1
    for (int d = int(p.idx_rank) - 1; d >= 0; --d) { c[d] = rem % p.idx_shape[d]; rem /= p.idx_shape[d]; }
    uint64_t off = o * p.self_pre_stride;
    bool ok = true;
#pragma unroll 1
    for (uint32_t k = 0; k < p.n_idx; ++k) {
      int64_t io = 0;
#pragma unroll 1
      for (uint32_t d = 0; d < p.idx_rank; ++d) io += int64_t(c[d]) * p.idx_stride[k][d];
      int64_t v = p.idx[k][io];
      if (v < 0) v += int64_t(p.dim_size[k]);
      if (v < 0 || uint64_t(v) >= p.dim_size[k]) { ok = false; break; }
      off += uint64_t(v) * p.dim_stride[k];
    }
    if (!ok) { if (status) atomicExch(status, 1); continue; }
    out[i] = self_[off + w];
  }
}

// ---- isin -------------------------------------------------------------------------------
// The test set goes into an open-addressing hash table in shared memory (kIsinTile entries per
// pass at load factor 1/2; a 1024-entry stop-id set is one pass) and every element probes it.
// A 64 Kbit filter (one bit per 16-bit hash of a test value) answers "certainly absent" with a
// single 4-byte shared-memory load, which is the common answer for a small stop-id set.
// Elements are read two per 16-byte load and results written eight per store.
constexpr int kIsinTile = 2048;
constexpr int kIsinSlots = 2 * kIsinTile;
constexpr unsigned long long kIsinEmpty = 0x8000000000000000ull;    // INT64_MIN marks a free slot

constexpr int kIsinFilterWords = 2048;                              // 65536 bits
__device__ __forceinline__ uint32_t isin_filter_hash(unsigned long long v) {
  return uint32_t((v * 0x9E3779B97F4A7C15ull) >> 48);               // 16 bits; the top 12 index the table (kIsinSlots)
}
__device__ __forceinline__ bool isin_probe(const unsigned long long* slots, const uint32_t* filter, bool has_empty_key, long long v) {
  const unsigned long long u = static_cast<unsigned long long>(v);
  if (u == kIsinEmpty) return has_empty_key;
  const uint32_t fh = isin_filter_hash(u);
  if (!((filter[fh >> 5] >> (fh & 31u)) & 1u)) return false;
  uint32_t h = fh >> 4;
  for (int probes = 0; probes < kIsinSlots; ++probes) {             // ends at the first free slot
    const unsigned long long sl = slots[h];
    if (sl == u) return true;
    if (sl == kIsinEmpty) return false;
    h = (h + 1) & (kIsinSlots - 1);
  }
  return false;
}

__global__ void __launch_bounds__(512)
isin_kernel(uint64_t n, const int64_t* __restrict__ elems, uint64_t m, const int64_t* __restrict__ tests, int invert,
            uint8_t* __restrict__ out, uint64_t per_block, int vec_ok) {
  __shared__ unsigned long long slots[kIsinSlots];
  __shared__ uint32_t filter[kIsinFilterWords];
  __shared__ int has_empty_key;
  const uint64_t lo = uint64_t(blockIdx.x) * per_block;      // per_block is a multiple of 8
  const uint64_t hi = lo + per_block < n ? lo + per_block : n;
  if (lo >= n) return;
  const uint8_t inv = invert ? 1 : 0;
  for (uint64_t t0 = 0; t0 < m; t0 += kIsinTile) {
    const uint32_t cnt = uint32_t(m - t0 < uint64_t(kIsinTile) ? m - t0 : uint64_t(kIsinTile));
    const bool first = t0 == 0, last = t0 + kIsinTile >= m;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < uint32_t(kIsinSlots); i += blockDim.x) slots[i] = kIsinEmpty;
    for (uint32_t i = threadIdx.x; i < uint32_t(kIsinFilterWords); i += blockDim.x) filter[i] = 0u;
    if (threadIdx.x == 0) has_empty_key = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < cnt; i += blockDim.x) {
      const unsigned long long u = static_cast<unsigned long long>(tests[t0 + i]);
      if (u == kIsinEmpty) { has_empty_key = 1; continue; }
      const uint32_t fh = isin_filter_hash(u);
      atomicOr(&filter[fh >> 5], 1u << (fh & 31u));
      uint32_t h = fh >> 4;
      for (int probes = 0; probes < kIsinSlots; ++probes) {
        const unsigned long long prev = atomicCAS(&slots[h], kIsinEmpty, u);
        if (prev == kIsinEmpty || prev == u) break;
        h = (h + 1) & (kIsinSlots - 1);
      }
    }
    __syncthreads();
    const bool hek = has_empty_key != 0;
    // out holds the running "found in an earlier pass" flag between passes; the last pass applies invert
    auto finish = [&](bool hit, uint8_t prev) -> uint8_t {
      const uint8_t f = (hit || (!first && prev)) ? 1 : 0;
      return last ? uint8_t(f ^ inv) : f;
    };
    uint64_t e0 = lo;
    if (vec_ok) {
      const uint64_t groups = (hi - lo) / 8;
      for (uint64_t g = threadIdx.x; g < groups; g += blockDim.x) {
        const uint64_t e = lo + g * 8;
        int4 raw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) raw[q] = __ldcs(reinterpret_cast<const int4*>(elems + e) + q);
        const long long* v = reinterpret_cast<const long long*>(raw);
        uint2 prev = make_uint2(0u, 0u);
        if (!first) prev = *reinterpret_cast<const uint2*>(out + e);
        const uint8_t* pb = reinterpret_cast<const uint8_t*>(&prev);
        uint2 res;
        uint8_t* rb = reinterpret_cast<uint8_t*>(&res);
#pragma unroll
        for (int q = 0; q < 8; ++q) rb[q] = finish(isin_probe(slots, filter, hek, v[q]), pb[q]);
        *reinterpret_cast<uint2*>(out + e) = res;
      }
      e0 = lo + groups * 8;
    }
    for (uint64_t e = e0 + threadIdx.x; e < hi; e += blockDim.x)
      out[e] = finish(isin_probe(slots, filter, hek, elems[e]), first ? uint8_t(0) : out[e]);
  }
}

}  // namespace kuiops

using namespace kuiops;

static bool elem_ok(uint32_t b) { return b == 1 || b == 2 || b == 4 || b == 8; }

extern "C" {

int kuiops_gather(uint32_t elem_bytes, uint32_t rank, uint32_t dim, const uint64_t* inp_shape,
                  const uint64_t* idx_shape, const void* inp, const int64_t* idx, void* out, uint64_t n,
                  int32_t* status, kuiops_stream_t s) {
  if (!elem_ok(elem_bytes) || rank == 0 || rank > KUIOPS_MAX_RANK || dim >= rank) return KUIOPS_EINVAL;
  if (!inp_shape || !idx_shape || !inp || !idx || !out) return KUIOPS_EINVAL;
  uint64_t numel = 1, total_addr = 1;
  for (uint32_t d = 0; d < rank; ++d) {
    if (d != dim && idx_shape[d] > inp_shape[d]) return KUIOPS_EINVAL;   // shape_le off the gathered axis
    numel *= idx_shape[d];
    total_addr *= inp_shape[d];
  }
  if (numel == 0 || n != numel) return KUIOPS_EINVAL;
  CoordMap cm;
  build_coord_map(rank, dim, idx_shape, inp_shape, cm);
  cudaStream_t st = as_stream(s);
  // innermost-axis gather that takes a fair share of each input row: stage the row on chip
  if (cm.dim_stride == 1 && (cm.rank == 1 || (cm.rank == 2 && cm.stride[0] == cm.dim_size))) {
    const uint64_t rows_w = cm.rank == 2 ? cm.shape[0] : 1, cols_w = cm.shape[cm.rank - 1], cols_f = cm.dim_size;
    const RowsLaunch rl = rows_launch(rows_w, cols_f, elem_bytes);
    if (rl.ok && cols_w * 4 >= cols_f) {
#define RCASE(B, WT)                                                                                          \
  case B: if (!allow_smem(gather_rows_kernel<WT>, rl.smem)) return KUIOPS_ELAUNCH;                             \
    gather_rows_kernel<WT><<<rl.grid, rl.threads, rl.smem, st>>>(rows_w, cols_w, cols_f, static_cast<const WT*>(inp), idx, \
                                                                  static_cast<WT*>(out), status); break;
      switch (elem_bytes) { RCASE(1, uint8_t) RCASE(2, uint16_t) RCASE(4, uint32_t) RCASE(8, uint64_t) }
#undef RCASE
      return check_launch();
    }
  }
  unsigned grid = stream_grid(n, 256 * 2, 16);
#define ARGS cm, static_cast<const W*>(inp), idx, static_cast<W*>(out), n, status
  {
    const bool small = n < (1ull << 31) && total_addr < (1ull << 32);
    switch (elem_bytes) {
#define GCASE(B, WT)                                                                                          \
  case B: { using W = WT;                                                                                     \
    if (small) gather_kernel<W, uint32_t><<<grid, 256, 0, st>>>(ARGS);                                        \
    else gather_kernel<W, uint64_t><<<grid, 256, 0, st>>>(ARGS); } break;
      GCASE(1, uint8_t) GCASE(2, uint16_t) GCASE(4, uint32_t) GCASE(8, uint64_t)
#undef GCASE
    }
  }
#undef ARGS
  return check_launch();
}

int kuiops_scatter(uint32_t elem_bytes, uint32_t rank, uint32_t dim, const uint64_t* self_shape,
                   const uint64_t* src_shape, const void* self_, const void* src, const int64_t* idx, void* out,
                   uint64_t n, int32_t* status, kuiops_stream_t s) {
  if (!elem_ok(elem_bytes) || rank == 0 || rank > KUIOPS_MAX_RANK || dim >= rank) return KUIOPS_EINVAL;
  if (!self_shape || !src_shape || !self_ || !src || !idx || !out) return KUIOPS_EINVAL;
  uint64_t numel = 1, total_addr = 1;
  for (uint32_t d = 0; d < rank; ++d) {
    // an injective index map cannot address more cells than the axis has, so <= holds on `dim` too
    if (src_shape[d] > self_shape[d]) return KUIOPS_EINVAL;
    numel *= src_shape[d];
    total_addr *= self_shape[d];
  }
  if (numel == 0 || n != numel || total_addr == 0) return KUIOPS_EINVAL;
  cudaStream_t st = as_stream(s);
  CoordMap cm;
  build_coord_map(rank, dim, src_shape, self_shape, cm);
  // innermost-axis scatter: clone and scatter row by row through shared memory, one pass
  if (cm.dim_stride == 1 && (cm.rank == 1 || (cm.rank == 2 && cm.stride[0] == cm.dim_size))) {
    const uint64_t rows_w = cm.rank == 2 ? cm.shape[0] : 1, cols_w = cm.shape[cm.rank - 1], cols_f = cm.dim_size;
    const uint64_t rows_f = total_addr / cols_f;
    const RowsLaunch rl = rows_launch(rows_f, cols_f, elem_bytes);
    if (rl.ok) {
#define RCASE(B, WT)                                                                                          \
  case B: if (!allow_smem(scatter_rows_kernel<WT>, rl.smem)) return KUIOPS_ELAUNCH;                            \
    scatter_rows_kernel<WT><<<rl.grid, rl.threads, rl.smem, st>>>(rows_f, rows_w, cols_w, cols_f,              \
        static_cast<const WT*>(self_), static_cast<const WT*>(src), idx, static_cast<WT*>(out), status); break;
      switch (elem_bytes) { RCASE(1, uint8_t) RCASE(2, uint16_t) RCASE(4, uint32_t) RCASE(8, uint64_t) }
#undef RCASE
      return check_launch();
    }
  }
  if (self_ != out) {
    int rc = copy_bytes(self_, out, total_addr * elem_bytes, st);
    if (rc != KUIOPS_OK) return rc;
  }
  unsigned grid = stream_grid(n, 256 * 2, 16);
#define ARGS cm, static_cast<const W*>(src), idx, static_cast<W*>(out), n, status
  {
    const bool small = n < (1ull << 31) && total_addr < (1ull << 32);
    switch (elem_bytes) {
#define SCASE(B, WT)                                                                                          \
  case B: { using W = WT;                                                                                     \
    if (small) scatter_kernel<W, uint32_t><<<grid, 256, 0, st>>>(ARGS);                                       \
    else scatter_kernel<W, uint64_t><<<grid, 256, 0, st>>>(ARGS); } break;
      SCASE(1, uint8_t) SCASE(2, uint16_t) SCASE(4, uint32_t) SCASE(8, uint64_t)
#undef SCASE
    }
  }
#undef ARGS
  return check_launch();
}

int kuiops_cat(uint32_t elem_bytes, uint32_t rank, uint32_t dim, const uint64_t* a_shape, uint64_t b_dim,
               const void* A, const void* B, void* out, uint64_t n, kuiops_stream_t s) {
  if (!a_shape || rank == 0 || rank > KUIOPS_MAX_RANK || dim >= rank) return KUIOPS_EINVAL;
  uint64_t numel = 1;
  for (uint32_t d = 0; d < rank; ++d) numel *= (d == dim) ? a_shape[d] + b_dim : a_shape[d];
  if (n != numel || n == 0) return KUIOPS_EINVAL;       // out_dim = a_dim + b_dim, Kuiops.Cat.fsti:50-52
  const uint64_t dims[2] = {a_shape[dim], b_dim};
  const void* ptrs[2] = {A, B};
  return cat_impl(elem_bytes, rank, dim, 2, a_shape, dims, ptrs, out, as_stream(s));
}

int kuiops_cat_n(uint32_t elem_bytes, uint32_t rank, uint32_t dim, uint32_t count, const uint64_t* shape,
                 const uint64_t* dim_sizes, const void* const* ptrs, void* out, kuiops_stream_t s) {
  return cat_impl(elem_bytes, rank, dim, count, shape, dim_sizes, ptrs, out, as_stream(s));
}

int kuiops_index(uint32_t elem_bytes, uint32_t self_rank, const uint64_t* self_shape, uint32_t first_dim,
                 uint32_t n_idx, const int64_t* const* idx_ptrs, uint32_t idx_rank, const uint64_t* idx_shape,
                 const int64_t* idx_strides, const void* self_, void* out, int32_t* status, kuiops_stream_t s) {
  if (!elem_ok(elem_bytes) || self_rank == 0 || self_rank > KUIOPS_MAX_RANK) return KUIOPS_EINVAL;
  if (n_idx == 0 || n_idx > 4 || first_dim + n_idx > self_rank || idx_rank > KUIOPS_MAX_RANK) return KUIOPS_EINVAL;
  if (!self_shape || !idx_ptrs || (idx_rank && (!idx_shape || !idx_strides)) || !self_ || !out) return KUIOPS_EINVAL;
  IndexParams p = {};
  p.n_idx = n_idx; p.idx_rank = idx_rank;
  p.pre = 1; p.nb = 1; p.inner = 1;
  for (uint32_t d = 0; d < first_dim; ++d) p.pre *= self_shape[d];
  for (uint32_t d = first_dim + n_idx; d < self_rank; ++d) p.inner *= self_shape[d];
  for (uint32_t d = 0; d < idx_rank; ++d) { p.idx_shape[d] = idx_shape[d]; p.nb *= idx_shape[d]; }
  uint64_t st_run = 1;
  for (int k = int(n_idx) - 1; k >= 0; --k) {
    if (!idx_ptrs[k]) return KUIOPS_EINVAL;
    p.idx[k] = idx_ptrs[k];
    p.dim_size[k] = self_shape[first_dim + k];
    p.dim_stride[k] = st_run * p.inner;
    st_run *= self_shape[first_dim + k];
    for (uint32_t d = 0; d < idx_rank; ++d) p.idx_stride[k][d] = idx_strides[k * idx_rank + d];
  }
  p.self_pre_stride = st_run * p.inner;
  if (p.pre == 0 || p.nb == 0 || p.inner == 0) return KUIOPS_EINVAL;
  // move trailing runs as the widest word that divides them
  uint32_t word = elem_bytes;
  const uint64_t inner_bytes = p.inner * elem_bytes;
  for (uint32_t w = 16; w > elem_bytes; w >>= 1)
    if (inner_bytes % w == 0 && reinterpret_cast<uintptr_t>(self_) % w == 0 && reinterpret_cast<uintptr_t>(out) % w == 0) { word = w; break; }
  const uint64_t scale = word / elem_bytes;
  p.inner /= scale;
  for (uint32_t k = 0; k < n_idx; ++k) p.dim_stride[k] /= scale;
  p.self_pre_stride /= scale;
  const uint64_t total = p.pre * p.nb * p.inner;
  unsigned grid = stream_grid(total, 256 * 2, 16);
  cudaStream_t st = as_stream(s);
  switch (word) {
    case 16: index_kernel<int4><<<grid, 256, 0, st>>>(p, static_cast<const int4*>(self_), static_cast<int4*>(out), status); break;
    case 8: index_kernel<uint64_t><<<grid, 256, 0, st>>>(p, static_cast<const uint64_t*>(self_), static_cast<uint64_t*>(out), status); break;
    case 4: index_kernel<uint32_t><<<grid, 256, 0, st>>>(p, static_cast<const uint32_t*>(self_), static_cast<uint32_t*>(out), status); break;
    case 2: index_kernel<uint16_t><<<grid, 256, 0, st>>>(p, static_cast<const uint16_t*>(self_), static_cast<uint16_t*>(out), status); break;
    default: index_kernel<uint8_t><<<grid, 256, 0, st>>>(p, static_cast<const uint8_t*>(self_), static_cast<uint8_t*>(out), status); break;
  }
  return check_launch();
}

int kuiops_isin_i64(uint64_t n, const int64_t* elements, uint64_t m, const int64_t* test_elements, int invert,
                    void* out, kuiops_stream_t s) {
  if (n == 0 || !elements || !out) return KUIOPS_EINVAL;
  if (m > 0 && !test_elements) return KUIOPS_EINVAL;
  // each block rebuilds the hash table, so give a block enough elements to amortise that
  uint64_t per_block = 4096;
  uint64_t blocks = (n + per_block - 1) / per_block;
  if (blocks > uint64_t(num_sms()) * 8) {
    blocks = uint64_t(num_sms()) * 8;
    per_block = ((n + blocks - 1) / blocks + 7) / 8 * 8;
    blocks = (n + per_block - 1) / per_block;
  }
  if (m == 0) {
    // empty test set: everything is "not in"
    return cudaMemsetAsync(out, invert ? 1 : 0, n, as_stream(s)) == cudaSuccess ? KUIOPS_OK : KUIOPS_ELAUNCH;
  }
  const int vec_ok = aligned16(elements) && (reinterpret_cast<uintptr_t>(out) % 8 == 0);
  isin_kernel<<<unsigned(blocks), 512, 0, as_stream(s)>>>(n, elements, m, test_elements, invert,
                                                          static_cast<uint8_t*>(out), per_block, vec_ok);
  return check_launch();
}

}  // extern "C"
