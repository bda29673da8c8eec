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
// The test set is sorted in shared memory one tile at a time (bitonic, kIsinTile entries) and
// every element does a binary search per tile.  A 1024-entry stop-id set is one tile.
constexpr int kIsinTile = 4096;

__global__ void __launch_bounds__(512)
isin_kernel(uint64_t n, const int64_t* __restrict__ elems, uint64_t m, const int64_t* __restrict__ tests, int invert,
            uint8_t* __restrict__ out, uint64_t per_block) {
  __shared__ long long tile[kIsinTile];
  const uint64_t lo = uint64_t(blockIdx.x) * per_block;
  const uint64_t hi = lo + per_block < n ? lo + per_block : n;
  if (lo >= n) return;
  for (uint64_t t0 = 0; t0 < m; t0 += kIsinTile) {
    const uint32_t cnt = uint32_t(m - t0 < uint64_t(kIsinTile) ? m - t0 : uint64_t(kIsinTile));
    uint32_t pow2 = 1;
    while (pow2 < cnt) pow2 <<= 1;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < pow2; i += blockDim.x) tile[i] = i < cnt ? tests[t0 + i] : LLONG_MAX;
    __syncthreads();
    for (uint32_t k = 2; k <= pow2; k <<= 1) {
      for (uint32_t j = k >> 1; j > 0; j >>= 1) {
        for (uint32_t i = threadIdx.x; i < pow2; i += blockDim.x) {
          const uint32_t l = i ^ j;
          if (l > i) {
            const long long a = tile[i], b = tile[l];
            const bool up = (i & k) == 0;
            if ((a > b) == up) { tile[i] = b; tile[l] = a; }
          }
        }
        __syncthreads();
      }
    }
    for (uint64_t e = lo + threadIdx.x; e < hi; e += blockDim.x) {
      const long long v = elems[e];
      uint32_t a = 0, b = cnt;       // first position with tile[pos] >= v
      while (a < b) {
        const uint32_t mid = (a + b) >> 1;
        if (tile[mid] < v) a = mid + 1; else b = mid;
      }
      const bool hit = a < cnt && tile[a] == v;
      if (t0 == 0) out[e] = hit ? 1 : 0;
      else if (hit) out[e] = 1;
    }
  }
  if (invert) {
    __syncthreads();
    for (uint64_t e = lo + threadIdx.x; e < hi; e += blockDim.x) out[e] = out[e] ? 0 : 1;
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
  if (self_ != out) {
    int rc = copy_bytes(self_, out, total_addr * elem_bytes, st);
    if (rc != KUIOPS_OK) return rc;
  }
  CoordMap cm;
  build_coord_map(rank, dim, src_shape, self_shape, cm);
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
  // each block re-sorts the test set, so give a block enough elements to amortise that
  uint64_t per_block = 2048;
  uint64_t blocks = (n + per_block - 1) / per_block;
  if (blocks > uint64_t(kNumSMs) * 4) { blocks = uint64_t(kNumSMs) * 4; per_block = (n + blocks - 1) / blocks; }
  if (m == 0) {
    // empty test set: everything is "not in"
    return cudaMemsetAsync(out, invert ? 1 : 0, n, as_stream(s)) == cudaSuccess ? KUIOPS_OK : KUIOPS_ELAUNCH;
  }
  isin_kernel<<<unsigned(blocks), 512, 0, as_stream(s)>>>(n, elements, m, test_elements, invert,
                                                          static_cast<uint8_t*>(out), per_block);
  return check_launch();
}

}  // extern "C"
