// tcgen05 GEMM for bf16 / f16 operands with fp32 accumulation in tensor memory.
//
// One kernel template serves two operand placements.  The 128 TMEM lanes carry the "P" operand
// and the BN TMEM columns the "Q" operand:
//   * normal  (M > 128): P = A rows (m), Q = B columns (n); persistent CTAs walk 128 x BN tiles
//     with two accumulator stages so the epilogue of a tile overlaps the MMAs of the next.
//   * swapped (M <= 128, decode shapes): P = B columns (n, the weight rows that have to be
//     streamed from HBM), Q = A rows (m, padded to 16..128).  K is split over several CTAs per
//     tile (one thread-block cluster per tile) so that every SM streams weights; the fp32
//     partials stay in shared memory and are summed in slice order through distributed shared
//     memory, each CTA finishing a share of the tile's columns (in-kernel reduction,
//     deterministic, no global scratch).
// Warp roles: warp 0 = TMA producer (one lane), warp 1 = TMEM allocator + UMMA issuer (one
// lane), warps 2..5 = epilogue (TMEM -> registers -> alpha/beta/bias -> global); the normal
// placement adds warps 6..9 as a second epilogue group, one group per accumulator stage, so that
// short-K problems whose time is all epilogue (bmm with K = 128) drain two tiles at once.
// Operands arrive through 3-D tensor maps (inner, rows, batch) with 128-byte swizzle; edges in
// M, N and K rely on TMA zero fill, so no divisibility is required beyond the 16-byte stride
// rule.  Replaces Klas.GEMM.TensorCore2D (wmma fragments, kuiops/mm/Kuiops.Mm.Inst.fst.j2:9-11).
#include "gemm.cuh"
#include "tc_ptx.cuh"
#include <cooperative_groups.h>
#include <mutex>
#include <type_traits>
#include <string>
#include <unordered_map>
#include <cstdio>

namespace cg = cooperative_groups;
namespace kuiops {

constexpr int TBM = 128;   // TMEM lanes = rows of the P operand per tile
constexpr int TBK = 64;    // K elements per pipeline stage (one 128-byte swizzle span)
constexpr int kTcThreads = 192;        // swapped placement: one epilogue warpgroup
constexpr int kTcThreadsWide = 320;    // normal placement: one epilogue warpgroup per accumulator stage

struct TcParams {
  uint32_t rowsP, rowsQ, K, batch;
  uint32_t tilesP, tilesQ, splits, kblocks, kb_per_split;
  uint32_t bandP;            // P tiles per rasterisation band
  int swapped, out_f32, epi;
  uint32_t M, N;
  float alpha, beta;
  const void* Cin; int64_t ldcin, stride_cin;
  void* C; int64_t ldc, stride_c;
  unsigned int* err;
  // "push" epilogue (tensor parallel, swapped placement only): the result is a partial sum that
  // goes into slot (epoch & 1, my_rank) of every rank's receive area instead of C, as 8-byte cells of
  // two elements and the stamp epoch + 1: a cell is valid the moment it is seen with the right
  // stamp, so the exchange needs no fence, no flag and no last-CTA election
  uint32_t n_ranks, my_rank;          // n_ranks == 0: ordinary epilogue
  uint64_t peer_base[KUIOPS_MAX_PEERS];
  uint64_t slot_bytes;
  const unsigned int* epoch;          // device word, advanced by the consumer of the partials
  // "rope" epilogue (epi == 2, swapped placement, split K): the output rows are packed q | k | v heads
  // of 128; q and k heads get the rotary embedding of their row's position, k and v heads are also
  // appended to the caches
  // RMSNorm folded into a pair of GEMMs (swapped placement): a producer leaves, per 128-feature tile and
  // row, the sum of squares of what it stored (ssq_out[tile * M + m]); a consumer whose A operand is
  // that output multiplies row m of its product by rsqrt(sum over tiles / K + eps)
  float* ssq_out;
  const float* ssq_in;
  uint32_t ssq_tiles;
  float ssq_eps;
  unsigned long long* trace;          // debug: CTA 0 stores %globaltimer at the stations of its critical path (kuiops_debug_gemm_trace)
  const long long* positions;
  float log2_theta;
  void* k_cache; void* v_cache;
  uint64_t cache_cap;
  uint32_t hq, hk, rows_per_seq;
};

__device__ unsigned int g_tc_error = 0;
// Debug: device buffer of >= 16 uint64 that CTA 0 of every later tcgen05 GEMM stamps with %globaltimer.
std::atomic<unsigned long long*> g_gemm_trace{nullptr};
std::atomic<int> g_gemm_sm_reserve{0};

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_stamp(const unsigned long long* base, int slot) {
  if (base != nullptr && blockIdx.x == 0) const_cast<unsigned long long*>(base)[slot] = global_ns();
}
// Wait on an mbarrier phase for at most ~2 s of wall time.
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity) {
  if (tc::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  while (!tc::mbar_try_wait(bar, parity)) {
    if (global_ns() - t0 > 2000000000ull) return false;
  }
  return true;
}

// Tile t of a batch -> (P tile, Q tile).  Tiles are walked down the P axis in bands of p.bandP
// P-tiles, all Q tiles of a band before the next band: the CTAs that run at the same time then
// share a band of the P operand (32 tiles x 128 rows x K: it stays in L2 while the Q operand
// streams past) instead of each re-reading a P panel that no longer fits the cache when the P
// extent is large (prefill: 65536 rows).
__device__ __forceinline__ void tile_coords(const TcParams& p, uint32_t t, uint32_t& tp, uint32_t& tq) {
  const uint32_t band_tiles = p.bandP * p.tilesQ;
  const uint32_t band = t / band_tiles, r = t % band_tiles;
  const uint32_t first = band * p.bandP;
  const uint32_t height = min(p.bandP, p.tilesP - first);      // the last band may be shorter
  tp = first + r % height;
  tq = r / height;
}

template <typename TIN>
__device__ __forceinline__ void store_elem(const TcParams& p, uint32_t b, uint32_t lane_row, uint32_t col, float acc) {
  const uint32_t m = p.swapped ? col : lane_row;
  const uint32_t n = p.swapped ? lane_row : col;
  if (m >= p.M || n >= p.N) return;
  float v = p.alpha * acc;
  if (p.Cin) {
    const TIN* cin = static_cast<const TIN*>(p.Cin) + size_t(b) * p.stride_cin;
    v += p.beta * ElemTraits<TIN>::to_f(cin[size_t(m) * p.ldcin + n]);
  }
  const size_t off = size_t(b) * p.stride_c + size_t(m) * p.ldc + n;
  if (p.out_f32) static_cast<float*>(p.C)[off] = v;
  else static_cast<TIN*>(p.C)[off] = ElemTraits<TIN>::from_f(v);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

// SwiGLU epilogue, swapped placement: lane n holds column n of the fused gate|up product for row
// `col`; gate and up of one output sit in neighbouring lanes (rows 2j, 2j+1 of the weight).
// Warp-collective: every lane of the warp must call it.
template <typename TIN>
__device__ __forceinline__ void store_swiglu_swapped(const TcParams& p, uint32_t lane_row, uint32_t col, float acc) {
  const float other = __shfl_xor_sync(0xffffffffu, acc, 1);
  if ((lane_row & 1u) || col >= p.M || lane_row >= p.N) return;
  const float v = silu_mul(acc, other);
  const size_t off = size_t(col) * p.ldc + (lane_row >> 1);
  if (p.out_f32) static_cast<float*>(p.C)[off] = v;
  else static_cast<TIN*>(p.C)[off] = ElemTraits<TIN>::from_f(v);
}

// Rotary embedding + KV-cache append on a finished element of the packed QKV projection (swapped
// placement: lane_row = output feature n, col = row m).  `acc` is the element itself, `pacc` its
// partner at feature n ^ 64 inside the same head of 128.  The arithmetic repeats, rounding for
// rounding, what the separate kernel does on the stored projection (and what eager does): the
// projection is rounded to the element type first, cos / sin are computed in fp32 and rounded,
// each product and the sum are rounded.
template <typename TIN>
__device__ __forceinline__ void store_rope(const TcParams& p, uint32_t lane_row, uint32_t col, float acc, float pacc) {
  const uint32_t m = col, n = lane_row;
  if (m >= p.M || n >= p.N) return;
  auto rnd = [](float x) { return ElemTraits<TIN>::to_f(ElemTraits<TIN>::from_f(x)); };
  const uint32_t head = n >> 7, j = n & 127u, i = j & 63u;
  const bool hi = j >= 64;
  const long long pos = p.positions[m];
  const float own = rnd(p.alpha * acc), partner = rnd(p.alpha * pacc);
  float val = own;
  if (head < p.hq + p.hk) {
    const float inv_freq = exp2f(-p.log2_theta * (2.f * float(i) / 128.f));
    float sn, cs;
    sincosf(float(pos) * inv_freq, &sn, &cs);
    const float csr = rnd(cs), snr = rnd(sn);
    const float a = hi ? partner : own, b = hi ? own : partner;      // (x[i], x[i + 64])
    val = hi ? rnd(rnd(b * csr) + rnd(a * snr)) : rnd(rnd(a * csr) + rnd(-b * snr));
  }
  const TIN out = ElemTraits<TIN>::from_f(val);
  static_cast<TIN*>(p.C)[size_t(m) * p.ldc + n] = out;
  if (head >= p.hq && p.k_cache != nullptr && pos >= 0 && uint64_t(pos) < p.cache_cap) {
    const bool is_k = head < p.hq + p.hk;
    const uint32_t kvh = is_k ? head - p.hq : head - p.hq - p.hk;
    const uint64_t seq = m / p.rows_per_seq;
    TIN* dst = static_cast<TIN*>(is_k ? p.k_cache : p.v_cache) + ((seq * p.hk + kvh) * p.cache_cap + uint64_t(pos)) * 128 + j;
    *dst = out;
  }
}

// Four consecutive output features n0 .. n0 + 3 of row m (swapped placement), finished: the plain /
// bias / push epilogue with one 8-byte store per destination where alignment allows.
// Returns the sum of squares of the values as stored (rounded to the output type; 0 where nothing is stored).
template <typename TIN>
__device__ __forceinline__ float store_quad(const TcParams& p, uint32_t b, uint32_t n0, uint32_t m, const float (&acc)[4], uint64_t push_off,
                                            uint32_t push_stamp) {
  if (m >= p.M || n0 >= p.N) return 0.f;
  const bool full = n0 + 4 <= p.N;
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = p.alpha * acc[i];
  if (p.n_ranks) {
    // the same two cells of the (epoch & 1, my_rank) slot on every rank, this one included: 16 bytes per
    // destination, each 8-byte half carrying two elements and the stamp (N is a multiple of 4 here)
    const uint64_t off = push_off + (size_t(m) * p.N + n0) * 4;
    const uint4 w = make_uint4(pack2<TIN>(v[0], v[1]), push_stamp, pack2<TIN>(v[2], v[3]), push_stamp);
#pragma unroll 1
    for (uint32_t r = 0; r < p.n_ranks; ++r) *reinterpret_cast<uint4*>(p.peer_base[r] + off) = w;
    return 0.f;
  }
  if (p.Cin) {
    const TIN* cin = static_cast<const TIN*>(p.Cin) + size_t(b) * p.stride_cin + size_t(m) * p.ldcin + n0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (n0 + i < p.N) v[i] += p.beta * ElemTraits<TIN>::to_f(cin[i]);
  }
  const size_t off = size_t(b) * p.stride_c + size_t(m) * p.ldc + n0;
  float ss = 0.f;
  if (p.out_f32) {
    float* dst = static_cast<float*>(p.C) + off;
#pragma unroll
    for (int i = 0; i < 4; ++i) if (n0 + i < p.N) ss += v[i] * v[i];
    if (full && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    else {
#pragma unroll
      for (int i = 0; i < 4; ++i) if (n0 + i < p.N) dst[i] = v[i];
    }
  } else {
    TIN* dst = static_cast<TIN*>(p.C) + off;
    TIN r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[i] = ElemTraits<TIN>::from_f(v[i]);
      const float f = ElemTraits<TIN>::to_f(r[i]);
      if (n0 + i < p.N) ss += f * f;
    }
    if (full && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) *reinterpret_cast<uint2*>(dst) = make_uint2(pack2<TIN>(v[0], v[1]), pack2<TIN>(v[2], v[3]));
    else {
#pragma unroll
      for (int i = 0; i < 4; ++i) if (n0 + i < p.N) dst[i] = r[i];
    }
  }
  return ss;
}

// SwiGLU on four consecutive columns of the fused gate|up product (two (gate, up) pairs) of row m.
template <typename TIN>
__device__ __forceinline__ void store_swiglu_quad(const TcParams& p, uint32_t n0, uint32_t m, const float (&acc)[4]) {
  if (m >= p.M) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (n0 + 2 * i + 1 < p.N) {
      const float v = silu_mul(acc[2 * i], acc[2 * i + 1]);
      const size_t off = size_t(m) * p.ldc + ((n0 >> 1) + i);
      if (p.out_f32) static_cast<float*>(p.C)[off] = v;
      else static_cast<TIN*>(p.C)[off] = ElemTraits<TIN>::from_f(v);
    }
  }
}

// Split-K reduction of one output tile whose SPLITS K-slices are parked, column-major fp32, in the
// shared memory of the SPLITS CTAs of a cluster.  CTA `rank` finishes columns rank, rank + SPLITS, ...
// A warp takes whole columns: lane L reads the four features 4 L .. 4 L + 3 of a column from every
// slice with one 16-byte distributed-shared-memory load each (a quarter of the requests of a
// scalar walk; the remote reads are what this phase waits for), sums them and runs the epilogue
// on the four results.  The loads of a step go to SPLITS different CTAs, starting with the
// reader's own (CTA r reads slice r, r + 1, ... cyclically), so that the readers do not all queue
// at the same CTA; a column is summed in that cyclic order, which is fixed by the column alone
// (its owner is column mod SPLITS): same plan, same bits.
template <typename TIN, int SPLITS>
__device__ __forceinline__ void reduce_tile(const TcParams& p, cg::cluster_group& cluster, float* red, uint32_t rank, uint32_t ncols,
                                            uint32_t warp_in_group, uint32_t lane, uint32_t b, uint32_t tp, uint32_t col0, uint64_t push_off,
                                            uint32_t push_stamp, const float* row_scale) {
  constexpr int CW = SPLITS >= 5 ? 1 : (SPLITS >= 3 ? 2 : 4);      // columns a warp has in flight: CW * SPLITS <= 8 loads of 16 bytes
  const float* peer[SPLITS];
#pragma unroll
  for (int s = 0; s < SPLITS; ++s) {
    uint32_t src = rank + s;
    if (src >= SPLITS) src -= SPLITS;
    peer[s] = cluster.map_shared_rank(red, src);
  }
  const uint32_t nj = ncols > rank ? (ncols - rank + SPLITS - 1) / SPLITS : 0u;
  const uint32_t n0 = tp * TBM + lane * 4;                          // first of this lane's four output features
  for (uint32_t j0 = warp_in_group * CW; j0 < nj; j0 += 4 * CW) {
    float4 v[CW][SPLITS];
#pragma unroll
    for (int j = 0; j < CW; ++j) {
      const uint32_t c = rank + (j0 + j) * SPLITS;
#pragma unroll
      for (int s = 0; s < SPLITS; ++s)
        v[j][s] = (j0 + j < nj) ? *reinterpret_cast<const float4*>(peer[s] + c * TBM + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sum[CW][4], psum[CW][4];
#pragma unroll
    for (int j = 0; j < CW; ++j) {
      sum[j][0] = v[j][0].x; sum[j][1] = v[j][0].y; sum[j][2] = v[j][0].z; sum[j][3] = v[j][0].w;
#pragma unroll
      for (int s = 1; s < SPLITS; ++s) { sum[j][0] += v[j][s].x; sum[j][1] += v[j][s].y; sum[j][2] += v[j][s].z; sum[j][3] += v[j][s].w; }
#pragma unroll
      for (int i = 0; i < 4; ++i) psum[j][i] = 0.f;
    }
    if (p.epi == 2) {
      // the rotary partners (features n ^ 64 of the same head), summed the same way
#pragma unroll
      for (int j = 0; j < CW; ++j) {
        const uint32_t c = rank + (j0 + j) * SPLITS;
#pragma unroll
        for (int s = 0; s < SPLITS; ++s)
          v[j][s] = (j0 + j < nj) ? *reinterpret_cast<const float4*>(peer[s] + c * TBM + ((lane * 4) ^ 64u)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < CW; ++j) {
        psum[j][0] = v[j][0].x; psum[j][1] = v[j][0].y; psum[j][2] = v[j][0].z; psum[j][3] = v[j][0].w;
#pragma unroll
        for (int s = 1; s < SPLITS; ++s) { psum[j][0] += v[j][s].x; psum[j][1] += v[j][s].y; psum[j][2] += v[j][s].z; psum[j][3] += v[j][s].w; }
      }
    }
#pragma unroll
    for (int j = 0; j < CW; ++j) {
      if (j0 + j < nj) {
        const uint32_t m = col0 + rank + (j0 + j) * SPLITS;
        if (row_scale != nullptr) {
          // the folded RMSNorm of the A operand: one factor per output row
          const float rs = row_scale[rank + (j0 + j) * SPLITS];
#pragma unroll
          for (int i = 0; i < 4; ++i) { sum[j][i] *= rs; psum[j][i] *= rs; }
        }
        if (p.epi == 2) {
#pragma unroll
          for (int i = 0; i < 4; ++i) store_rope<TIN>(p, n0 + i, m, sum[j][i], psum[j][i]);
        } else if (p.epi == 1) {
          store_swiglu_quad<TIN>(p, n0, m, sum[j]);
        } else {
          float ss = store_quad<TIN>(p, b, n0, m, sum[j], push_off, push_stamp);
          if (p.ssq_out != nullptr) {
            // this warp holds all 128 features of tile tp for row m: their sum of squares, for the norm of the consumer
            ss = warp_sum(ss);
            if (lane == 0 && m < p.M) p.ssq_out[size_t(tp) * p.M + m] = ss;
          }
        }
      }
    }
  }
}

template <typename TIN, int BN, int STAGES, int ACC_STAGES, bool P_MN, bool Q_MN>
// (the weight-streaming variants are sized for three CTAs per SM: registers included)
__global__ void __launch_bounds__(ACC_STAGES == 2 ? kTcThreadsWide : kTcThreads, ACC_STAGES == 2 ? 1 : 3)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmapP, const __grid_constant__ CUtensorMap tmapQ,
               const TcParams p) {
  constexpr uint32_t P_BYTES = TBM * TBK * 2;
  constexpr uint32_t Q_BYTES = BN * TBK * 2;
  constexpr uint32_t STAGE_BYTES = P_BYTES + Q_BYTES;
  constexpr uint32_t TMEM_COLS = (ACC_STAGES * BN) < 32 ? 32 : (ACC_STAGES * BN);
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns must be a power of two <= 512");
  static_assert(!Q_MN || BN % 64 == 0, "an MN-major Q tile is loaded in 64-element boxes");

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle atoms need
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_STAGES);
  // normal placement only: 4 KB per epilogue warp (8 warps) to turn row-per-thread results into row-contiguous stores
  unsigned char* epi_stage = smem + STAGES * STAGE_BYTES + 256;
  // swapped placement: per-row factors of a folded RMSNorm (at most 128 rows)
  float* rs_s = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t tiles_per_batch = p.tilesP * p.tilesQ;
  const uint32_t units = tiles_per_batch * p.batch * p.splits;
  // one pipeline stage: the P and Q tiles of k-block kb of tile (tp, tq) of batch b
  auto issue_stage = [&](uint32_t s, uint32_t kb, uint32_t tp, uint32_t tq, uint32_t b) {
    unsigned char* ps = smem + s * STAGE_BYTES;
    unsigned char* qs = ps + P_BYTES;
    tc::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
    const int k0 = int(kb * TBK);
    if (P_MN) {
#pragma unroll
      for (int j = 0; j < TBM / 64; ++j)
        tc::tma_load_3d(ps + j * (TBK * 128), &tmapP, &full_bar[s], int(tp * TBM) + j * 64, k0, int(b));
    } else {
      tc::tma_load_3d(ps, &tmapP, &full_bar[s], k0, int(tp * TBM), int(b));
    }
    if (Q_MN) {
#pragma unroll
      for (int j = 0; j < BN / 64; ++j)
        tc::tma_load_3d(qs + j * (TBK * 128), &tmapQ, &full_bar[s], int(tq * BN) + j * 64, k0, int(b));
    } else {
      tc::tma_load_3d(qs, &tmapQ, &full_bar[s], k0, int(tq * BN), int(b));
    }
  };
  uint32_t npre = 0;          // stages of the first unit already requested during set-up (thread 0 only)

  if (threadIdx.x == 0) {
    trace_stamp(p.trace, 0);                                    // CTA started
    tc::prefetch_tmap(&tmapP);
    tc::prefetch_tmap(&tmapQ);
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full_bar[s], 1); tc::mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < ACC_STAGES; ++s) { tc::mbar_init(&acc_full[s], 1); tc::mbar_init(&acc_empty[s], 4); }
    tc::fence_barrier_init();
    // The first copies need nothing but these barriers: start them now, so that they fly while the
    // tensor memory is being allocated and the CTA meets below.  (The operands may still be being
    // written by the previous kernel in the stream: wait for it first.)
    pdl_wait();
    trace_stamp(p.trace, 1);                                    // the previous kernel in the stream has completed
    if (blockIdx.x < units) {
      const uint32_t u = blockIdx.x, split = u % p.splits, tile = u / p.splits;
      const uint32_t b = tile / tiles_per_batch, t = tile % tiles_per_batch;
      uint32_t tp, tq;
      tile_coords(p, t, tp, tq);
      const uint32_t kb0 = split * p.kb_per_split;
      const uint32_t kb1 = min(kb0 + p.kb_per_split, p.kblocks);
      npre = min(uint32_t(STAGES), kb1 - kb0);
      for (uint32_t i = 0; i < npre; ++i) issue_stage(i, kb0 + i, tp, tq, b);
    }
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched only this CTA's shared memory, TMEM and the kernel parameters; the
  // operands may still be being written by the previous kernel in the stream
  if (threadIdx.x != 0) pdl_wait();      // thread 0 did before it started the first copies
  pdl_trigger();
  // push epilogue: which half of the double-buffered receive areas this launch writes
  unsigned int push_epoch = 0;
  uint64_t push_off = 0;
  if (p.n_ranks) {
    push_epoch = *reinterpret_cast<const volatile unsigned int*>(p.epoch);
    push_off = (uint64_t(push_epoch & 1u) * p.n_ranks + p.my_rank) * p.slot_bytes;
  }

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const uint32_t split = u % p.splits, tile = u / p.splits;
        const uint32_t b = tile / tiles_per_batch, t = tile % tiles_per_batch;
        uint32_t tp, tq;
        tile_coords(p, t, tp, tq);
        const uint32_t kb0 = split * p.kb_per_split;
        const uint32_t kb1 = min(kb0 + p.kb_per_split, p.kblocks);
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
          if (it < npre) continue;                    // requested during set-up
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!bounded_wait(&empty_bar[s], ph ^ 1)) { atomicExch(p.err, 1u); ok = false; break; }
          issue_stage(s, kb, tp, tq, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ UMMA issuer -------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = tc::make_idesc(std::is_same<TIN, __nv_bfloat16>::value ? 1 : 0, P_MN ? 1 : 0, Q_MN ? 1 : 0, TBM, BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x, ++acc_it) {
        const uint32_t split = u % p.splits;
        const uint32_t kb0 = split * p.kb_per_split;
        const uint32_t kb1 = min(kb0 + p.kb_per_split, p.kblocks);
        const uint32_t as = acc_it % ACC_STAGES, aph = (acc_it / ACC_STAGES) & 1;
        if (!bounded_wait(&acc_empty[as], aph ^ 1)) { atomicExch(p.err, 2u); ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (uint32_t kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!bounded_wait(&full_bar[s], ph)) { atomicExch(p.err, 3u); ok = false; break; }
          if (it == 0) trace_stamp(p.trace, 2);                 // first operand tiles have landed
          tc::tc_fence_after();
          const uint32_t pa = tc::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t qa = pa + P_BYTES;
#pragma unroll
          for (int kk = 0; kk < TBK / 16; ++kk) {
            // K-major: 16 elements = 32 bytes inside the swizzle span, 8-row groups 1024 B apart.
            // MN-major: 16 k-rows = 2048 B, 8-row groups 1024 B apart, 64-element column blocks
            // TBK * 128 B apart.
            const uint64_t da = P_MN ? tc::make_smem_desc(pa + kk * 2048, TBK * 128, 1024)
                                     : tc::make_smem_desc(pa + kk * 32, 16, 1024);
            const uint64_t db = Q_MN ? tc::make_smem_desc(qa + kk * 2048, TBK * 128, 1024)
                                     : tc::make_smem_desc(qa + kk * 32, 16, 1024);
            tc::umma_f16(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          tc::umma_commit(&empty_bar[s]);     // stage may be refilled once these MMAs have read it
        }
        if (ok) tc::umma_commit(&acc_full[as]);
        if (acc_it == 0) trace_stamp(p.trace, 3);               // every MMA of the first unit issued
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------------------
    const uint32_t quarter = warp & 3;                    // TMEM lanes this warp may touch
    const uint32_t lane_in_tile = quarter * 32 + lane;
    if (ACC_STAGES == 1 && p.ssq_in != nullptr) {
      // folded RMSNorm: thread t adds up the tile partials of row t in tile order and keeps the row's factor;
      // this runs while the main loop streams, the four epilogue warps meet on their own barrier
      const uint32_t t = threadIdx.x - 64;
      if (t < p.M) {
        float ssq = 0.f;
        for (uint32_t q = 0; q < p.ssq_tiles; ++q) ssq += p.ssq_in[size_t(q) * p.M + t];
        rs_s[t] = rsqrtf(ssq / float(p.K) + p.ssq_eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    // facts that allow 16-byte stores of 8 consecutive outputs of a row (normal placement only)
    const bool c_vec = !p.swapped && !p.out_f32 && (p.ldc % 8 == 0) && (p.stride_c % 8 == 0) &&
                       ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
    const bool cin_vec = !p.Cin || (((reinterpret_cast<uintptr_t>(p.Cin) & 15u) == 0) && (p.ldcin % 8 == 0) &&
                                    (p.stride_cin % 8 == 0));
    // epilogue group g owns accumulator stage g: it takes this CTA's tiles g, g + groups, ...
    constexpr uint32_t kGroups = ACC_STAGES == 2 ? 2 : 1;
    const uint32_t group = (warp - 2) >> 2;
    uint32_t acc_it = group;
    bool ok = true;
    for (uint32_t u = blockIdx.x + group * gridDim.x; u < units && ok; u += kGroups * gridDim.x, acc_it += kGroups) {
      const uint32_t tile = u / p.splits;
      const uint32_t b = tile / tiles_per_batch, t = tile % tiles_per_batch;
      uint32_t tp, tq;
        tile_coords(p, t, tp, tq);
      const uint32_t as = acc_it % ACC_STAGES, aph = (acc_it / ACC_STAGES) & 1;
      if (!bounded_wait(&acc_full[as], aph)) { atomicExch(p.err, 4u); ok = false; break; }
      if (acc_it == group && threadIdx.x == 64) trace_stamp(p.trace, 4);     // accumulator complete
      tc::tc_fence_after();
      const uint32_t taddr = tmem_base + as * BN + ((quarter * 32) << 16);
      const uint32_t row = tp * TBM + lane_in_tile;
      const uint32_t col0 = tq * BN;
      // columns beyond the Q extent hold zeros (TMA fill) and are never stored
      const uint32_t ncols = min(uint32_t(BN), p.rowsQ > col0 ? p.rowsQ - col0 : 0u);
      float v[16];
      if (p.splits == 1 && p.n_ranks == 0 && p.ssq_out == nullptr) {
        uint32_t c = 0;
        if (ACC_STAGES == 2 && p.epi == 0 && c_vec && (!p.Cin || (p.ldcin == 0 && cin_vec))) {
          // 64 columns at a time: a thread owns one row of the accumulator, so direct stores would
          // touch 32 rows per instruction.  The warp's 32 x 64 block goes through shared memory
          // (16-byte chunks XOR-swizzled by row, conflict-free both ways) and leaves as 128-byte
          // row segments, four rows per store instruction.
          unsigned char* stg = epi_stage + (warp - 2) * 4096;
          TIN* cbase = static_cast<TIN*>(p.C) + size_t(b) * p.stride_c + col0;
          for (; c + 64 <= ncols; c += 64) {
            float w[64];
            tc::tmem_ld32(taddr + c, w);
            tc::tmem_ld32(taddr + c + 32, w + 32);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float add[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) add[e] = 0.f;
              if (p.Cin) {
                const Vec16<TIN> bv = ld16(static_cast<const TIN*>(p.Cin) + size_t(b) * p.stride_cin + col0 + c + j * 8);
#pragma unroll
                for (int e = 0; e < 8; ++e) add[e] = p.beta * ElemTraits<TIN>::to_f(bv.v[e]);
              }
              Vec16<TIN> o;
#pragma unroll
              for (int e = 0; e < 8; ++e) o.v[e] = ElemTraits<TIN>::from_f(fmaf(p.alpha, w[j * 8 + e], add[e]));
              *reinterpret_cast<Vec16<TIN>*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t r = i * 4 + (lane >> 3), ch = lane & 7;
              const Vec16<TIN> o = *reinterpret_cast<const Vec16<TIN>*>(stg + r * 128 + ((ch ^ (r & 7)) << 4));
              const uint32_t grow = tp * TBM + quarter * 32 + r;
              if (grow < p.M) st16(cbase + size_t(grow) * p.ldc + c + ch * 8, o);
            }
            __syncwarp();
          }
        }
        for (; c < ncols; c += 16) {
          tc::tmem_ld16(taddr + c, v);
          tc::tmem_ld_wait();
          if (p.epi == 1) {
            if (p.swapped) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                store_swiglu_swapped<TIN>(p, row, col0 + c + j, (ACC_STAGES == 1 && p.ssq_in != nullptr) ? v[j] * rs_s[min(c + j, uint32_t(TBM - 1))] : v[j]);
            } else if (row < p.M) {
              // 16 consecutive columns = 8 (gate, up) pairs of one row -> 8 outputs
              const uint32_t oc = (col0 + c) >> 1;
              if (!p.out_f32 && (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) && col0 + c + 16 <= p.N) {
                Vec16<TIN> o;
#pragma unroll
                for (int j = 0; j < 8; ++j) o.v[j] = ElemTraits<TIN>::from_f(silu_mul(v[2 * j], v[2 * j + 1]));
                st16(static_cast<TIN*>(p.C) + size_t(row) * p.ldc + oc, o);
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (col0 + c + 2 * j + 1 < p.N) {
                    const float r = silu_mul(v[2 * j], v[2 * j + 1]);
                    const size_t off = size_t(row) * p.ldc + oc + j;
                    if (p.out_f32) static_cast<float*>(p.C)[off] = r;
                    else static_cast<TIN*>(p.C)[off] = ElemTraits<TIN>::from_f(r);
                  }
                }
              }
            }
          } else if (c_vec && cin_vec && row < p.M && col0 + c + 16 <= p.N) {
            // 16 consecutive outputs of one row: two 16-byte stores, addend fetched the same way
            float add[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) add[j] = 0.f;
            if (p.Cin) {
              const TIN* src = static_cast<const TIN*>(p.Cin) + size_t(b) * p.stride_cin + size_t(row) * p.ldcin + col0 + c;
              const Vec16<TIN> a0 = ld16(src), a1 = ld16(src + 8);
#pragma unroll
              for (int j = 0; j < 8; ++j) { add[j] = p.beta * ElemTraits<TIN>::to_f(a0.v[j]); add[8 + j] = p.beta * ElemTraits<TIN>::to_f(a1.v[j]); }
            }
            TIN* dst = static_cast<TIN*>(p.C) + size_t(b) * p.stride_c + size_t(row) * p.ldc + col0 + c;
            Vec16<TIN> o0, o1;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              o0.v[j] = ElemTraits<TIN>::from_f(fmaf(p.alpha, v[j], add[j]));
              o1.v[j] = ElemTraits<TIN>::from_f(fmaf(p.alpha, v[8 + j], add[8 + j]));
            }
            st16(dst, o0);
            st16(dst + 8, o1);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) store_elem<TIN>(p, b, row, col0 + c + j, v[j]);
          }
        }
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&acc_empty[as]);
      } else {
        // split-K, or the push epilogue (one unit per CTA): park the fp32 partial in this CTA's shared memory, column-major.
        // The pipeline buffers are free: every MMA that read them has completed.
        float* red = reinterpret_cast<float*>(smem);
        for (uint32_t c = 0; c < ncols; c += 16) {
          tc::tmem_ld16(taddr + c, v);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) red[(c + j) * TBM + lane_in_tile] = v[j];
        }
        tc::tc_fence_before();
      }
    }
  }
  // ------------------------------ split-K reduction across the cluster ---------------------
  // The CTAs of a cluster hold the K-slices of one output tile.  After a cluster barrier each CTA
  // sums a share of the tile's columns over all slices, reading its peers' partials through
  // distributed shared memory in slice order (deterministic), and runs the epilogue on them.
  const bool parked = p.splits > 1 || p.n_ranks != 0 || p.ssq_out != nullptr;
  if (parked) {
    cg::cluster_group cluster = cg::this_cluster();
    // the producer and issuer lanes ran their loops alone: bring every warp back together first,
    // the cluster barrier instructions are warp-collective
    __syncwarp();
    if (threadIdx.x == 64) trace_stamp(p.trace, 5);              // partial parked in shared memory
    cluster.sync();
    if (threadIdx.x == 64) trace_stamp(p.trace, 6);              // all slices of the tile are parked
    if (warp >= 2 && warp < 6 && blockIdx.x < units) {
      const uint32_t quarter = warp & 3, lane_in_tile = quarter * 32 + lane;
      const uint32_t tile = blockIdx.x / p.splits, rank = blockIdx.x % p.splits;
      const uint32_t b = tile / tiles_per_batch, t = tile % tiles_per_batch;
      uint32_t tp, tq;
        tile_coords(p, t, tp, tq);
      const uint32_t col0 = tq * BN;
      const uint32_t ncols = min(uint32_t(BN), p.rowsQ > col0 ? p.rowsQ - col0 : 0u);
      float* red = reinterpret_cast<float*>(smem);
      (void)lane_in_tile;
      switch (p.splits) {
        case 1: reduce_tile<TIN, 1>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
        case 2: reduce_tile<TIN, 2>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
        case 3: reduce_tile<TIN, 3>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
        case 4: reduce_tile<TIN, 4>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
        case 5: reduce_tile<TIN, 5>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
        case 6: reduce_tile<TIN, 6>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
        case 7: reduce_tile<TIN, 7>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
        default: reduce_tile<TIN, 8>(p, cluster, red, rank, ncols, quarter, uint32_t(lane), b, tp, col0, push_off, push_epoch + 1u, p.ssq_in ? rs_s : nullptr); break;
      }
    }
    __syncwarp();
    if (threadIdx.x == 64) trace_stamp(p.trace, 7);              // this CTA's share of the tile reduced and stored
    // Nobody's shared memory may go away while a peer still reads it: arrive now (this CTA's remote reads
    // are done), wait at the very end, so that the teardown below overlaps the peers' last reads.
    cluster.barrier_arrive();
  }
  // ------------------------------ teardown ------------------------------------------------
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();                      // the allocator instructions want the whole warp converged
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (parked) {
    cg::this_cluster().barrier_wait();
    if (threadIdx.x == 64) trace_stamp(p.trace, 8);
  }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static std::once_flag g_encode_once;

bool encode_tmap_2byte(CUtensorMap* map, const void* base, uint32_t rank, const uint64_t* dims,
                       const uint64_t* strides_elems, const uint32_t* box) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (!g_encode) return false;
  cuuint64_t gdim[5], gstride[4];
  cuuint32_t gbox[5], estride[5];
  for (uint32_t i = 0; i < rank; ++i) { gdim[i] = dims[i]; gbox[i] = box[i]; estride[i] = 1; }
  for (uint32_t i = 1; i < rank; ++i) gstride[i - 1] = strides_elems[i] * 2;
  // bf16 and f16 move identically; the type only matters for OOB fill, which is zero
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim, gstride, gbox,
                        estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

unsigned int* tc_error_word_device() {
  // the symbol has one address per device; look it up once for each
  static std::atomic<unsigned int*> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  unsigned int* ptr = cache[dev & 63].load(std::memory_order_acquire);
  if (ptr) return ptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_tc_error) != cudaSuccess) return nullptr;
  cache[dev & 63].store(ptr, std::memory_order_release);
  return ptr;
}

bool gemm_tc_eligible(const GemmArgs& a) {
  if (a.dtype != KUIOPS_BF16 && a.dtype != KUIOPS_F16) return false;
  if (a.M == 0 || a.N == 0 || a.K == 0 || a.batch == 0) return false;
  if (!aligned16(a.A) || !aligned16(a.B)) return false;
  if (a.lda % 8 || a.ldb % 8) return false;
  if (a.batch > 1 && (a.stride_a % 8 || a.stride_b % 8)) return false;
  // tensor-map extents are 32-bit boxes over 64-bit dims; strides must stay below 2^40 bytes
  if (uint64_t(a.lda) * 2 >= (1ull << 40) || uint64_t(a.ldb) * 2 >= (1ull << 40)) return false;
  return true;
}

struct TcPlan { bool swapped; int bn; uint32_t tilesP, tilesQ, splits, kblocks, kb_per_split; };

// Pipeline depth of the swapped placement: chosen so that three CTAs (two for the 128-column
// tile) fit one SM; what keeps HBM busy is the number of resident CTAs, each with a few tiles in
// flight, not the depth of one CTA's ring.
constexpr uint32_t swapped_stages(int bn) { return bn <= 16 ? 4u : 3u; }

// ---- tuned plans ------------------------------------------------------------------------------
// A tuner (kuipy.tuner, behind KUIPY_RE_TUNE) times the alternatives of a shape and records the best
// here; make_plan consults the table before its own rule.  Keyed by (dtype, epilogue, transposed B,
// M, N, K); the value is the K split of the weight-streaming placement or the column tile of the
// normal one.
struct TunedPlan { int splits, bn; };
static std::mutex g_tuned_mu;
static std::unordered_map<std::string, TunedPlan> g_tuned;
static std::atomic<int> g_tuned_count{0};

static std::string tuned_key(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K) {
  char buf[96];
  snprintf(buf, sizeof buf, "%d/%d/%d/%u/%u/%u", dtype, epilogue, trans_b ? 1 : 0, M, N, K);
  return buf;
}

static bool tuned_lookup(const GemmArgs& a, TunedPlan* out) {
  if (g_tuned_count.load(std::memory_order_acquire) == 0 || a.batch != 1) return false;
  std::lock_guard<std::mutex> lock(g_tuned_mu);
  auto it = g_tuned.find(tuned_key(a.dtype, a.epilogue, a.trans_b, a.M, a.N, a.K));
  if (it == g_tuned.end()) return false;
  *out = it->second;
  return true;
}

static TcPlan make_plan(const GemmArgs& a) {
  TcPlan pl = {};
  pl.kblocks = (a.K + TBK - 1) / TBK;
  pl.swapped = a.M <= 128;
  TunedPlan tuned = {0, 0};
  const bool have_tuned = tuned_lookup(a, &tuned);
  if (pl.swapped) {
    pl.bn = a.M <= 16 ? 16 : (a.M <= 32 ? 32 : (a.M <= 64 ? 64 : 128));
    pl.tilesP = (a.N + TBM - 1) / TBM;
    pl.tilesQ = 1;
  } else {
    pl.bn = a.N > 128 ? 256 : 128;
    if (have_tuned && (tuned.bn == 128 || tuned.bn == 256)) pl.bn = tuned.bn;
    pl.tilesP = (a.M + TBM - 1) / TBM;
    pl.tilesQ = (a.N + pl.bn - 1) / pl.bn;
  }
  const uint64_t tiles = uint64_t(pl.tilesP) * pl.tilesQ * a.batch;
  pl.splits = 1;
  if (pl.swapped && have_tuned && tuned.splits >= 1 && tuned.splits <= 8 && uint32_t(tuned.splits) <= pl.kblocks) {
    pl.splits = uint32_t(tuned.splits);
    pl.kb_per_split = (pl.kblocks + pl.splits - 1) / pl.splits;
    pl.splits = (pl.kblocks + pl.kb_per_split - 1) / pl.kb_per_split;   // no empty slice
    return pl;
  }
  if (pl.swapped) {
    // Too few output tiles to occupy the machine: split K over the CTAs of a cluster (at most 8, the
    // portable cluster size).  Aim at as many CTAs as can be resident at once.
    const uint32_t smem_cta = swapped_stages(pl.bn) * (TBM * TBK * 2 + uint32_t(pl.bn) * TBK * 2) + 2048;
    uint32_t per_sm = (227u * 1024u) / smem_cta;
    if (per_sm > 3) per_sm = 3;
    if (per_sm < 1) per_sm = 1;
    const uint64_t resident = uint64_t(num_sms()) * per_sm;
    if (tiles < resident) {
      uint32_t want = uint32_t(resident / tiles);
      uint32_t cap = pl.kblocks / 4;               // keep at least 4 k-blocks (256 of K) per slice
      if (cap < 1) cap = 1;
      pl.splits = want < cap ? want : cap;
      if (pl.splits > 8) pl.splits = 8;
      if (pl.splits > 4 && pl.splits < 8) pl.splits = 4;   // clusters of 5..7 CTAs place badly on the GPCs (measured: 6 is far slower than 4 or 8)
      if (pl.splits < 1) pl.splits = 1;
    }
  }
  pl.kb_per_split = (pl.kblocks + pl.splits - 1) / pl.splits;
  pl.splits = (pl.kblocks + pl.kb_per_split - 1) / pl.kb_per_split;   // no empty slice
  if (pl.splits > 4 && pl.splits < 8) {
    pl.kb_per_split = (pl.kblocks + 3) / 4;
    pl.splits = (pl.kblocks + pl.kb_per_split - 1) / pl.kb_per_split;
  }
  return pl;
}

int gemm_tune_set(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K, int splits, int bn) {
  if (dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EUNSUPPORTED;
  if (M == 0 || N == 0 || K == 0 || epilogue < 0 || epilogue > 2) return KUIOPS_EINVAL;
  if (splits < 0 || splits > 8 || !(bn == 0 || bn == 128 || bn == 256)) return KUIOPS_EINVAL;
  std::lock_guard<std::mutex> lock(g_tuned_mu);
  const std::string key = tuned_key(dtype, epilogue, trans_b, M, N, K);
  if (splits == 0 && bn == 0) g_tuned.erase(key);
  else g_tuned[key] = TunedPlan{splits, bn};
  g_tuned_count.store(int(g_tuned.size()), std::memory_order_release);
  return KUIOPS_OK;
}

void gemm_tune_clear() {
  std::lock_guard<std::mutex> lock(g_tuned_mu);
  g_tuned.clear();
  g_tuned_count.store(0, std::memory_order_release);
}

int gemm_tune_query(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K, int* splits, int* bn, int* swapped) {
  if (M == 0 || N == 0 || K == 0) return KUIOPS_EINVAL;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = dtype; a.batch = 1; a.M = M; a.N = N; a.K = K; a.trans_b = trans_b; a.epilogue = epilogue;
  const TcPlan pl = make_plan(a);
  if (splits) *splits = int(pl.splits);
  if (bn) *bn = pl.bn;
  if (swapped) *swapped = pl.swapped ? 1 : 0;
  return KUIOPS_OK;
}

// The split-K partials live in shared memory, so the GEMM kernels need no global scratch; the
// query is kept for callers written against the workspace contract.
size_t gemm_tc_workspace_bytes(uint32_t, uint32_t, uint32_t, uint32_t) { return KUIOPS_GEMM_COUNTER_BYTES; }

template <typename TIN, int BN, int STAGES, int ACC_STAGES, bool P_MN, bool Q_MN>
static int launch_tc(const CUtensorMap& mp, const CUtensorMap& mq, const TcParams& p, unsigned grid, cudaStream_t st) {
  static_assert(size_t(BN) * TBM * sizeof(float) <= size_t(STAGES) * (TBM * TBK * 2 + BN * TBK * 2),
                "the split-K partial is parked in the pipeline buffers");
  // pipeline stages + alignment slack + barriers + (normal placement) the epilogue's staging blocks
  constexpr size_t smem = size_t(STAGES) * (TBM * TBK * 2 + BN * TBK * 2) + 1024 + 256 + (ACC_STAGES == 2 ? 32768 : 512);
  static_assert(smem <= 227 * 1024, "shared memory budget of one CTA");
  auto kern = gemm_tc_kernel<TIN, BN, STAGES, ACC_STAGES, P_MN, Q_MN>;
  // the opt-in for large dynamic shared memory is per device: do it once per (kernel, device)
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return KUIOPS_ELAUNCH;
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return KUIOPS_ELAUNCH;
    configured.fetch_or(bit, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(ACC_STAGES == 2 ? kTcThreadsWide : kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled.load(std::memory_order_relaxed) ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mp, mq, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return e == cudaSuccess ? KUIOPS_OK : KUIOPS_ELAUNCH;
}

template <typename TIN>
static int gemm_tc_typed(const GemmArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const TcPlan pl = make_plan(a);
  (void)workspace; (void)workspace_bytes;
  // Tensor maps.  "Rows" of an operand are the index that is NOT K.
  // A is always K-major: dims (K, M, batch).  B is K-major when trans_b (stored [N, K]) and
  // MN-major otherwise (stored [K, N]: dims (N, K, batch)).
  CUtensorMap mapA, mapB;
  const uint32_t a_box_rows = pl.swapped ? uint32_t(pl.bn) : uint32_t(TBM);
  {
    const uint64_t dims[3] = {a.K, a.M, a.batch};
    const uint64_t strides[3] = {1, uint64_t(a.lda), uint64_t(a.batch > 1 ? a.stride_a : int64_t(a.lda) * a.M)};
    const uint32_t box[3] = {TBK, a_box_rows, 1};
    if (!encode_tmap_2byte(&mapA, a.A, 3, dims, strides, box)) return KUIOPS_EDRIVER;
  }
  const uint32_t b_box_rows = pl.swapped ? uint32_t(TBM) : uint32_t(pl.bn);
  if (a.trans_b) {
    const uint64_t dims[3] = {a.K, a.N, a.batch};
    const uint64_t strides[3] = {1, uint64_t(a.ldb), uint64_t(a.batch > 1 ? a.stride_b : int64_t(a.ldb) * a.N)};
    const uint32_t box[3] = {TBK, b_box_rows, 1};
    if (!encode_tmap_2byte(&mapB, a.B, 3, dims, strides, box)) return KUIOPS_EDRIVER;
  } else {
    const uint64_t dims[3] = {a.N, a.K, a.batch};
    const uint64_t strides[3] = {1, uint64_t(a.ldb), uint64_t(a.batch > 1 ? a.stride_b : int64_t(a.ldb) * a.K)};
    const uint32_t box[3] = {64, TBK, 1};
    if (!encode_tmap_2byte(&mapB, a.B, 3, dims, strides, box)) return KUIOPS_EDRIVER;
  }
  TcParams p = {};
  p.K = a.K; p.batch = a.batch;
  p.bandP = pl.tilesP < 32 ? pl.tilesP : 32;
  p.tilesP = pl.tilesP; p.tilesQ = pl.tilesQ; p.splits = pl.splits; p.kblocks = pl.kblocks; p.kb_per_split = pl.kb_per_split;
  p.swapped = pl.swapped ? 1 : 0; p.out_f32 = a.out_dtype == KUIOPS_F32 ? 1 : 0; p.epi = a.epilogue;
  p.M = a.M; p.N = a.N;
  p.rowsP = pl.swapped ? a.N : a.M; p.rowsQ = pl.swapped ? a.M : a.N;
  p.alpha = a.alpha; p.beta = a.beta;
  p.Cin = a.Cin; p.ldcin = a.ldcin; p.stride_cin = a.stride_cin;
  p.C = a.C; p.ldc = a.ldc; p.stride_c = a.stride_c;
  p.err = tc_error_word_device();
  if (!p.err) return KUIOPS_ELAUNCH;
  p.trace = g_gemm_trace.load(std::memory_order_relaxed);
  if (a.ssq_out || a.ssq_in) {
    // both halves of the folded norm live in the weight-streaming placement, one row factor per MMA column
    if (!pl.swapped || a.batch != 1 || (a.ssq_out && a.epilogue != 0) || (a.ssq_in && a.ssq_tiles == 0)) return KUIOPS_EUNSUPPORTED;
    p.ssq_out = a.ssq_out; p.ssq_in = a.ssq_in; p.ssq_tiles = a.ssq_tiles; p.ssq_eps = a.ssq_eps;
  }
  if (a.epilogue == 2) {
    // needs the swapped placement with K split (the partner feature is read from the parked partials)
    if (!pl.swapped || pl.splits < 2 || a.batch != 1 || !a.rope || a.out_dtype != a.dtype) return KUIOPS_EUNSUPPORTED;
    p.positions = reinterpret_cast<const long long*>(a.rope->positions); p.log2_theta = log2f(a.rope->theta);
    p.k_cache = a.rope->k_cache; p.v_cache = a.rope->v_cache; p.cache_cap = a.rope->cache_cap;
    p.hq = a.rope->hq; p.hk = a.rope->hk; p.rows_per_seq = a.rope->rows_per_seq ? a.rope->rows_per_seq : 1u;
  }
  if (a.push) {
    if (!pl.swapped || a.epilogue != 0 || a.batch != 1 || a.N % 4) return KUIOPS_EUNSUPPORTED;
    p.n_ranks = a.push->n_ranks; p.my_rank = a.push->rank;
    for (uint32_t r = 0; r < p.n_ranks; ++r) p.peer_base[r] = a.push->peer_base[r];
    p.slot_bytes = a.push->slot_bytes;
    p.epoch = a.push->epoch;
  }
  const uint64_t units = uint64_t(pl.tilesP) * pl.tilesQ * a.batch * pl.splits;
  if (units >= (1ull << 31)) return KUIOPS_EUNSUPPORTED;
  const bool b_mn = !a.trans_b;
  if (pl.swapped) {
    // one unit per CTA so several small CTAs share an SM and keep more loads in flight
    const unsigned grid = unsigned(units);
    const CUtensorMap& mp = mapB; const CUtensorMap& mq = mapA;
#define KUIOPS_SW(BNV)                                                                             \
  case BNV: return b_mn ? launch_tc<TIN, BNV, int(swapped_stages(BNV)), 1, true, false>(mp, mq, p, grid, st)   \
                        : launch_tc<TIN, BNV, int(swapped_stages(BNV)), 1, false, false>(mp, mq, p, grid, st);
    switch (pl.bn) { KUIOPS_SW(16) KUIOPS_SW(32) KUIOPS_SW(64) KUIOPS_SW(128) }
#undef KUIOPS_SW
    return KUIOPS_EUNSUPPORTED;
  }
  // persistent CTAs, one per SM, minus the SMs the caller asked to keep free for a kernel of another stream
  const int reserve = g_gemm_sm_reserve.load(std::memory_order_relaxed);
  const uint64_t sms = uint64_t(num_sms() - reserve > 1 ? num_sms() - reserve : 1);
  const unsigned grid = unsigned(units < sms ? units : sms);
  if (pl.bn == 256)
    return b_mn ? launch_tc<TIN, 256, 4, 2, false, true>(mapA, mapB, p, grid, st)
                : launch_tc<TIN, 256, 4, 2, false, false>(mapA, mapB, p, grid, st);
  return b_mn ? launch_tc<TIN, 128, 6, 2, false, true>(mapA, mapB, p, grid, st)
              : launch_tc<TIN, 128, 6, 2, false, false>(mapA, mapB, p, grid, st);
}

int gemm_tc(const GemmArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!gemm_tc_eligible(a)) return KUIOPS_EUNSUPPORTED;
  if (a.dtype == KUIOPS_BF16) return gemm_tc_typed<__nv_bfloat16>(a, workspace, workspace_bytes, st);
  return gemm_tc_typed<__half>(a, workspace, workspace_bytes, st);
}

}  // namespace kuiops
