// Split-KV attention on tcgen05 for decode: a few query tokens per sequence against a long KV
// cache (bf16 / f16, head dim 128, grouped-query heads, optional device-side key counts).
//
// HBM bound: every K/V byte is read once per GQA group.  A CTA owns one (batch, KV head) and one
// slice of the keys.  The query rows of the whole group - G heads x l positions, at most 128 -
// are loaded as ONE TMA box into the first rows of a 128-row UMMA tile, so the G heads share
// each K/V tile; the remaining rows of the tile are zero and ignored.  The pipeline is the one
// of the prefill kernel (TMA ring of 64-key tiles -> S = Q K^T in TMEM -> online softmax in
// registers -> P to shared memory -> O += P V in TMEM).  With more than one slice per (batch, KV
// head) each CTA parks its (max, sum, unnormalised O) record in the workspace and the CTA that
// draws the last ticket of the unit merges the records in slice order and writes the output.
// Replaces the lane-per-key SIMT kernel for these shapes; the reference has no counterpart
// (its only attention kernel is the naive biased one, kuiops/sdpa/Kuiops.Sdpa.fst.1).
#include "sdpa.cuh"
#include "gemm.cuh"
#include "tc_ptx.cuh"
#include <type_traits>

namespace kuiops {

constexpr int DBM = 128;      // UMMA tile rows (TMEM lanes); only the first G*l carry queries
constexpr int DBN = 64;       // keys per tile
constexpr int DD = 128;       // head dim
constexpr int kDecThreads = 192;
constexpr uint32_t D_Q_BYTES = DBM * DD * 2;
constexpr uint32_t D_K_BYTES = DBN * DD * 2;
constexpr uint32_t D_V_BYTES = DBN * DD * 2;
constexpr uint32_t D_P_BYTES = DBM * DBN * 2;
constexpr uint32_t D_SMEM = D_Q_BYTES + 2 * (D_K_BYTES + D_V_BYTES) + D_P_BYTES;   // 112 KB: two CTAs per SM
constexpr uint32_t D_BAR_BYTES = 160;      // 16 mbarriers, the TMEM slot word and the merge flag behind the tiles
constexpr uint32_t D_TMEM_COLS = 256;
constexpr float kDecRescale = 8.0f;
constexpr int D_REC = DD + 4;  // floats per parked row: 128 accumulators, max, sum, 2 pad (keeps rows 16-byte aligned)

struct DecParams {
  uint32_t n, h, h_kv, l, s, G, rows, splits;
  float scale_log2;
  int is_causal;
  const int64_t* kv_lens;
  void* out; int64_t o_sn, o_sh, o_sl;
  float* lse;
  float* partials; int* counters;
  unsigned int* err;
  unsigned long long* trace;          // debug: CTA 0 stamps the stations of its critical path (kuiops_debug_gemm_trace, slots 16..23)
};

__device__ __forceinline__ uint64_t dec_global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void dec_stamp(unsigned long long* t, int slot) {
  if (t != nullptr && blockIdx.x == 0) t[slot] = dec_global_ns();
}
__device__ __forceinline__ bool dec_wait(uint64_t* bar, uint32_t parity) {
  if (tc::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = dec_global_ns();
  while (!tc::mbar_try_wait(bar, parity)) {
    if (dec_global_ns() - t0 > 2000000000ull) return false;
  }
  return true;
}

// SMALL (at most 8 query rows, e.g. 4 GQA heads x 1 token): the Q and P operands keep a single
// 8-row core-matrix group in shared memory and their descriptors use a zero stride between row
// groups, so all 16 groups of the 128-row UMMA tile read the same 1 KB (TMEM lanes 8..127 then
// hold copies of lanes 0..7 and are ignored).  The 46 KB this frees go to a third K/V ring slot.
template <typename T, bool SMALL>
__global__ void __launch_bounds__(kDecThreads, 2)
sdpa_decode_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const DecParams p) {
  // The 128-byte swizzle atoms need a 1024-byte aligned base.  The dynamic shared window of a
  // kernel without static shared memory starts on such a boundary; there is no room for padding
  // (two CTAs must fit one SM), so a misaligned base is reported instead of worked around.
  extern __shared__ __align__(1024) unsigned char smem[];
  if ((tc::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.err, 0u, 10u);
    return;
  }
  constexpr uint32_t NSLOT = SMALL ? 3 : 2;                    // K/V ring depth
  constexpr uint32_t Q_HALF = SMALL ? 1024u : uint32_t(DBM) * 128u;   // bytes of one 64-column half of Q
  constexpr uint32_t Q_BYTES = 2 * Q_HALF;
  constexpr uint32_t P_BYTES = SMALL ? 1024u : D_P_BYTES;
  // SMALL: two P buffers, so that the softmax of tile j + 1 does not wait for the P V product of tile j
  // (with one buffer a tile costs a softmax plus an MMA round trip; the large form has no room for a second)
  constexpr uint32_t PBUF = SMALL ? 2u : 1u;
  constexpr uint32_t ROW_GROUP_STRIDE = SMALL ? 0u : 1024u;      // SBO of the Q and P descriptors
  unsigned char* q_s = smem;
  unsigned char* kv_s = q_s + Q_BYTES;                         // slot i: K at kv_s + i*32K, V right after K
  unsigned char* p_s = kv_s + NSLOT * (D_K_BYTES + D_V_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + PBUF * P_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // NSLOT (room for 3)
  uint64_t* v_full = bars + 4;      // NSLOT
  uint64_t* kv_empty = bars + 7;    // NSLOT
  uint64_t* s_full = bars + 10;     // 2: S is double buffered so that Q K^T of the next tile overlaps this tile's softmax
  // One barrier per P buffer.  A waiter must never fall two phases behind its barrier (the parity test cannot
  // tell "not yet" from "twice since"): with two P buffers the softmax of tile j + 1 does not depend on the
  // issuer having seen tile j's arrival, so both arrivals on ONE barrier could pass between two polls of the
  // issuer.  On p_ready[j & 1] the next phase (tile j + 2) needs scores that are only issued after the issuer
  // has seen tile j.
  uint64_t* p_ready = bars + 12;    // PBUF (room for 2): P of tile j arrives on p_ready[j % PBUF]
  uint64_t* o_done = bars + 14;     // 2: P V of tile j arrives on o_done[j & 1] (SMALL) or o_done[0] (one P buffer)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) dec_stamp(p.trace, 16);                 // CTA started
  // unit = (batch, KV head); blockIdx.x = unit * splits + split
  const uint32_t split = blockIdx.x % p.splits;
  const uint32_t unit = blockIdx.x / p.splits;
  const uint32_t kvh = unit % p.h_kv;
  const uint32_t b = unit / p.h_kv;
  // rows of the tile that carry no query must not feed NaN bit patterns into the MMA
  for (uint32_t i = threadIdx.x; i < Q_BYTES / 16; i += blockDim.x) reinterpret_cast<int4*>(q_s)[i] = make_int4(0, 0, 0, 0);
  tc::fence_proxy_async();

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    for (uint32_t i = 0; i < NSLOT; ++i) { tc::mbar_init(&k_full[i], 1); tc::mbar_init(&v_full[i], 1); tc::mbar_init(&kv_empty[i], 1); }
    tc::mbar_init(&s_full[0], 1);
    tc::mbar_init(&s_full[1], 1);
    // SMALL: only the warp that holds the (at most 8) query rows takes part in the tile loop.  With two P
    // buffers a warp is no longer held back by the previous tile's product, so a warp without rows could run
    // ahead and its arrival for tile j + 1 would be counted for tile j; the others skip the loop instead.
    tc::mbar_init(&p_ready[0], SMALL ? 1 : 4);
    tc::mbar_init(&p_ready[1], SMALL ? 1 : 4);
    tc::mbar_init(&o_done[0], 1);
    tc::mbar_init(&o_done[1], 1);
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmQ); tc::prefetch_tmap(&tmK); tc::prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, D_TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128;
  pdl_wait();          // Q, the cache and the key counts may still be being written by earlier kernels
  pdl_trigger();
  if (threadIdx.x == 0) dec_stamp(p.trace, 17);                 // predecessor complete
  // keys of this batch entry, optionally counted on the device
  uint32_t S = p.s;
  if (p.kv_lens) {
    const long long kl = p.kv_lens[b];
    S = kl < 0 ? 0u : (kl < (long long)p.s ? uint32_t(kl) : p.s);
  }
  // this CTA's slice of the keys, in whole tiles
  const uint32_t tiles_total = (S + DBN - 1) / DBN;
  const uint32_t tiles_per = (tiles_total + p.splits - 1) / p.splits;
  const uint32_t s_lo = min(split * tiles_per * DBN, S);
  const uint32_t s_hi = min(s_lo + tiles_per * DBN, S);
  const uint32_t n_tiles = (s_hi - s_lo + DBN - 1) / DBN;


  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      tc::mbar_expect_tx(q_full, 2u * p.rows * 128u);
      tc::tma_load_4d(q_s, &tmQ, q_full, 0, 0, int(kvh * p.G), int(b));
      tc::tma_load_4d(q_s + Q_HALF, &tmQ, q_full, 64, 0, int(kvh * p.G), int(b));
      for (uint32_t j = 0; j < n_tiles; ++j) {
        const uint32_t slot = j % NSLOT, ph = (j / NSLOT) & 1;
        if (!dec_wait(&kv_empty[slot], ph ^ 1)) { atomicCAS(p.err, 0u, 11u); break; }
        unsigned char* ks = kv_s + slot * (D_K_BYTES + D_V_BYTES);
        unsigned char* vs = ks + D_K_BYTES;
        const int key0 = int(s_lo + j * DBN);
        tc::mbar_expect_tx(&k_full[slot], D_K_BYTES);
        tc::tma_load_4d(ks, &tmK, &k_full[slot], 0, key0, int(kvh), int(b));
        tc::tma_load_4d(ks + DBN * 128, &tmK, &k_full[slot], 64, key0, int(kvh), int(b));
        tc::mbar_expect_tx(&v_full[slot], D_V_BYTES);
        tc::tma_load_4d(vs, &tmV, &v_full[slot], 0, key0, int(kvh), int(b));
        tc::tma_load_4d(vs + DBN * 128, &tmV, &v_full[slot], 64, key0, int(kvh), int(b));
      }
    }
  } else if (warp == 1) {
    // ------------------------------ UMMA issuer -------------------------------------------
    if (lane == 0) {
      constexpr int is_bf16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_qk = tc::make_idesc(is_bf16, 0, 0, DBM, DBN);
      constexpr uint32_t idesc_pv = tc::make_idesc(is_bf16, 0, 1, DBM, DD);
      bool ok = dec_wait(q_full, 0);
      if (!ok) atomicCAS(p.err, 0u, 12u);
      const uint32_t qa = tc::smem_u32(q_s), pa = tc::smem_u32(p_s);
      // S = Q K^T of tile j into S buffer j & 1: two 64-wide halves of the head dim x four 16-wide steps
      auto issue_qk = [&](uint32_t j) -> bool {
        const uint32_t slot = j % NSLOT, ph = (j / NSLOT) & 1, sbuf = j & 1;
        const uint32_t ka = tc::smem_u32(kv_s + slot * (D_K_BYTES + D_V_BYTES));
        if (!dec_wait(&k_full[slot], ph)) { atomicCAS(p.err, 0u, 13u); return false; }
        tc::tc_fence_after();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t da = tc::make_smem_desc(qa + hh * Q_HALF + kk * 32, 16, ROW_GROUP_STRIDE);
            const uint64_t db = tc::make_smem_desc(ka + hh * (DBN * 128) + kk * 32, 16, 1024);
            tc::umma_f16(tmem_S + sbuf * DBN, da, db, idesc_qk, (hh | kk) ? 1u : 0u);
          }
        tc::umma_commit(&s_full[sbuf]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_qk(0);
      for (uint32_t j = 0; j < n_tiles && ok; ++j) {
        const uint32_t slot = j % NSLOT, ph = (j / NSLOT) & 1;
        const uint32_t va = tc::smem_u32(kv_s + slot * (D_K_BYTES + D_V_BYTES)) + D_K_BYTES;
        // the next tile's scores are computed while the softmax warps work on this one; their S
        // buffer was released when p_ready of tile j - 1 arrived
        if (j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
        if (!dec_wait(&p_ready[j % PBUF], (j / PBUF) & 1)) { atomicCAS(p.err, 0u, 14u); ok = false; break; }
        if (!dec_wait(&v_full[slot], ph)) { atomicCAS(p.err, 0u, 15u); ok = false; break; }
        tc::tc_fence_after();
        // O += P V over the 64 keys of the tile: four 16-key steps; V is MN-major (head dim contiguous)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t da = tc::make_smem_desc(pa + (j % PBUF) * P_BYTES + kk * 32, 16, ROW_GROUP_STRIDE);
          const uint64_t db = tc::make_smem_desc(va + kk * 2048, DBN * 128, 1024);
          tc::umma_f16(tmem_O, da, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc::umma_commit(&kv_empty[slot]);
        tc::umma_commit(&o_done[j % PBUF]);
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------------------
    const uint32_t quarter = warp & 3;
    const uint32_t r = quarter * 32 + lane;               // row of the tile: (head in group, position)
    const uint32_t g = r / p.l, li = r % p.l;
    const bool row_valid = r < p.rows;
    const bool warp_active = quarter * 32 < p.rows;       // warps without a query row only keep the barriers in step
    const uint32_t head = kvh * p.G + g;
    const uint32_t lane_addr = (quarter * 32) << 16;
    const uint32_t epi_tid = threadIdx.x - 64;
    // last key this row may see (inclusive, bottom-right aligned causal mask), capped to this slice
    int64_t row_lim = p.is_causal ? int64_t(li) + int64_t(S) - int64_t(p.l) : int64_t(S) - 1;
    if (row_lim > int64_t(s_hi) - 1) row_lim = int64_t(s_hi) - 1;
    if (!row_valid) row_lim = -1;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    const bool in_loop = !SMALL || warp_active;
    for (uint32_t j = 0; j < n_tiles && ok && in_loop; ++j) {
      if (!dec_wait(&s_full[j & 1], (j >> 1) & 1)) { atomicCAS(p.err, 0u, 16u); ok = false; break; }
      if (j == 0 && (warp & 3) == 0 && lane == 0) dec_stamp(p.trace, 18);       // first scores ready (Q, K landed, first MMA done)
      tc::tc_fence_after();
      float sv[DBN];
      float corr = 1.f;
      if (warp_active) {
        tc::tmem_ld32(tmem_S + (j & 1) * DBN + lane_addr, sv);
        tc::tmem_ld32(tmem_S + (j & 1) * DBN + lane_addr + 32, sv + 32);
        tc::tmem_ld_wait();
        const int64_t key0 = int64_t(s_lo) + int64_t(j) * DBN;
        const bool edge = key0 + DBN - 1 > row_lim;
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < DBN; ++c) {
          if (edge && key0 + c > row_lim) sv[c] = -INFINITY;
          mx = fmaxf(mx, sv[c]);
        }
        mx *= p.scale_log2;                       // scale > 0: the max commutes with the scaling
        if (mx > m_used + kDecRescale || m_used == -INFINITY) {
          const float m_new = fmaxf(mx, m_used);
          // a row that has not seen a key yet has nothing accumulated: no rescale (a factor other than 1 would make
          // the whole warp wait for the previous product for nothing)
          corr = (m_used == -INFINITY) ? ((m_new == -INFINITY || j == 0) ? 1.f : 0.f) : exp2f(m_used - m_new);
          m_used = m_new;
        }
        const float mm = (m_used == -INFINITY) ? 0.f : m_used;
        float rs = 0.f;
#pragma unroll
        for (int c = 0; c < DBN; ++c) { sv[c] = exp2f(fmaf(sv[c], p.scale_log2, -mm)); rs += sv[c]; }
        l_run = l_run * corr + rs;
      }
      // O may only be rescaled once every earlier P V product has landed in it, and the P buffer of this
      // tile may only be overwritten once the product that read it last (tile j - PBUF) has completed.
      // One buffer: both are "tile j - 1 done".  Two buffers: the rescale (rare after the first tiles, the
      // running maximum is only raised by steps of 2^8) waits for tile j - 1, everything else for tile j - 2.
      const bool rescale = warp_active && __any_sync(0xffffffffu, corr != 1.f);
      if (PBUF == 1) {
        if (j > 0) {
          if (!dec_wait(&o_done[0], (j - 1) & 1)) { atomicCAS(p.err, 0u, 17u); ok = false; break; }
          tc::tc_fence_after();
        }
      } else {
        if (j > 1) {
          if (!dec_wait(&o_done[j & 1], ((j >> 1) - 1) & 1)) { atomicCAS(p.err, 0u, 17u); ok = false; break; }
          tc::tc_fence_after();
        }
        if (j > 0 && rescale) {
          if (!dec_wait(&o_done[(j - 1) & 1], ((j - 1) >> 1) & 1)) { atomicCAS(p.err, 0u, 19u); ok = false; break; }
          tc::tc_fence_after();
        }
      }
      if (j > 0) {
        if (rescale) {
#pragma unroll
          for (int c0 = 0; c0 < DD; c0 += 32) {
            float ov[32];
            tc::tmem_ld32(tmem_O + lane_addr + c0, ov);
            tc::tmem_ld_wait();
            uint32_t ou[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) ou[c] = __float_as_uint(ov[c] * corr);
            tc::tmem_st32(tmem_O + lane_addr + c0, ou);
          }
          tc::tmem_st_wait();
        }
      }
      if (warp_active && (!SMALL || r < 8)) {
        unsigned char* prow = p_s + (j % PBUF) * P_BYTES + (SMALL ? 0u : (r >> 3) * 1024) + (r & 7) * 128;
#pragma unroll
        for (int c = 0; c < DBN / 8; ++c) {
          uint4 pk;
          pk.x = row_valid ? pack2<T>(sv[c * 8 + 0], sv[c * 8 + 1]) : 0u;
          pk.y = row_valid ? pack2<T>(sv[c * 8 + 2], sv[c * 8 + 3]) : 0u;
          pk.z = row_valid ? pack2<T>(sv[c * 8 + 4], sv[c * 8 + 5]) : 0u;
          pk.w = row_valid ? pack2<T>(sv[c * 8 + 6], sv[c * 8 + 7]) : 0u;
          *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = pk;
        }
      } else if (j == 0 && !SMALL) {
        // rows that never carry a query: one zero fill keeps the P operand free of stale bit patterns
        unsigned char* prow = p_s + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int c = 0; c < DBN / 8; ++c) *reinterpret_cast<int4*>(prow + (c << 4)) = make_int4(0, 0, 0, 0);
      }
      tc::fence_proxy_async();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&p_ready[j % PBUF]);
    }
    if (ok && n_tiles > 0 && in_loop) {
      // products complete in issue order: the last one's arrival covers them all
      const uint32_t jl = n_tiles - 1;
      const bool done = PBUF == 1 ? dec_wait(&o_done[0], jl & 1) : dec_wait(&o_done[jl & 1], (jl >> 1) & 1);
      if (!done) { atomicCAS(p.err, 0u, 18u); ok = false; }
    }
    tc::tc_fence_after();
    if ((warp & 3) == 0 && lane == 0) dec_stamp(p.trace, 19);    // every tile of this slice accumulated (the warp that holds row 0)
    if (p.splits == 1) {
      if (ok && warp_active) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        T* orow = static_cast<T*>(p.out) + size_t(b) * p.o_sn + size_t(head) * p.o_sh + size_t(li) * p.o_sl;
#pragma unroll
        for (int c0 = 0; c0 < DD; c0 += 32) {
          float ov[32];
          if (n_tiles > 0) {
            tc::tmem_ld32(tmem_O + lane_addr + c0, ov);
            tc::tmem_ld_wait();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) ov[c] = 0.f;
          }
          if (row_valid) {
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              Vec16<T> o;
#pragma unroll
              for (int e = 0; e < 8; ++e) o.v[e] = ElemTraits<T>::from_f(ov[c + e] * inv);
              st16(orow + c0 + c, o);
            }
          }
        }
        if (p.lse && row_valid)
          p.lse[(size_t(b) * p.h + head) * p.l + li] = l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
    } else {
      // park this slice's record, then the last slice of the unit to arrive merges them all
      float* rec = p.partials + ((size_t(unit) * p.splits + split) * p.rows + r) * D_REC;
      if (warp_active) {
#pragma unroll
        for (int c0 = 0; c0 < DD; c0 += 32) {
          float ov[32];
          if (ok && n_tiles > 0) {
            tc::tmem_ld32(tmem_O + lane_addr + c0, ov);
            tc::tmem_ld_wait();
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) ov[c] = 0.f;
          }
          if (row_valid) {
#pragma unroll
            for (int c = 0; c < 32; c += 4) __stcg(reinterpret_cast<float4*>(rec + c0 + c), make_float4(ov[c], ov[c + 1], ov[c + 2], ov[c + 3]));
          }
        }
        if (row_valid) { __stcg(rec + DD, m_used); __stcg(rec + DD + 1, l_run); }
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (epi_tid == 0) {
        const int old = atomicAdd(&p.counters[unit], 1);
        *last_flag = (old == int(p.splits) - 1) ? 1 : 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (epi_tid == 0) dec_stamp(p.trace, 20);                 // record parked, ticket drawn
      if (*last_flag) {
        __threadfence();
        // The four epilogue warps take the rows in turn (row rr goes to warp rr mod 4), a lane four columns of a
        // row: the rows of a unit are merged side by side instead of one after another, every slice's record is
        // fetched with one 16-byte load per lane, and the loads of several slices are in flight together.  The
        // slices are still added in slice order, so the result does not depend on which slice arrived last.
        const uint32_t wq = epi_tid >> 5, ln = epi_tid & 31;
        const float* base = p.partials + size_t(unit) * p.splits * p.rows * D_REC;
        for (uint32_t rr = wq; rr < p.rows; rr += 4) {
          float mm = -INFINITY;
          for (uint32_t s2 = ln; s2 < p.splits; s2 += 32) mm = fmaxf(mm, __ldcg(base + (size_t(s2) * p.rows + rr) * D_REC + DD));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
          float acc[4] = {0.f, 0.f, 0.f, 0.f}, den = 0.f;
#pragma unroll 4
          for (uint32_t s2 = 0; s2 < p.splits; ++s2) {
            const float* rc = base + (size_t(s2) * p.rows + rr) * D_REC;
            const float mw = __ldcg(rc + DD);
            const float lw = __ldcg(rc + DD + 1);
            const float4 x = __ldcg(reinterpret_cast<const float4*>(rc + ln * 4));
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
            acc[0] += f * x.x; acc[1] += f * x.y; acc[2] += f * x.z; acc[3] += f * x.w;
            den += f * lw;
          }
          const uint32_t hh = kvh * p.G + rr / p.l, ll = rr % p.l;
          T* orow = static_cast<T*>(p.out) + size_t(b) * p.o_sn + size_t(hh) * p.o_sh + size_t(ll) * p.o_sl + ln * 4;
          // (o_sl, o_sh, o_sn are multiples of 8 elements and the base is 16-byte aligned: an 8-byte store is aligned)
          *reinterpret_cast<uint2*>(orow) = make_uint2(pack2<T>(den > 0.f ? acc[0] / den : 0.f, den > 0.f ? acc[1] / den : 0.f),
                                                       pack2<T>(den > 0.f ? acc[2] / den : 0.f, den > 0.f ? acc[3] / den : 0.f));
          if (p.lse && ln == 0)
            p.lse[(size_t(b) * p.h + hh) * p.l + ll] = den > 0.f ? (mm + log2f(den)) * 0.6931471805599453f : -INFINITY;
        }
        if (epi_tid == 0) p.counters[unit] = 0;
        if (epi_tid == 0 && p.trace != nullptr) p.trace[21] = dec_global_ns();     // merged (whichever CTA was last; unit 0 only when CTA 0's)
      }
    }
    if (epi_tid == 0) dec_stamp(p.trace, 22);                   // epilogue done
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, D_TMEM_COLS);
  }
}


bool sdpa_decode_tc_eligible(const SdpaArgs& a) {
  if (a.dtype != KUIOPS_BF16 && a.dtype != KUIOPS_F16) return false;
  if (!(a.scale > 0.f)) return false;               // the softmax takes the row max before scaling
  if (a.e != DD || a.ev != DD || a.bias != nullptr) return false;
  const uint32_t G = a.h / a.h_kv;
  if (a.l > 16 || uint64_t(G) * a.l > uint64_t(DBM) || G > 128) return false;
  auto ok_stride = [](int64_t s) { return s > 0 && s % 8 == 0 && uint64_t(s) * 2 < (1ull << 40); };
  if (!ok_stride(a.k_ss) || !ok_stride(a.v_ss) || a.o_sl % 8) return false;
  if (a.l > 1 && !ok_stride(a.q_sl)) return false;
  if (a.h > 1 && (!ok_stride(a.q_sh) || a.o_sh % 8)) return false;
  if (a.h_kv > 1 && (!ok_stride(a.k_sh) || !ok_stride(a.v_sh))) return false;
  if (a.n > 1 && (!ok_stride(a.q_sn) || !ok_stride(a.k_sn) || !ok_stride(a.v_sn) || a.o_sn % 8)) return false;
  if (!aligned16(a.Q) || !aligned16(a.K) || !aligned16(a.V) || !aligned16(a.out)) return false;
  return uint64_t(a.n) * a.h_kv * 64 < (1ull << 31);
}

// Debug override of the split count (0 = the rule below); see kuiops_debug_sdpa_splits.
std::atomic<int> g_sdpa_splits_override{0};

static uint32_t decode_tc_splits(const SdpaArgs& a) {
  const uint64_t units = uint64_t(a.n) * a.h_kv;
  const int forced = g_sdpa_splits_override.load(std::memory_order_relaxed);
  if (forced > 0) {
    const uint32_t tiles = (a.s + DBN - 1) / DBN;
    const uint32_t f = uint32_t(forced) < tiles ? uint32_t(forced) : (tiles ? tiles : 1u);
    return f > 64 ? 64 : f;
  }
  const uint64_t resident = 2 * uint64_t(num_sms());          // two CTAs per SM
  if (units >= resident) return 1;
  uint32_t want = uint32_t(resident / units);               // whole waves only: a partial second wave costs a full one
  uint32_t cap = a.s / (4 * DBN);                           // at least four key tiles per slice
  if (cap < 1) cap = 1;
  uint32_t splits = want < cap ? want : cap;
  return splits > 64 ? 64 : splits;
}

size_t sdpa_decode_tc_workspace_bytes(const SdpaArgs& a) {
  const uint32_t splits = decode_tc_splits(a);
  if (splits == 1) return 0;
  const uint64_t units = uint64_t(a.n) * a.h_kv;
  const uint32_t rows = (a.h / a.h_kv) * a.l;
  return ((units * 4 + 255) & ~size_t(255)) + size_t(units) * splits * rows * D_REC * sizeof(float);
}

size_t sdpa_decode_tc_counter_bytes(const SdpaArgs& a) {
  return decode_tc_splits(a) == 1 ? 0 : ((uint64_t(a.n) * a.h_kv * 4 + 255) & ~size_t(255));
}

template <typename T, bool SMALL>
static int decode_tc_launch_variant(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const DecParams& p,
                                    unsigned grid, size_t smem, cudaStream_t st) {
  auto kern = sdpa_decode_tc_kernel<T, SMALL>;
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return KUIOPS_ELAUNCH;
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return KUIOPS_ELAUNCH;
    configured.fetch_or(bit, std::memory_order_release);
  }
  return launch_pdl(kern, dim3(grid), dim3(kDecThreads), smem, st, mq, mk, mv, p);
}

template <typename T>
static int decode_tc_launch(const SdpaArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const uint32_t G = a.h / a.h_kv;
  DecParams p = {};
  p.splits = decode_tc_splits(a);
  if (p.splits > 1) {
    if (!workspace || workspace_bytes < sdpa_decode_tc_workspace_bytes(a)) {
      p.splits = 1;                 // no scratch: one CTA walks all keys of its (batch, KV head)
    } else {
      p.counters = static_cast<int*>(workspace);
      p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + ((uint64_t(a.n) * a.h_kv * 4 + 255) & ~size_t(255)));
    }
  }
  CUtensorMap mq, mk, mv;
  {
    // Q: (d, l, h, n); one box takes the l positions of the G heads of a group
    const uint64_t dims[4] = {DD, a.l, a.h, a.n};
    const uint64_t s_l = a.l > 1 ? uint64_t(a.q_sl) : uint64_t(DD);
    const uint64_t s_h = a.h > 1 ? uint64_t(a.q_sh) : s_l * a.l;
    const uint64_t strides[4] = {1, s_l, s_h, uint64_t(a.n > 1 ? uint64_t(a.q_sn) : s_h * a.h)};
    const uint32_t box[4] = {64, a.l, G, 1};
    if (!encode_tmap_2byte(&mq, a.Q, 4, dims, strides, box)) return KUIOPS_EDRIVER;
  }
  auto enc_kv = [](CUtensorMap* m, const void* base, uint32_t rows, uint32_t heads, uint32_t n, int64_t s_row,
                   int64_t s_head, int64_t s_n) {
    const uint64_t dims[4] = {DD, rows, heads, n};
    const uint64_t sh = heads > 1 ? uint64_t(s_head) : uint64_t(s_row) * rows;
    const uint64_t strides[4] = {1, uint64_t(s_row), sh, uint64_t(n > 1 ? uint64_t(s_n) : sh * heads)};
    const uint32_t box[4] = {64, DBN, 1, 1};
    return encode_tmap_2byte(m, base, 4, dims, strides, box);
  };
  if (!enc_kv(&mk, a.K, a.s, a.h_kv, a.n, a.k_ss, a.k_sh, a.k_sn)) return KUIOPS_EDRIVER;
  if (!enc_kv(&mv, a.V, a.s, a.h_kv, a.n, a.v_ss, a.v_sh, a.v_sn)) return KUIOPS_EDRIVER;
  p.n = a.n; p.h = a.h; p.h_kv = a.h_kv; p.l = a.l; p.s = a.s; p.G = G; p.rows = G * a.l;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.is_causal = a.is_causal;
  p.kv_lens = a.kv_lens;
  p.out = a.out; p.o_sn = a.o_sn; p.o_sh = a.o_sh; p.o_sl = a.o_sl; p.lse = a.lse;
  p.err = tc_error_word_device();
  if (!p.err) return KUIOPS_ELAUNCH;
  p.trace = g_gemm_trace.load(std::memory_order_relaxed);
  const unsigned grid = unsigned(uint64_t(a.n) * a.h_kv * p.splits);
  if (p.rows <= 8)
    return decode_tc_launch_variant<T, true>(mq, mk, mv, p, grid, 2048 + 3 * (D_K_BYTES + D_V_BYTES) + 2 * 1024 + D_BAR_BYTES, st);
  return decode_tc_launch_variant<T, false>(mq, mk, mv, p, grid, D_SMEM + D_BAR_BYTES, st);
}

void sdpa_decode_tc_force_splits(int splits) { g_sdpa_splits_override.store(splits > 0 ? splits : 0, std::memory_order_relaxed); }

int sdpa_decode_tc(const SdpaArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (a.dtype == KUIOPS_BF16) return decode_tc_launch<__nv_bfloat16>(a, workspace, workspace_bytes, st);
  return decode_tc_launch<__half>(a, workspace, workspace_bytes, st);
}

}  // namespace kuiops
