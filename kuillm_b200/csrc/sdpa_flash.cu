// Flash-attention forward on tcgen05 for prefill: bf16 / f16, head dim 128, optional causal mask
// (bottom-right aligned), grouped-query heads, no bias.
//
// A CTA owns 128 query rows of one (batch, head).  K and V tiles of 64 keys arrive through one
// in-order TMA ring of five 16 KB buffers (K0 V0 K1 V1 ...): a K buffer is released as soon as
// its Q K^T has run and a V buffer after its P V, so loads run two to three tiles ahead of the
// softmax and their latency stays hidden.  Per tile:
//     S = Q K^T        UMMA 128 x 64 x 128, both operands K-major in shared memory, S in TMEM
//                      (two S buffers, so the next tile's scores are computed during this softmax)
//     softmax          4 warps, one query row per thread: tcgen05.ld S, online max / sum in the
//                      log2 domain in registers (3-input max, packed f32x2 FMA / add, ex2.approx);
//                      the O accumulator in TMEM is rescaled only when a row's running max grew by
//                      more than 2^8 (the stale max stays exact because the final normalisation
//                      uses the same max)
//     P                16-bit, stored back into TMEM over the S buffer it came from: the A operand
//                      of the second UMMA is read from TMEM, no shared-memory round trip
//     O += P V         UMMA 128 x 128 x 64, V MN-major as loaded
// Two CTAs share an SM (112 KB of shared memory and 256 TMEM columns each), so one CTA's softmax
// overlaps the other's MMAs.  The two warpgroups split the register file unevenly (setmaxnreg):
// the copy / issue warps keep 56 registers a thread, the four softmax warps take 200.
// Epilogue: O / l to global, natural-log LSE.
// This is the causal / grouped-query attention the dispatcher reaches as
// aten._scaled_dot_product_flash_attention; the reference only has the naive biased kernel
// (kuiops/sdpa/Kuiops.Sdpa.fst.1) and keeps it disconnected.
#include "sdpa.cuh"
#include "tc_ptx.cuh"
#include <type_traits>

namespace kuiops {

constexpr int FBM = 128;      // query rows per CTA (TMEM lanes)
constexpr int FBN = 64;       // keys per tile
constexpr int FD = 128;       // head dim
constexpr int kFlashThreads = 256;      // warp 0: TMA, warp 1: UMMA issue, warps 2-3: idle, warps 4-7: softmax
// setmaxnreg moves registers between the warpgroups of one CTA; the CTA's total stays what it was
// given at launch (256 threads x 128 registers, the most that lets two CTAs share an SM), and a
// warpgroup that asks for more than the other released would wait for ever.
constexpr int kFlashRegsLaunch = 128;
constexpr int kFlashRegsLow = 56;       // registers per thread kept by warps 0-3 ...
constexpr int kFlashRegsHigh = 200;     // ... and taken by the four softmax warps
static_assert(128 * kFlashRegsLow + 128 * kFlashRegsHigh <= kFlashThreads * kFlashRegsLaunch,
              "register budget of the CTA after setmaxnreg");
static_assert(2 * kFlashThreads * kFlashRegsLaunch <= 65536, "two CTAs per SM");
constexpr uint32_t F_Q_BYTES = FBM * FD * 2;        // 32 KB: two 64-column halves of 16 KB
constexpr uint32_t F_T_BYTES = FBN * FD * 2;        // 16 KB: one K or V tile, two 64-column boxes of 8 KB
constexpr int F_RING = 5;                           // ring position 2 j holds K of tile j, 2 j + 1 its V
constexpr uint32_t F_SMEM = F_Q_BYTES + F_RING * F_T_BYTES + 128;   // 112 KB + barriers
static_assert(2 * (F_SMEM + 1024) <= 227 * 1024, "two CTAs per SM");
constexpr uint32_t F_TMEM_COLS = 256;               // two S buffers at columns 0 and 64, O at column 128
constexpr float kRescaleThreshold = 8.0f;           // log2 units

struct FlashParams {
  uint32_t n, h, h_kv, l, s;
  float scale_log2;
  int is_causal;
  void* out; int64_t o_sn, o_sh, o_sl;
  float* lse;
  unsigned int* err;
};

__device__ __forceinline__ uint64_t flash_global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool flash_wait(uint64_t* bar, uint32_t parity) {
  if (tc::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = flash_global_ns();
  while (!tc::mbar_try_wait(bar, parity)) {
    if (flash_global_ns() - t0 > 2000000000ull) return false;
  }
  return true;
}

__device__ __forceinline__ float f_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float f_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// (a0, a1) = (a0, a1) * s + c as one packed instruction
__device__ __forceinline__ void f_fma2(float& a0, float& a1, float s, float c) {
  asm("{.reg .b64 ra, rb, rc;\n mov.b64 ra, {%0, %1};\n mov.b64 rb, {%2, %2};\n mov.b64 rc, {%3, %3};\n"
      " fma.rn.f32x2 ra, ra, rb, rc;\n mov.b64 {%0, %1}, ra;}"
      : "+f"(a0), "+f"(a1) : "f"(s), "f"(c));
}
__device__ __forceinline__ void f_add2(float& a0, float& a1, float b0, float b1) {
  asm("{.reg .b64 ra, rb;\n mov.b64 ra, {%0, %1};\n mov.b64 rb, {%2, %3};\n add.rn.f32x2 ra, ra, rb;\n mov.b64 {%0, %1}, ra;}"
      : "+f"(a0), "+f"(a1) : "f"(b0), "f"(b1));
}

template <typename T>
__global__ void __launch_bounds__(kFlashThreads, 2)
sdpa_flash_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  // The 128-byte swizzle atoms need a 1024-byte aligned base.  The dynamic shared window of a
  // kernel without static shared memory starts on such a boundary; there is no room for padding
  // (two CTAs must fit one SM), so a misaligned base is reported instead of worked around.
  extern __shared__ __align__(1024) unsigned char smem[];
  if ((tc::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.err, 10u);
    return;
  }
  unsigned char* q_s = smem;
  unsigned char* ring = q_s + F_Q_BYTES;                       // F_RING buffers of one K or V tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + F_RING * F_T_BYTES);
  uint64_t* q_full = bars;               // 1
  uint64_t* t_full = bars + 1;           // F_RING: tile landed
  uint64_t* t_empty = t_full + F_RING;   // F_RING: the UMMAs that read the tile have completed
  uint64_t* s_full = t_empty + F_RING;   // 2: S is double buffered so that Q K^T of the next tile overlaps this tile's softmax
  uint64_t* p_ready = s_full + 2;        // 1
  uint64_t* o_done = p_ready + 1;        // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heaviest query tiles (most visible keys under the causal mask) are scheduled first
  const uint32_t q_tiles = (p.l + FBM - 1) / FBM;
  const uint32_t qt = q_tiles - 1 - (blockIdx.x % q_tiles);
  const uint32_t head = (blockIdx.x / q_tiles) % p.h;
  const uint32_t b = blockIdx.x / (q_tiles * p.h);
  const uint32_t kvh = head / (p.h / p.h_kv);
  const uint32_t row0 = qt * FBM;
  // keys visible to this tile: all of them, or up to the diagonal of its last row
  uint32_t s_end = p.s;
  if (p.is_causal) {
    const uint64_t lim = uint64_t(min(row0 + FBM, p.l) - 1) + (p.s - p.l) + 1;
    s_end = uint32_t(lim < p.s ? lim : p.s);
  }
  const uint32_t n_tiles = (s_end + FBN - 1) / FBN;

  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmQ); tc::prefetch_tmap(&tmK); tc::prefetch_tmap(&tmV);
    tc::mbar_init(q_full, 1);
    for (int i = 0; i < F_RING; ++i) { tc::mbar_init(&t_full[i], 1); tc::mbar_init(&t_empty[i], 1); }
    tc::mbar_init(&s_full[0], 1);
    tc::mbar_init(&s_full[1], 1);
    tc::mbar_init(p_ready, 4);
    tc::mbar_init(o_done, 1);
    tc::fence_barrier_init();
    // The copies of Q and of the first ring positions need nothing but these barriers: start them
    // now, so that they fly while the tensor memory is being allocated and the CTA meets below.
    // (Q, K, V may still be being written by the previous kernel in the stream: wait for it first.)
    pdl_wait();
    tc::mbar_expect_tx(q_full, F_Q_BYTES);
    tc::tma_load_4d(q_s, &tmQ, q_full, 0, int(row0), int(head), int(b));
    tc::tma_load_4d(q_s + FBM * 128, &tmQ, q_full, 64, int(row0), int(head), int(b));
    const uint32_t first = min(uint32_t(F_RING), 2 * n_tiles);
    for (uint32_t n = 0; n < first; ++n) {
      unsigned char* dst = ring + n * F_T_BYTES;
      const CUtensorMap* tm = (n & 1) ? &tmV : &tmK;
      const int key0 = int((n >> 1) * FBN);
      tc::mbar_expect_tx(&t_full[n], F_T_BYTES);
      tc::tma_load_4d(dst, tm, &t_full[n], 0, key0, int(kvh), int(b));
      tc::tma_load_4d(dst + FBN * 128, tm, &t_full[n], 64, key0, int(kvh), int(b));
    }
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, F_TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128;
  if (threadIdx.x != 0) pdl_wait();      // thread 0 did before it started the first copies
  pdl_trigger();

  if (warp < 4) {
    // the warpgroup that only copies and issues gives most of its registers away
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kFlashRegsLow));
    if (warp == 0) {
      // ------------------------------ TMA producer ------------------------------------------
      if (lane == 0) {
        // ring position n = 2 j (K of tile j) or 2 j + 1 (V): buffer n % F_RING, use number n / F_RING;
        // Q and the first F_RING positions were requested during set-up
        for (uint32_t n = F_RING; n < 2 * n_tiles; ++n) {
          const uint32_t buf = n % F_RING, ph = (n / F_RING) & 1;
          if (!flash_wait(&t_empty[buf], ph ^ 1)) { atomicExch(p.err, 11u); break; }
          unsigned char* dst = ring + buf * F_T_BYTES;
          const CUtensorMap* tm = (n & 1) ? &tmV : &tmK;
          const int key0 = int((n >> 1) * FBN);
          tc::mbar_expect_tx(&t_full[buf], F_T_BYTES);
          tc::tma_load_4d(dst, tm, &t_full[buf], 0, key0, int(kvh), int(b));
          tc::tma_load_4d(dst + FBN * 128, tm, &t_full[buf], 64, key0, int(kvh), int(b));
        }
      }
    } else if (warp == 1) {
      // ------------------------------ UMMA issuer -------------------------------------------
      if (lane == 0) {
        constexpr int is_bf16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
        constexpr uint32_t idesc_qk = tc::make_idesc(is_bf16, 0, 0, FBM, FBN);
        constexpr uint32_t idesc_pv = tc::make_idesc(is_bf16, 0, 1, FBM, FD);
        bool ok = flash_wait(q_full, 0);
        if (!ok) atomicExch(p.err, 12u);
        const uint32_t qa = tc::smem_u32(q_s);
        // S = Q K^T of tile j into S buffer j & 1: two 64-wide halves of the head dim x four 16-wide steps
        auto issue_qk = [&](uint32_t j) -> bool {
          const uint32_t n = 2 * j, buf = n % F_RING, ph = (n / F_RING) & 1;
          const uint32_t ka = tc::smem_u32(ring + buf * F_T_BYTES);
          if (!flash_wait(&t_full[buf], ph)) { atomicExch(p.err, 13u); return false; }
          tc::tc_fence_after();
  #pragma unroll
          for (int hh = 0; hh < 2; ++hh)
  #pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t da = tc::make_smem_desc(qa + hh * (FBM * 128) + kk * 32, 16, 1024);
              const uint64_t db = tc::make_smem_desc(ka + hh * (FBN * 128) + kk * 32, 16, 1024);
              tc::umma_f16(tmem_S + (j & 1) * FBN, da, db, idesc_qk, (hh | kk) ? 1u : 0u);
            }
          tc::umma_commit(&t_empty[buf]);      // K of tile j may be overwritten once these have run
          tc::umma_commit(&s_full[j & 1]);
          return true;
        };
        if (ok && n_tiles > 0) ok = issue_qk(0);
        for (uint32_t j = 0; j < n_tiles && ok; ++j) {
          const uint32_t n = 2 * j + 1, buf = n % F_RING, ph = (n / F_RING) & 1;
          const uint32_t va = tc::smem_u32(ring + buf * F_T_BYTES);
          // The next tile's scores are computed while the softmax warps work on this one.  Their S
          // buffer holds P of tile j - 1; the UMMA that reads it was issued before this one and the
          // pipe runs in order, and the softmax warps left it when p_ready of tile j - 1 arrived.
          if (j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
          if (!flash_wait(p_ready, j & 1)) { atomicExch(p.err, 14u); ok = false; break; }
          if (!flash_wait(&t_full[buf], ph)) { atomicExch(p.err, 15u); ok = false; break; }
          tc::tc_fence_after();
          // O += P V over the 64 keys of the tile: four 16-key steps; P (16 keys = 8 TMEM columns of
          // the S buffer the softmax overwrote) from TMEM, V MN-major (head dim contiguous)
  #pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t db = tc::make_smem_desc(va + kk * 2048, FBN * 128, 1024);
            tc::umma_f16_ts(tmem_O, tmem_S + (j & 1) * FBN + kk * 8, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          }
          tc::umma_commit(&t_empty[buf]);
          tc::umma_commit(o_done);
        }
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kFlashRegsHigh));
    const uint32_t quarter = warp & 3;
    const uint32_t r = quarter * 32 + lane;               // row inside the tile
    const uint32_t row = row0 + r;
    const uint32_t lane_addr = (quarter * 32) << 16;
    // last key this row may see (inclusive); rows beyond l see nothing useful but stay finite
    const int64_t row_lim = p.is_causal ? int64_t(min(row, p.l - 1)) + int64_t(p.s) - int64_t(p.l) : int64_t(p.s) - 1;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (uint32_t j = 0; j < n_tiles && ok; ++j) {
      if (!flash_wait(&s_full[j & 1], (j >> 1) & 1)) { atomicExch(p.err, 16u); ok = false; break; }
      tc::tc_fence_after();
      float sv[FBN];
      tc::tmem_ld32(tmem_S + (j & 1) * FBN + lane_addr, sv);
      tc::tmem_ld32(tmem_S + (j & 1) * FBN + lane_addr + 32, sv + 32);
      tc::tmem_ld_wait();
      const int64_t key0 = int64_t(j) * FBN;
      // tile crosses this row's limit (or the end of the keys): only the diagonal and last tiles
      if (__any_sync(0xffffffffu, key0 + FBN - 1 > row_lim)) {
#pragma unroll
        for (int c = 0; c < FBN; ++c)
          if (key0 + c > row_lim) sv[c] = -INFINITY;
      }
      float m0 = f_max3(sv[0], sv[1], sv[2]), m1 = f_max3(sv[3], sv[4], sv[5]);
      float m2 = f_max3(sv[6], sv[7], sv[8]), m3 = f_max3(sv[9], sv[10], sv[11]);
#pragma unroll
      for (int c = 12; c + 8 <= FBN; c += 8) {
        m0 = f_max3(m0, sv[c], sv[c + 1]);
        m1 = f_max3(m1, sv[c + 2], sv[c + 3]);
        m2 = f_max3(m2, sv[c + 4], sv[c + 5]);
        m3 = f_max3(m3, sv[c + 6], sv[c + 7]);
      }
      // 12 + 8 * 6 = 60: the last four columns
      m0 = f_max3(m0, sv[FBN - 4], sv[FBN - 3]);
      m1 = f_max3(m1, sv[FBN - 2], sv[FBN - 1]);
      float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * p.scale_log2;   // scale > 0: the max commutes with the scaling
      float corr = 1.f;
      if (mx > m_used + kRescaleThreshold || m_used == -INFINITY) {
        const float m_new = fmaxf(mx, m_used);
        corr = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
        m_used = m_new;
      }
      const float nmm = (m_used == -INFINITY) ? 0.f : -m_used;   // a fully masked row keeps p = 0
      float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
      uint32_t pk[FBN / 2];                       // P as packed 16-bit pairs (key 2c, key 2c + 1)
#pragma unroll
      for (int c = 0; c < FBN; c += 4) {
        f_fma2(sv[c], sv[c + 1], p.scale_log2, nmm);
        f_fma2(sv[c + 2], sv[c + 3], p.scale_log2, nmm);
        const float e0 = f_ex2(sv[c]), e1 = f_ex2(sv[c + 1]), e2 = f_ex2(sv[c + 2]), e3 = f_ex2(sv[c + 3]);
        f_add2(r0, r1, e0, e1);
        f_add2(r2, r3, e2, e3);
        pk[c / 2] = pack2<T>(e0, e1);
        pk[c / 2 + 1] = pack2<T>(e2, e3);
      }
      l_run = l_run * corr + ((r0 + r1) + (r2 + r3));
      const bool rescale = j > 0 && __any_sync(0xffffffffu, corr != 1.f);
      if (j > 0) {
        // The previous P V must be done before O is touched.  It is waited for in every tile, also
        // when nothing depends on it: a parity wait only tells the current phase of the barrier from the one before, so
        // every phase has to be observed in turn.  The wait sits after this tile's exponentials,
        // by which time that UMMA has normally completed.
        if (!flash_wait(o_done, (j - 1) & 1)) { atomicExch(p.err, 17u); ok = false; break; }
        tc::tc_fence_after();
      }
      if (rescale) {
#pragma unroll
        for (int c0 = 0; c0 < FD; c0 += 16) {
          float ov[16];
          tc::tmem_ld16(tmem_O + lane_addr + c0, ov);
          tc::tmem_ld_wait();
          uint32_t ou[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) ou[c] = __float_as_uint(ov[c] * corr);
          tc::tmem_st16(tmem_O + lane_addr + c0, ou);
        }
        tc::tmem_st_wait();
      }
      // row r of P goes into the S buffer this tile came from, column c = keys 2c and 2c + 1
      tc::tmem_st32(tmem_S + (j & 1) * FBN + lane_addr, pk);
      tc::tmem_st_wait();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(p_ready);
    }
    if (ok && n_tiles > 0) {
      if (!flash_wait(o_done, (n_tiles - 1) & 1)) { atomicExch(p.err, 18u); ok = false; }
    }
    if (ok) {
      tc::tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      T* orow = static_cast<T*>(p.out) + size_t(b) * p.o_sn + size_t(head) * p.o_sh + size_t(row) * p.o_sl;
#pragma unroll
      for (int c0 = 0; c0 < FD; c0 += 32) {
        float ov[32];
        if (n_tiles > 0) {
          tc::tmem_ld32(tmem_O + lane_addr + c0, ov);
          tc::tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) ov[c] = 0.f;
        }
        if (row < p.l) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            Vec16<T> o;
#pragma unroll
            for (int e = 0; e < 8; ++e) o.v[e] = ElemTraits<T>::from_f(ov[c + e] * inv);
            st16(orow + c0 + c, o);
          }
        }
      }
      if (p.lse && row < p.l)
        p.lse[(size_t(b) * p.h + head) * p.l + row] = l_run > 0.f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, F_TMEM_COLS);
  }
}

bool sdpa_flash_eligible(const SdpaArgs& a) {
  if (a.dtype != KUIOPS_BF16 && a.dtype != KUIOPS_F16) return false;
  if (!(a.scale > 0.f)) return false;               // the softmax takes the row max before scaling
  if (a.e != FD || a.ev != FD || a.bias != nullptr || a.kv_lens != nullptr) return false;
  if (a.l < 64) return false;                       // short query blocks belong to the split-KV kernel
  if (a.is_causal && a.l > a.s) return false;       // rows without any visible key
  auto ok_stride = [](int64_t s) { return s > 0 && s % 8 == 0 && uint64_t(s) * 2 < (1ull << 40); };
  if (!ok_stride(a.q_sl) || !ok_stride(a.k_ss) || !ok_stride(a.v_ss) || a.o_sl % 8) return false;
  if ((a.h > 1 && (!ok_stride(a.q_sh) || a.o_sh % 8)) || (a.h_kv > 1 && (!ok_stride(a.k_sh) || !ok_stride(a.v_sh)))) return false;
  if (a.n > 1 && (!ok_stride(a.q_sn) || !ok_stride(a.k_sn) || !ok_stride(a.v_sn) || a.o_sn % 8)) return false;
  if (!aligned16(a.Q) || !aligned16(a.K) || !aligned16(a.V) || !aligned16(a.out)) return false;
  const uint64_t ctas = uint64_t(a.n) * a.h * ((a.l + FBM - 1) / FBM);
  return ctas < (1ull << 31);
}

template <typename T>
static int flash_launch(const SdpaArgs& a, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  auto enc = [](CUtensorMap* m, const void* base, uint32_t rows, uint32_t heads, uint32_t n, int64_t s_row,
                int64_t s_head, int64_t s_n, uint32_t box_rows) {
    const uint64_t dims[4] = {FD, rows, heads, n};
    // a dimension of extent 1 may carry any stride; keep it a legal multiple of 16 bytes
    const uint64_t strides[4] = {1, uint64_t(s_row), uint64_t(heads > 1 ? s_head : s_row * rows),
                                 uint64_t(n > 1 ? s_n : (heads > 1 ? s_head * heads : s_row * rows))};
    const uint32_t box[4] = {64, box_rows, 1, 1};
    return encode_tmap_2byte(m, base, 4, dims, strides, box);
  };
  if (!enc(&mq, a.Q, a.l, a.h, a.n, a.q_sl, a.q_sh, a.q_sn, FBM)) return KUIOPS_EDRIVER;
  if (!enc(&mk, a.K, a.s, a.h_kv, a.n, a.k_ss, a.k_sh, a.k_sn, FBN)) return KUIOPS_EDRIVER;
  if (!enc(&mv, a.V, a.s, a.h_kv, a.n, a.v_ss, a.v_sh, a.v_sn, FBN)) return KUIOPS_EDRIVER;
  FlashParams p = {};
  p.n = a.n; p.h = a.h; p.h_kv = a.h_kv; p.l = a.l; p.s = a.s;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.is_causal = a.is_causal;
  p.out = a.out; p.o_sn = a.o_sn; p.o_sh = a.o_sh; p.o_sl = a.o_sl; p.lse = a.lse;
  p.err = tc_error_word_device();
  if (!p.err) return KUIOPS_ELAUNCH;
  constexpr size_t smem = F_SMEM;
  auto kern = sdpa_flash_kernel<T>;
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return KUIOPS_ELAUNCH;
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return KUIOPS_ELAUNCH;
    // the register hand-over inside the kernel assumes the allocation the compiler reported; a
    // build with fewer registers per thread would leave a warpgroup waiting for registers for ever
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) return KUIOPS_ELAUNCH;
    if (fa.numRegs * kFlashThreads < 128 * kFlashRegsLow + 128 * kFlashRegsHigh) return KUIOPS_EUNSUPPORTED;
    configured.fetch_or(bit, std::memory_order_release);
  }
  const unsigned grid = unsigned(uint64_t(a.n) * a.h * ((a.l + FBM - 1) / FBM));
  return launch_pdl(kern, dim3(grid), dim3(kFlashThreads), smem, st, mq, mk, mv, p);
}

int sdpa_flash(const SdpaArgs& a, cudaStream_t st) {
  if (a.dtype == KUIOPS_BF16) return flash_launch<__nv_bfloat16>(a, st);
  return flash_launch<__half>(a, st);
}

}  // namespace kuiops
