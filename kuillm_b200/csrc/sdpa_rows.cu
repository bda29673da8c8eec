// SIMT scaled-dot-product attention for short query blocks.
//
// A CTA owns up to R query rows that read the same KV head (the heads of one GQA group times a
// few query positions) and a slice of the keys.  Its four warps walk 32-key tiles on their own:
// for the QK^T step every lane owns one key and dots it against the R query rows held in
// shared memory; for the PV step every lane owns DV adjacent value columns, so each V row is
// one coalesced warp read shared by all R rows.  Softmax is online in the log2 domain.  The
// warps' states are merged through shared memory; when the keys are split over several CTAs
// (decode against a long cache) the partial (max, sum, acc) triples meet in the workspace and
// the CTA drawing the last ticket merges them.
// This is the kernel for decode (one query token against a KV cache, HBM bound: each K/V byte
// is read once per GQA group) and the fallback for every shape / dtype / bias form the
// tensor-core prefill kernel does not take.  It computes what Kuiper.Kernel.SDPA.LSE
// (kuiops/sdpa/Kuiops.Sdpa.fst.1:13-27) computes, without materialising the L x S scores.
#include "common.cuh"
#include "sdpa.cuh"

namespace kuiops {

constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;

template <typename T> struct KvLoad;
template <> struct KvLoad<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* o) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct KvLoad<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
  }
};
template <> struct KvLoad<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __half* p, float* o) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
  }
};

template <typename T, int R, int DV>
__global__ void __launch_bounds__(128)
sdpa_rows_kernel(const SdpaArgs p, const SdpaRowsPlan pl) {
  extern __shared__ __align__(16) float sm[];
  float* q_s = sm;                                  // [R][e_pad]
  float* mrg = sm + R * pl.e_pad;                   // [4 warps + 1][R][DV*32 + 2]
  __shared__ int last_flag;
  constexpr int ACCW = DV * 32 + 2;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // unit = (batch, head group, query block); blockIdx.x = unit * splits + split
  const uint32_t split = blockIdx.x % pl.splits;
  const uint32_t unit = blockIdx.x / pl.splits;
  const uint32_t lblk = unit % pl.lblocks;
  const uint32_t hgrp = (unit / pl.lblocks) % pl.hgroups;
  const uint32_t b = unit / (pl.lblocks * pl.hgroups);
  const uint32_t G = p.h / p.h_kv;
  const uint32_t kvh = (hgrp * pl.rows_h) / G;
  const uint32_t rows = pl.rows_h * pl.rows_l;

  // keys of this batch entry (a device-side count lets one captured launch serve a growing cache)
  uint32_t S = p.s;
  if (p.kv_lens) {
    const long long kl = p.kv_lens[b];
    S = kl < 0 ? 0u : (kl < (long long)p.s ? uint32_t(kl) : p.s);
  }
  // key slice of this split
  const uint32_t per = (S + pl.splits - 1) / pl.splits;
  const uint32_t s_lo = min(split * per, S), s_hi_raw = min(s_lo + per, S);

  // stage the query rows (pre-multiplied by scale * log2 e) and find the causal limits
  const float qmul = p.scale * kLog2eF;
  for (uint32_t i = tid; i < R * pl.e_pad; i += 128) {
    const uint32_t r = i / pl.e_pad, e = i % pl.e_pad;
    float v = 0.f;
    if (r < rows && e < p.e) {
      const uint32_t head = hgrp * pl.rows_h + r / pl.rows_l, li = lblk * pl.rows_l + r % pl.rows_l;
      if (li < p.l)
        v = ElemTraits<T>::to_f(static_cast<const T*>(p.Q)[size_t(b) * p.q_sn + size_t(head) * p.q_sh + size_t(li) * p.q_sl + e]) * qmul;
    }
    q_s[i] = v;
  }
  __syncthreads();

  int lim[R];          // last visible key of each row (inclusive); -1 = none
  int lim_max = -1;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t li = lblk * pl.rows_l + uint32_t(r) % pl.rows_l;
    if (uint32_t(r) < rows && li < p.l) {
      const long long c = p.is_causal ? (long long)li + (long long)S - (long long)p.l : (long long)S - 1;
      lim[r] = int(c < (long long)S - 1 ? c : (long long)S - 1);
    } else {
      lim[r] = -1;
    }
    lim_max = max(lim_max, lim[r]);
  }
  const uint32_t s_hi = min(s_hi_raw, uint32_t(lim_max + 1));

  float m[R], lsum[R], acc[R][DV];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -INFINITY; lsum[r] = 0.f;
#pragma unroll
    for (int d = 0; d < DV; ++d) acc[r][d] = 0.f;
  }

  const T* Kb = static_cast<const T*>(p.K) + size_t(b) * p.k_sn + size_t(kvh) * p.k_sh;
  const T* Vb = static_cast<const T*>(p.V) + size_t(b) * p.v_sn + size_t(kvh) * p.v_sh;
  constexpr int KN = KvLoad<T>::N;

  for (uint32_t tile = s_lo + warp * 32; tile < s_hi; tile += 128) {
    const uint32_t j = tile + lane;
    const bool kvalid = j < s_hi;
    float sc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) sc[r] = 0.f;
    if (kvalid) {
      const T* krow = Kb + size_t(j) * p.k_ss;
      if (pl.k_vec) {
        for (uint32_t e = 0; e < p.e; e += KN) {
          float kf[KN];
          KvLoad<T>::load(krow + e, kf);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float* q = q_s + r * pl.e_pad + e;
#pragma unroll
            for (int t = 0; t < KN; ++t) sc[r] = fmaf(q[t], kf[t], sc[r]);
          }
        }
      } else {
        for (uint32_t e = 0; e < p.e; ++e) {
          const float kf = ElemTraits<T>::to_f(krow[e]);
#pragma unroll
          for (int r = 0; r < R; ++r) sc[r] = fmaf(q_s[r * pl.e_pad + e], kf, sc[r]);
        }
      }
    }
    float pr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float s2 = sc[r];
      const bool vis = kvalid && int(j) <= lim[r];
      if (vis && p.bias) {
        const uint32_t head = hgrp * pl.rows_h + uint32_t(r) / pl.rows_l, li = lblk * pl.rows_l + uint32_t(r) % pl.rows_l;
        s2 += ElemTraits<T>::to_f(static_cast<const T*>(p.bias)[((size_t(b) * p.h + head) * p.l + li) * p.s + j]) * kLog2eF;
      }
      if (!vis) s2 = -INFINITY;
      const float mt = warp_max(s2);
      const float mn = fmaxf(m[r], mt);
      float corr = 1.f, pv = 0.f;
      if (mn != -INFINITY) {
        corr = exp2f(m[r] - mn);            // m[r] = -inf gives 0
        pv = exp2f(s2 - mn);                // masked keys give 0
      }
      lsum[r] = lsum[r] * corr + warp_sum(pv);
      m[r] = mn;
#pragma unroll
      for (int d = 0; d < DV; ++d) acc[r][d] *= corr;
      pr[r] = pv;
    }
    // PV: lane owns value columns [lane*DV, lane*DV + DV)
    const uint32_t d0 = lane * DV;
    const uint32_t nk = min(32u, s_hi - tile);
    for (uint32_t jj = 0; jj < nk; ++jj) {
      const T* vrow = Vb + size_t(tile + jj) * p.v_ss + d0;
      float vf[DV];
      if (pl.v_vec && d0 + DV <= p.ev) {
        if (sizeof(T) * DV == 16) {
          float tmp[KvLoad<T>::N];
          KvLoad<T>::load(vrow, tmp);
#pragma unroll
          for (int d = 0; d < DV; ++d) vf[d] = tmp[d];
        } else if (sizeof(T) * DV == 8) {
          uint2 raw = *reinterpret_cast<const uint2*>(vrow);
          const T* t2 = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int d = 0; d < DV; ++d) vf[d] = ElemTraits<T>::to_f(t2[d]);
        } else if (sizeof(T) * DV == 4) {
          uint32_t raw = *reinterpret_cast<const uint32_t*>(vrow);
          const T* t2 = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int d = 0; d < DV; ++d) vf[d] = ElemTraits<T>::to_f(t2[d]);
        } else {
#pragma unroll
          for (int d = 0; d < DV; ++d) vf[d] = ElemTraits<T>::to_f(vrow[d]);
        }
      } else {
#pragma unroll
        for (int d = 0; d < DV; ++d) vf[d] = (d0 + d < p.ev) ? ElemTraits<T>::to_f(vrow[d]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float pj = __shfl_sync(0xffffffffu, pr[r], jj);
#pragma unroll
        for (int d = 0; d < DV; ++d) acc[r][d] = fmaf(pj, vf[d], acc[r][d]);
      }
    }
  }

  // ---- merge the four warps ---------------------------------------------------------------
  {
    float* mine = mrg + size_t(warp) * R * ACCW;
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int d = 0; d < DV; ++d) mine[r * ACCW + lane * DV + d] = acc[r][d];
      if (lane == 0) { mine[r * ACCW + DV * 32] = m[r]; mine[r * ACCW + DV * 32 + 1] = lsum[r]; }
    }
  }
  __syncthreads();
  // merged state of the CTA -> `fin` ([R][ACCW]: DV*32 accumulators, then max, then sum)
  float* fin = mrg + size_t(4) * R * ACCW;
  for (uint32_t i = tid; i < R * ACCW; i += 128) {
    const uint32_t r = i / ACCW, c = i % ACCW;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mrg[(size_t(w) * R + r) * ACCW + DV * 32]);
    float a = mm;
    if (c != DV * 32) {
      a = 0.f;
      for (int w = 0; w < 4; ++w) {
        const float mw = mrg[(size_t(w) * R + r) * ACCW + DV * 32];
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
        a += f * mrg[(size_t(w) * R + r) * ACCW + c];
      }
    }
    fin[i] = a;
  }
  __syncthreads();

  auto write_out = [&](const float* state) {
    for (uint32_t i = tid; i < rows * p.ev; i += 128) {
      const uint32_t r = i / p.ev, d = i % p.ev;
      const uint32_t head = hgrp * pl.rows_h + r / pl.rows_l, li = lblk * pl.rows_l + r % pl.rows_l;
      if (li >= p.l) continue;
      const float l = state[r * ACCW + DV * 32 + 1];
      const float o = l > 0.f ? state[r * ACCW + d] / l : 0.f;
      static_cast<T*>(p.out)[size_t(b) * p.o_sn + size_t(head) * p.o_sh + size_t(li) * p.o_sl + d] = ElemTraits<T>::from_f(o);
    }
    if (p.lse) {
      for (uint32_t r = tid; r < rows; r += 128) {
        const uint32_t head = hgrp * pl.rows_h + r / pl.rows_l, li = lblk * pl.rows_l + r % pl.rows_l;
        if (li >= p.l) continue;
        const float l = state[r * ACCW + DV * 32 + 1], mm = state[r * ACCW + DV * 32];
        p.lse[(size_t(b) * p.h + head) * p.l + li] = l > 0.f ? (mm + log2f(l)) * kLn2F : -INFINITY;
      }
    }
  };

  if (pl.splits == 1) {
    write_out(fin);
    return;
  }
  // ---- split-KV: park the state, last CTA of the unit merges ------------------------------
  float* part = pl.partials + (size_t(unit) * pl.splits + split) * (R * ACCW);
  for (uint32_t i = tid; i < R * ACCW; i += 128) __stcg(&part[i], fin[i]);
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&pl.counters[unit], 1);
    last_flag = (old == int(pl.splits) - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  const float* all = pl.partials + size_t(unit) * pl.splits * (R * ACCW);
  for (uint32_t i = tid; i < R * ACCW; i += 128) {
    const uint32_t r = i / ACCW, c = i % ACCW;
    float mm = -INFINITY;
    for (uint32_t s2 = 0; s2 < pl.splits; ++s2) mm = fmaxf(mm, __ldcg(&all[size_t(s2) * R * ACCW + r * ACCW + DV * 32]));
    float a = 0.f;
    if (c < DV * 32 || c == DV * 32 + 1) {
      for (uint32_t s2 = 0; s2 < pl.splits; ++s2) {
        const float mw = __ldcg(&all[size_t(s2) * R * ACCW + r * ACCW + DV * 32]);
        const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
        a += f * __ldcg(&all[size_t(s2) * R * ACCW + r * ACCW + c]);
      }
    } else {
      a = mm;
    }
    mrg[i] = a;                // the per-warp slots are free again
  }
  __syncthreads();
  write_out(mrg);
  if (tid == 0) pl.counters[unit] = 0;
}

template <typename T, int R, int DV>
static int launch_rows(const SdpaArgs& a, const SdpaRowsPlan& pl, cudaStream_t st) {
  constexpr int ACCW = DV * 32 + 2;
  const size_t smem = (size_t(R) * pl.e_pad + size_t(5) * R * ACCW) * sizeof(float);
  auto kern = sdpa_rows_kernel<T, R, DV>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
    return KUIOPS_ELAUNCH;
  const uint64_t grid = uint64_t(pl.units) * pl.splits;
  if (grid >= (1ull << 31)) return KUIOPS_EUNSUPPORTED;
  kern<<<unsigned(grid), 128, smem, st>>>(a, pl);
  return check_launch();
}

template <typename T, int R>
static int launch_rows_dv(const SdpaArgs& a, const SdpaRowsPlan& pl, cudaStream_t st) {
  if (a.ev <= 64) return launch_rows<T, R, 2>(a, pl, st);
  if (a.ev <= 128) return launch_rows<T, R, 4>(a, pl, st);
  if (a.ev <= 256) return launch_rows<T, R, 8>(a, pl, st);
  return KUIOPS_EUNSUPPORTED;
}

template <typename T>
static int launch_rows_t(const SdpaArgs& a, const SdpaRowsPlan& pl, cudaStream_t st) {
  const uint32_t rows = pl.rows_h * pl.rows_l;
  if (rows <= 1) return launch_rows_dv<T, 1>(a, pl, st);
  if (rows <= 4) return launch_rows_dv<T, 4>(a, pl, st);
  if (rows <= 8) return launch_rows_dv<T, 8>(a, pl, st);
  return launch_rows_dv<T, 16>(a, pl, st);
}

SdpaRowsPlan sdpa_rows_plan(const SdpaArgs& a) {
  SdpaRowsPlan pl = {};
  const uint32_t G = a.h / a.h_kv;
  if (G <= 16) { pl.rows_h = G; pl.rows_l = a.l < 16 / G ? a.l : 16 / G; }
  else { pl.rows_h = 1; pl.rows_l = a.l < 16 ? a.l : 16; }
  if (pl.rows_l == 0) pl.rows_l = 1;
  pl.hgroups = a.h / pl.rows_h;
  pl.lblocks = (a.l + pl.rows_l - 1) / pl.rows_l;
  pl.units = uint64_t(a.n) * pl.hgroups * pl.lblocks;
  pl.e_pad = (a.e + 7) & ~7u;
  pl.splits = 1;
  if (pl.units < 2 * uint64_t(num_sms())) {
    uint32_t want = uint32_t((4 * uint64_t(num_sms()) + pl.units - 1) / pl.units);
    uint32_t cap = a.s / 512;
    if (cap < 1) cap = 1;
    pl.splits = want < cap ? want : cap;
    if (pl.splits > 64) pl.splits = 64;
  }
  const uint32_t rows = pl.rows_h * pl.rows_l;
  pl.r_pad = rows <= 1 ? 1 : (rows <= 4 ? 4 : (rows <= 8 ? 8 : 16));
  pl.dv = a.ev <= 64 ? 2 : (a.ev <= 128 ? 4 : 8);
  return pl;
}

size_t sdpa_rows_workspace_bytes(const SdpaArgs& a) {
  SdpaRowsPlan pl = sdpa_rows_plan(a);
  if (pl.splits == 1) return 0;
  const size_t counters = (size_t(pl.units) * 4 + 255) & ~size_t(255);
  return counters + size_t(pl.units) * pl.splits * pl.r_pad * (pl.dv * 32 + 2) * sizeof(float);
}

size_t sdpa_rows_counter_bytes(const SdpaArgs& a) {
  SdpaRowsPlan pl = sdpa_rows_plan(a);
  return pl.splits == 1 ? 0 : ((size_t(pl.units) * 4 + 255) & ~size_t(255));
}

int sdpa_rows(const SdpaArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (a.ev > 256 || a.e > 1024) return KUIOPS_EUNSUPPORTED;
  SdpaRowsPlan pl = sdpa_rows_plan(a);
  if (pl.splits > 1) {
    if (!workspace || workspace_bytes < sdpa_rows_workspace_bytes(a)) {
      pl.splits = 1;        // no scratch: run unsplit rather than fail
    } else {
      pl.counters = static_cast<int*>(workspace);
      pl.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + ((size_t(pl.units) * 4 + 255) & ~size_t(255)));
    }
  }
  const size_t esz = a.dtype == KUIOPS_F32 ? 4 : 2;
  const uint32_t kn = a.dtype == KUIOPS_F32 ? 4 : 8;
  pl.k_vec = (a.e % kn == 0) && aligned16(a.K) && (a.k_ss * esz % 16 == 0) && (a.k_sh * esz % 16 == 0) && (a.k_sn * esz % 16 == 0);
  const size_t vchunk = pl.dv * esz;
  pl.v_vec = (reinterpret_cast<uintptr_t>(a.V) % vchunk == 0) && (a.v_ss * esz % vchunk == 0) &&
             (a.v_sh * esz % vchunk == 0) && (a.v_sn * esz % vchunk == 0);
  switch (a.dtype) {
    case KUIOPS_F32: return launch_rows_t<float>(a, pl, st);
    case KUIOPS_BF16: return launch_rows_t<__nv_bfloat16>(a, pl, st);
    case KUIOPS_F16: return launch_rows_t<__half>(a, pl, st);
  }
  return KUIOPS_EINVAL;
}

}  // namespace kuiops
