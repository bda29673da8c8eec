// Categorical sampling from the rows of an [m, n] fp32 matrix of non-negative weights
// (aten.multinomial with one sample per row, or several with replacement).  The reference lists
// multinomial as backlog only (KERNELS.md:68-90) and has no kernel.
//
// PyTorch's own multinomial draws from its generator's stream in an order private to its kernels,
// so the draws cannot be reproduced bit for bit; what is reproduced is the distribution.  The
// stream used here is documented instead, so that a caller (and the CPU oracle of the tests) can
// recompute every draw:
//   u(row, sample) = (x0 >> 8) * 2^-24, (x0, ..) = Philox4x32-10(counter = (offset_lo, offset_hi,
//   row, sample), key = (seed_lo, seed_hi)),
// and the sampled index is found by inverting the running sum of the row, evaluated in a fixed
// order: 4 elements per lane left to right, an inclusive Hillis-Steele scan over the 32 lanes of a
// 128-element group, groups added left to right inside a warp's segment, the 32 segments added
// left to right.  With target = u * total, the walk descends segment -> group -> lane -> element,
// at every level taking the first entry with non-zero weight whose running sum exceeds the target
// and, should rounding leave none, the last entry with non-zero weight.  An element of weight zero
// is therefore never drawn.
//
// One CTA of 32 warps per row; each warp streams its contiguous segment with coalesced 16-byte
// loads; only the warp that owns the target reads its segment a second time (from L2).
#include "common.cuh"

namespace kuiops {

constexpr int kSampThreads = 1024;
constexpr int kSampWarps = kSampThreads / 32;
constexpr int kSampGroup = 128;                    // elements per warp iteration: 32 lanes x 4

__host__ __device__ inline void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                               uint32_t out[4]) {
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = uint64_t(0xD2511F53u) * c0, p1 = uint64_t(0xCD9E8D57u) * c2;
    const uint32_t n0 = uint32_t(p1 >> 32) ^ c1 ^ k0, n1 = uint32_t(p1), n2 = uint32_t(p0 >> 32) ^ c3 ^ k1, n3 = uint32_t(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct GroupScan { float incl, excl, own; float a[4]; };

// This lane's four weights of the 128-element group starting at g0 (zero beyond n).
__device__ __forceinline__ float4 load_group(const float* __restrict__ p, uint32_t n, uint32_t g0, int lane, bool vec) {
  const uint32_t i0 = g0 + uint32_t(lane) * 4;
  if (vec && i0 + 4 <= n) return *reinterpret_cast<const float4*>(p + i0);
  float4 v;
  v.x = (i0 < n) ? p[i0] : 0.f;
  v.y = (i0 + 1 < n) ? p[i0 + 1] : 0.f;
  v.z = (i0 + 2 < n) ? p[i0 + 2] : 0.f;
  v.w = (i0 + 3 < n) ? p[i0 + 3] : 0.f;
  return v;
}

// A 128-element group from its loaded weights: the lane's four weights (zero where the weight is not a
// non-negative finite number), their left-to-right sum, and the inclusive / exclusive scans of the lanes'
// sums.  `bad` collects whether a weight was negative, infinite or NaN.
__device__ __forceinline__ GroupScan scan_loaded(float4 w4, int lane, bool& bad) {
  GroupScan r;
  r.a[0] = w4.x; r.a[1] = w4.y; r.a[2] = w4.z; r.a[3] = w4.w;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float w = r.a[j];
    if (!(w >= 0.f) || w > 3.402823466e38f) { bad = true; r.a[j] = 0.f; }
  }
  r.own = ((r.a[0] + r.a[1]) + r.a[2]) + r.a[3];
  float incl = r.own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  r.incl = incl;
  const float prev = __shfl_up_sync(0xffffffffu, incl, 1);
  r.excl = lane == 0 ? 0.f : prev;
  return r;
}

__device__ __forceinline__ GroupScan scan_group(const float* __restrict__ p, uint32_t n, uint32_t g0, int lane, bool vec, bool& bad) {
  return scan_loaded(load_group(p, n, g0, lane, vec), lane, bad);
}

__global__ void __launch_bounds__(kSampThreads)
multinomial_rows_kernel(uint32_t n, uint32_t num_samples, const float* __restrict__ P, int64_t* __restrict__ out,
                        uint32_t seed_lo, uint32_t seed_hi, uint32_t off_lo, uint32_t off_hi, int* status) {
  __shared__ float seg_sum[kSampWarps];
  __shared__ float prefix[kSampWarps + 1];
  __shared__ int pick_seg;
  __shared__ float pick_target;
  const uint32_t row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* p = P + size_t(row) * n;
  const bool vec = (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
  const uint32_t groups = (n + kSampGroup - 1) / kSampGroup;
  const uint32_t gpw = (groups + kSampWarps - 1) / kSampWarps;           // groups per warp segment
  const uint32_t gk0 = min(uint32_t(warp) * gpw, groups), gk1 = min(gk0 + gpw, groups);
  pdl_wait();
  pdl_trigger();

  // ---- phase A: the sum of every segment -----------------------------------------------------
  bool bad = false;
  float s = 0.f;
  for (uint32_t k = gk0; k < gk1; k += 4) {
    // four groups' loads in flight before the first scan (the order of the additions is unchanged)
    float4 v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) v[q] = (k + q < gk1) ? load_group(p, n, (k + q) * kSampGroup, lane, vec) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (k + q < gk1) {
        const GroupScan g = scan_loaded(v[q], lane, bad);
        s += __shfl_sync(0xffffffffu, g.incl, 31);
      }
    }
  }
  if (lane == 0) seg_sum[warp] = s;
  if (__any_sync(0xffffffffu, bad) && lane == 0 && status) atomicExch(status, 2);
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    prefix[0] = 0.f;
    for (int w = 0; w < kSampWarps; ++w) { run += seg_sum[w]; prefix[w + 1] = run; }
    if (!(run > 0.f) && status) atomicExch(status, 3);                   // nothing to draw from
  }
  __syncthreads();
  const float total = prefix[kSampWarps];

  // ---- phase B: one walk per sample ----------------------------------------------------------
  for (uint32_t smp = 0; smp < num_samples; ++smp) {
    if (tid == 0) {
      uint32_t x[4];
      philox4x32_10(off_lo, off_hi, row, smp, seed_lo, seed_hi, x);
      const float u = float(x[0] >> 8) * 5.9604644775390625e-08f;        // 2^-24: u in [0, 1)
      const float t = __fmul_rn(u, total);                               // no contraction with the subtraction below
      int w = -1, last = -1;
      for (int q = 0; q < kSampWarps; ++q) {
        if (seg_sum[q] > 0.f) {
          last = q;
          if (prefix[q + 1] > t) { w = q; break; }
        }
      }
      if (w < 0) w = last;
      pick_seg = w;
      pick_target = w >= 0 ? __fsub_rn(t, prefix[w]) : 0.f;
      if (w < 0) out[size_t(row) * num_samples + smp] = 0;
    }
    __syncthreads();
    if (warp == pick_seg) {
      const float t = pick_target;
      bool bad2 = false;
      float run = 0.f, hit_run = 0.f;
      uint32_t hit = 0xFFFFFFFFu, last = 0xFFFFFFFFu;
      float last_run = 0.f;
      for (uint32_t k = gk0; k < gk1; ++k) {
        const GroupScan g = scan_group(p, n, k * kSampGroup, lane, vec, bad2);
        const float gs = __shfl_sync(0xffffffffu, g.incl, 31);
        if (gs > 0.f) {
          last = k; last_run = run;
          if (run + gs > t) { hit = k; hit_run = run; break; }
        }
        run += gs;
      }
      if (hit == 0xFFFFFFFFu) { hit = last; hit_run = last_run; }
      if (hit == 0xFFFFFFFFu) {                       // a segment without weight is never picked; keep the walk in bounds anyway
        if (lane == 0) out[size_t(row) * num_samples + smp] = 0;
        hit = gk0 < groups ? gk0 : 0;
      }
      // inside the group: first lane with weight whose running sum exceeds the target, else the last lane with weight
      const GroupScan g = scan_group(p, n, hit * kSampGroup, lane, vec, bad2);
      const bool has = g.own > 0.f;
      const unsigned over = __ballot_sync(0xffffffffu, has && (hit_run + g.incl > t));
      const unsigned any = __ballot_sync(0xffffffffu, has);
      const int src = over ? (__ffs(over) - 1) : (31 - __clz(any));
      if (lane == src) {
        float e = 0.f;
        int choice = -1, lastnz = -1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          e = j == 0 ? g.a[0] : e + g.a[j];
          if (g.a[j] > 0.f) {
            lastnz = j;
            if (choice < 0 && hit_run + (g.excl + e) > t) choice = j;
          }
        }
        if (choice < 0) choice = lastnz;
        out[size_t(row) * num_samples + smp] = int64_t(hit) * kSampGroup + lane * 4 + choice;
      }
    }
    __syncthreads();
  }
}

// ---- fused sampler: temperature, top-k, top-p and the draw ------------------------------------------------------
// The k largest logits of every row (largest first, from topk_f32) are turned into weights
// e_r = exp((v_r - v_0) / T); rank r is kept while the running sum BEFORE it stays below top_p times the sum
// of all k (the set HuggingFace's temperature -> top-k -> top-p warpers keep, ranks taken largest first; rank 0
// is always kept); one Philox draw u (counter = (offset, row, 0), key = seed) picks the first kept rank whose
// running sum exceeds u times the kept sum.  Running sums are taken in a fixed order so that a CPU restatement
// reproduces them: 4 ranks per lane left to right, an inclusive Hillis-Steele scan over the lanes of a 128-rank
// group, groups added left to right; incl_r = (base of the group + sum of the lanes before) + sum inside the lane.
constexpr int kPickThreads = 256;                 // 8 groups of 128 ranks: k <= 1024

__global__ void __launch_bounds__(kPickThreads)
sample_pick_kernel(uint32_t k, const float* __restrict__ vals, const int64_t* __restrict__ idx, float inv_t, float top_p,
                   int64_t* __restrict__ out, float* __restrict__ out_prob, uint32_t seed_lo, uint32_t seed_hi, uint32_t off_lo,
                   uint32_t off_hi) {
  __shared__ float group_sum[kPickThreads / 32];
  __shared__ float group_base[kPickThreads / 32 + 1];
  __shared__ unsigned int kept_n, pick_r, last_r;
  __shared__ float kept_sum;
  const uint32_t row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_trigger();
  const float* v = vals + size_t(row) * k;
  const float v0 = v[0];
  if (tid == 0) { kept_n = 0; pick_r = 0xFFFFFFFFu; last_r = 0; }
  float a[4], run[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t r = uint32_t(tid) * 4 + j;
    float e = 0.f;
    if (r < k) {
      const float x = v[r];
      // the largest logit itself weighs 1 whatever it is (an infinite or NaN maximum would give inf - inf)
      e = (r == 0) ? 1.f : expf((x - v0) * inv_t);
      if (!(e >= 0.f) || e > 3.402823466e38f) e = 0.f;
    }
    a[j] = e;
    run[j] = j == 0 ? e : run[j - 1] + e;
  }
  float incl = run[3];
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  const float prev = __shfl_up_sync(0xffffffffu, incl, 1);
  const float lane_excl = lane == 0 ? 0.f : prev;
  if (lane == 31) group_sum[warp] = incl;
  __syncthreads();
  if (tid == 0) {
    float b = 0.f;
    for (int g = 0; g < kPickThreads / 32; ++g) { group_base[g] = b; b += group_sum[g]; }
    group_base[kPickThreads / 32] = b;
  }
  __syncthreads();
  const float total = group_base[kPickThreads / 32];
  const float before = group_base[warp] + lane_excl;            // running sum before this lane's first rank
  const float cut = __fmul_rn(top_p, total);
  // the kept ranks are a prefix: count them
  unsigned int mine = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t r = uint32_t(tid) * 4 + j;
    const float excl_r = j == 0 ? before : before + run[j - 1];
    if (r < k && (r == 0 || excl_r < cut)) ++mine;
  }
  if (mine) atomicAdd(&kept_n, mine);
  __syncthreads();
  const uint32_t R = kept_n;                                    // >= 1
  if ((R - 1) / 4 == uint32_t(tid)) kept_sum = before + run[(R - 1) & 3];
  __syncthreads();
  const float K = kept_sum;
  uint32_t x[4];
  philox4x32_10(off_lo, off_hi, row, 0u, seed_lo, seed_hi, x);
  const float u = float(x[0] >> 8) * 5.9604644775390625e-08f;
  const float t = __fmul_rn(u, K);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t r = uint32_t(tid) * 4 + j;
    if (r < R && a[j] > 0.f) {
      atomicMax(&last_r, r);
      if (before + run[j] > t) atomicMin(&pick_r, r);
    }
  }
  __syncthreads();
  if (tid == 0) {
    const uint32_t r = pick_r != 0xFFFFFFFFu ? pick_r : last_r;
    out[row] = idx[size_t(row) * k + r];
  }
  if (out_prob != nullptr) {
    const uint32_t r = pick_r != 0xFFFFFFFFu ? pick_r : last_r;
    if (r / 4 == uint32_t(tid)) out_prob[row] = K > 0.f ? a[r & 3] / K : 1.f;
  }
}

}  // namespace kuiops

using namespace kuiops;

extern "C" {

int kuiops_multinomial_f32(uint32_t m, uint32_t n, uint32_t num_samples, const void* probs, int64_t* out, uint64_t seed,
                           uint64_t offset, int* status, kuiops_stream_t s) {
  if (m == 0 || n == 0 || num_samples == 0 || !probs || !out) return KUIOPS_EINVAL;
  if (uint64_t(m) * n > (1ull << 31) || m > 0x7FFFFFFFu || num_samples > 4096) return KUIOPS_ELIMIT;
  return launch_pdl(multinomial_rows_kernel, dim3(m), dim3(kSampThreads), 0, as_stream(s), n, num_samples,
                    static_cast<const float*>(probs), out, uint32_t(seed), uint32_t(seed >> 32), uint32_t(offset),
                    uint32_t(offset >> 32), status);
}

size_t kuiops_sample_workspace_bytes(uint32_t m, uint32_t top_k) { return size_t(m) * top_k * 12 + 256; }

int kuiops_sample_topk_topp_f32(uint32_t m, uint32_t n, const void* logits, float temperature, uint32_t top_k, float top_p,
                                uint64_t seed, uint64_t offset, int64_t* out, float* out_prob, void* workspace,
                                size_t workspace_bytes, kuiops_stream_t s) {
  if (m == 0 || n == 0 || !logits || !out) return KUIOPS_EINVAL;
  if (!(temperature > 0.f) || !(top_p > 0.f) || top_p > 1.f || top_k == 0) return KUIOPS_EINVAL;
  const uint32_t k = top_k < n ? top_k : n;
  if (k > 4u * kPickThreads) return KUIOPS_ELIMIT;
  if (!workspace || workspace_bytes < kuiops_sample_workspace_bytes(m, k) || (reinterpret_cast<uintptr_t>(workspace) & 15u))
    return KUIOPS_EWORKSPACE;
  // [m, k] int64 indices first (8-byte aligned), then the [m, k] values
  int64_t* idx = static_cast<int64_t*>(workspace);
  float* vals = reinterpret_cast<float*>(idx + size_t(m) * k);
  const int rc = kuiops_topk_f32(m, n, k, logits, vals, idx, s);
  if (rc != KUIOPS_OK) return rc;
  return launch_pdl(sample_pick_kernel, dim3(m), dim3(kPickThreads), 0, as_stream(s), k, static_cast<const float*>(vals),
                    static_cast<const int64_t*>(idx), 1.f / temperature, top_p, out, out_prob, uint32_t(seed), uint32_t(seed >> 32),
                    uint32_t(offset), uint32_t(offset >> 32));
}

}  // extern "C"
