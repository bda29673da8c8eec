// Elementwise maps and the fused decoder-layer helpers built from them.
// One launch per map, 16-byte accesses, grid sized in whole multiples of the SM count.
#include "common.cuh"
#include "gemm.cuh"
#include "tc_ptx.cuh"

namespace kuiops {

// --------------------------------------------------------------------------------------
// The map family.  The reference instantiates one kernel per lambda and bakes scalar
// constants into it (kuipy/kuiops.py:292-296, kuiops/elementwise/Kuiops.Elementwise.fsti);
// here OP is a template parameter and the constants are kernel arguments.  Arithmetic is
// done in fp32 and rounded once to the element type, which is what eager PyTorch does for
// bf16/f16 tensors.
// --------------------------------------------------------------------------------------
template <int OP>
__device__ __forceinline__ float map_apply(float x, float y, float c1) {
  // y is the second operand (tensor element or the scalar c0); c1 is alpha of add/sub
  if (OP == KUIOPS_MAP_SILU) return __fdividef(x, 1.f + __expf(-x));     // special-function unit: exp2 and reciprocal, no division sequence
  if (OP == KUIOPS_MAP_NEG) return -x;
  if (OP == KUIOPS_MAP_RSQRT) return 1.f / sqrtf(x);
  if (OP == KUIOPS_MAP_COS) return cosf(x);
  if (OP == KUIOPS_MAP_SIN) return sinf(x);
  if (OP == KUIOPS_MAP_POW) return powf(x, y);
  if (OP == KUIOPS_MAP_SQUARE) return x * x;
  if (OP == KUIOPS_MAP_ADD) return x + c1 * y;
  if (OP == KUIOPS_MAP_MUL) return x * y;
  if (OP == KUIOPS_MAP_SUB) return x - c1 * y;
  if (OP == KUIOPS_MAP_DIV) return x / y;
  if (OP == KUIOPS_MAP_GELU) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  return x;
}

template <typename T, int OP, bool BINARY>
__global__ void __launch_bounds__(256)
map_kernel(uint64_t len, const T* X, const T* B, T* Y, float c0, float c1, int vec_ok) {
  constexpr int VN = Vec16<T>::N;
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  if (vec_ok) {
    const uint64_t nvec = len / VN;
    for (uint64_t v = gt; v < nvec; v += gs) {
      Vec16<T> a = ld16(X + v * VN), b, o;
      if (BINARY) b = ld16(B + v * VN);
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        float y = BINARY ? ElemTraits<T>::to_f(b.v[e]) : c0;
        o.v[e] = ElemTraits<T>::from_f(map_apply<OP>(ElemTraits<T>::to_f(a.v[e]), y, c1));
      }
      st16(Y + v * VN, o);
    }
    for (uint64_t i = nvec * VN + gt; i < len; i += gs) {
      float y = BINARY ? ElemTraits<T>::to_f(B[i]) : c0;
      Y[i] = ElemTraits<T>::from_f(map_apply<OP>(ElemTraits<T>::to_f(X[i]), y, c1));
    }
  } else {
    for (uint64_t i = gt; i < len; i += gs) {
      float y = BINARY ? ElemTraits<T>::to_f(B[i]) : c0;
      Y[i] = ElemTraits<T>::from_f(map_apply<OP>(ElemTraits<T>::to_f(X[i]), y, c1));
    }
  }
}

template <typename T, int OP, bool BINARY>
static int map_launch_op(uint64_t len, const void* X, const void* B, void* Y, double c0, double c1, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = aligned16(X) && aligned16(Y) && (!BINARY || aligned16(B));
  unsigned grid = stream_grid((len + VN - 1) / VN, 256 * 2, 16);
  map_kernel<T, OP, BINARY><<<grid, 256, 0, st>>>(len, static_cast<const T*>(X), static_cast<const T*>(B),
                                                   static_cast<T*>(Y), float(c0), float(c1), vec_ok);
  return check_launch();
}

template <typename T, bool BINARY>
static int map_launch(int op, uint64_t len, const void* X, const void* B, void* Y, double c0, double c1, cudaStream_t st) {
  if (len == 0 || !X || !Y || (BINARY && !B)) return KUIOPS_EINVAL;
#define KUIOPS_CASE(OPC) case OPC: return map_launch_op<T, OPC, BINARY>(len, X, B, Y, c0, c1, st);
  if (BINARY) {
    switch (op) {
      KUIOPS_CASE(KUIOPS_MAP_ADD) KUIOPS_CASE(KUIOPS_MAP_MUL) KUIOPS_CASE(KUIOPS_MAP_SUB) KUIOPS_CASE(KUIOPS_MAP_DIV)
      KUIOPS_CASE(KUIOPS_MAP_POW)
      default: return KUIOPS_EUNSUPPORTED;
    }
  }
  switch (op) {
    KUIOPS_CASE(KUIOPS_MAP_SILU) KUIOPS_CASE(KUIOPS_MAP_NEG) KUIOPS_CASE(KUIOPS_MAP_RSQRT) KUIOPS_CASE(KUIOPS_MAP_COS)
    KUIOPS_CASE(KUIOPS_MAP_SIN) KUIOPS_CASE(KUIOPS_MAP_POW) KUIOPS_CASE(KUIOPS_MAP_SQUARE) KUIOPS_CASE(KUIOPS_MAP_ADD)
    KUIOPS_CASE(KUIOPS_MAP_MUL) KUIOPS_CASE(KUIOPS_MAP_SUB) KUIOPS_CASE(KUIOPS_MAP_DIV) KUIOPS_CASE(KUIOPS_MAP_GELU)
    default: return KUIOPS_EUNSUPPORTED;
  }
#undef KUIOPS_CASE
}

// bool-byte maps, 16 bytes at a time
template <int OP>
__global__ void __launch_bounds__(256)
map_u8_kernel(uint64_t len, const uint8_t* X, const uint8_t* B, uint8_t* Y, int vec_ok) {
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  auto f = [](uint8_t a, uint8_t b) -> uint8_t {
    if (OP == KUIOPS_MAP_BNOT) return a ? 0 : 1;
    if (OP == KUIOPS_MAP_BAND) return (a && b) ? 1 : 0;
    return (a || b) ? 1 : 0;
  };
  uint64_t start = 0;
  if (vec_ok) {
    const uint64_t nvec = len / 16;
    for (uint64_t v = gt; v < nvec; v += gs) {
      Vec16<uint8_t> a = ld16(X + v * 16), b = a, o;
      if (OP != KUIOPS_MAP_BNOT) b = ld16(B + v * 16);
#pragma unroll
      for (int e = 0; e < 16; ++e) o.v[e] = f(a.v[e], b.v[e]);
      st16(Y + v * 16, o);
    }
    start = nvec * 16;
  }
  for (uint64_t i = start + gt; i < len; i += gs) Y[i] = f(X[i], OP != KUIOPS_MAP_BNOT ? B[i] : 0);
}

// float in -> bool byte out
template <typename T, int OP>
__global__ void __launch_bounds__(256)
map_nip_kernel(uint64_t len, const T* __restrict__ X, uint8_t* __restrict__ Y, float c0) {
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = gt; i < len; i += gs) {
    float x = ElemTraits<T>::to_f(X[i]);
    bool r = OP == KUIOPS_MAP_EQ ? (x == c0) : (OP == KUIOPS_MAP_LE ? (x <= c0) : (x < c0));
    Y[i] = r ? 1 : 0;
  }
}

template <typename T>
static int map_nip_launch(int op, uint64_t len, const void* X, void* Y, double c0, cudaStream_t st) {
  if (len == 0 || !X || !Y) return KUIOPS_EINVAL;
  unsigned grid = stream_grid(len, 256 * 4, 16);
  const T* x = static_cast<const T*>(X);
  uint8_t* y = static_cast<uint8_t*>(Y);
  switch (op) {
    case KUIOPS_MAP_EQ: map_nip_kernel<T, KUIOPS_MAP_EQ><<<grid, 256, 0, st>>>(len, x, y, float(c0)); break;
    case KUIOPS_MAP_LE: map_nip_kernel<T, KUIOPS_MAP_LE><<<grid, 256, 0, st>>>(len, x, y, float(c0)); break;
    case KUIOPS_MAP_LT: map_nip_kernel<T, KUIOPS_MAP_LT><<<grid, 256, 0, st>>>(len, x, y, float(c0)); break;
    default: return KUIOPS_EUNSUPPORTED;
  }
  return check_launch();
}

// where(cond, a, b) on raw payloads
template <typename P>
__global__ void __launch_bounds__(256)
where_kernel(uint64_t len, const uint8_t* __restrict__ cnd, const P* A, const P* B, P* Y) {
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = gt; i < len; i += gs) Y[i] = cnd[i] ? A[i] : B[i];
}

// --------------------------------------------------------------------------------------
// RMSNorm with optional residual add: the dispatcher sees this as
// to(f32) -> pow 2 -> mean -> add eps -> rsqrt -> mul -> to(bf16) -> mul weight, seven HBM
// round trips; fused it is one read and one write per row.  One to eight warps share a row of up
// to 1024 vectors, held in registers between the statistics and the scaling pass.
// --------------------------------------------------------------------------------------
template <typename T, int WPR>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(uint64_t m, uint32_t n, const T* __restrict__ x, const T* residual, const T* __restrict__ w,
               float eps, T* __restrict__ y, T* residual_out) {
  pdl_wait();
  pdl_trigger();
  // WPR warps share a row (1, 2, 4 or 8), each thread keeps at most 4 vectors of it in registers
  constexpr int VN = Vec16<T>::N, VECS = 4, RPB = 8 / WPR;
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row_in_block = warp / WPR, wsub = warp % WPR;
  const uint32_t nvec = n / VN;
  // the weights are the same for every row: requested once, up front, together with the first row
  Vec16<T> wv[VECS];
#pragma unroll
  for (int i = 0; i < VECS; ++i) {
    const uint32_t v = wsub * 32 + lane + i * (32 * WPR);
    if (v < nvec) wv[i] = ld16(w + size_t(v) * VN);
  }
  for (uint64_t base = uint64_t(blockIdx.x) * RPB; base < m; base += uint64_t(gridDim.x) * RPB) {
    const uint64_t row = base + row_in_block;
    const bool valid = row < m;
    const T* xr = x + row * n;
    Vec16<T> c[VECS];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const uint32_t v = wsub * 32 + lane + i * (32 * WPR);
      if (valid && v < nvec) {
        c[i] = ld16(xr + size_t(v) * VN);
        if (residual) {
          Vec16<T> r = ld16(residual + row * n + size_t(v) * VN);
#pragma unroll
          for (int e = 0; e < VN; ++e)
            c[i].v[e] = ElemTraits<T>::from_f(ElemTraits<T>::to_f(c[i].v[e]) + ElemTraits<T>::to_f(r.v[e]));
          st16(residual_out + row * n + size_t(v) * VN, c[i]);
        }
#pragma unroll
        for (int e = 0; e < VN; ++e) { float f = ElemTraits<T>::to_f(c[i].v[e]); ss += f * f; }
      }
    }
    ss = warp_sum(ss);
    if (WPR > 1) {
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      ss = 0.f;
#pragma unroll
      for (int k = 0; k < WPR; ++k) ss += red[row_in_block * WPR + k];
      __syncthreads();
    }
    const float r = rsqrtf(ss / float(n) + eps);
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const uint32_t v = wsub * 32 + lane + i * (32 * WPR);
      if (valid && v < nvec) {
        Vec16<T> o;
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          // torch's Llama RMSNorm rounds the normalised value to the element type before the weight multiply
          float nx = ElemTraits<T>::to_f(ElemTraits<T>::from_f(ElemTraits<T>::to_f(c[i].v[e]) * r));
          o.v[e] = ElemTraits<T>::from_f(nx * ElemTraits<T>::to_f(wv[i].v[e]));
        }
        st16(y + row * n + size_t(v) * VN, o);
      }
    }
  }
}

// RMSNorm whose input row is the sum of the partial rows that the ranks of a tensor-parallel group
// pushed into this rank's receive area (kuiops_gemm_push): the second half of the all-reduce, fused
// with the residual add and the normalisation that follow it.
//   x[row] = round_T( sum over r of slot(epoch & 1, r)[row] )   (fp32 sum in rank order)
//   resid_out[row] = x[row] + residual[row];  y[row] = rmsnorm(resid_out[row]) * w
// A slot holds 8-byte cells of two elements and a stamp; a cell belongs to the current exchange
// when its stamp is epoch + 1.  Every thread polls exactly the cells it is about to sum (for at
// most the wait limit, about 2 s unless lowered; then the error word is set and the kernel carries
// on with what it has), so there is no separate flag, and data that arrive early are consumed
// early.  The residual and the norm weights do not depend on the peers and are requested before
// the polling starts.  The last CTA advances the epoch.
__device__ __forceinline__ uint4 ld_volatile_u4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t elementwise_global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <typename T, int WPR>
__global__ void __launch_bounds__(256)
rmsnorm_gather_kernel(uint64_t m, uint32_t n, uint32_t n_ranks, const unsigned char* recv_base, uint64_t slot_bytes,
                      unsigned int* epoch, unsigned int* ticket, unsigned int* err, uint64_t wait_ns,
                      unsigned long long* trace, const T* residual, const T* __restrict__ w, float eps, T* __restrict__ y, T* residual_out) {
  static_assert(sizeof(T) == 2, "cells hold two 16-bit elements");
  if (trace && blockIdx.x == 0 && threadIdx.x == 0) trace[12] = elementwise_global_ns();       // CTA started
  pdl_wait();
  pdl_trigger();
  constexpr int VN = Vec16<T>::N, VECS = 4, RPB = 8 / WPR;
  __shared__ float red[8];
  const unsigned int e = *reinterpret_cast<volatile unsigned int*>(epoch);
  const unsigned int want = e + 1u;
  if (trace && blockIdx.x == 0 && threadIdx.x == 0) trace[13] = elementwise_global_ns();       // predecessor complete
  const unsigned char* slots = recv_base + size_t(e & 1u) * n_ranks * slot_bytes;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row_in_block = warp / WPR, wsub = warp % WPR;
  const uint32_t nvec = n / VN;
  bool timed_out = false;
  uint64_t t0 = 0;
  for (uint64_t base = uint64_t(blockIdx.x) * RPB; base < m; base += uint64_t(gridDim.x) * RPB) {
    const uint64_t row = base + row_in_block;
    const bool valid = row < m;
    Vec16<T> c[VECS], res[VECS], wv[VECS];
    // what does not come from the peers first: residual and weights
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const uint32_t v = wsub * 32 + lane + i * (32 * WPR);
      if (valid && v < nvec) {
        res[i] = ld16(residual + row * n + size_t(v) * VN);
        wv[i] = ld16(w + size_t(v) * VN);
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const uint32_t v = wsub * 32 + lane + i * (32 * WPR);
      if (valid && v < nvec) {
        float acc[VN];
#pragma unroll
        for (int k = 0; k < VN; ++k) acc[k] = 0.f;
        // 8 elements = 4 cells = 32 bytes per rank, written by another GPU.  The requests for all ranks go
        // out together (volatile reads); whatever does not carry the stamp yet is read again until it does.
        const unsigned char* cell0 = slots + (row * n + size_t(v) * VN) * 4;
        uint4 a[KUIOPS_MAX_PEERS], b[KUIOPS_MAX_PEERS];
#pragma unroll
        for (int r = 0; r < KUIOPS_MAX_PEERS; ++r) {
          if (uint32_t(r) < n_ranks) { a[r] = ld_volatile_u4(cell0 + r * slot_bytes); b[r] = ld_volatile_u4(cell0 + r * slot_bytes + 16); }
        }
#pragma unroll
        for (int r = 0; r < KUIOPS_MAX_PEERS; ++r) {
          if (uint32_t(r) < n_ranks) {
            while ((a[r].y != want || a[r].w != want || b[r].y != want || b[r].w != want) && !timed_out) {
              if (t0 == 0) t0 = elementwise_global_ns();
              if (elementwise_global_ns() - t0 > wait_ns) { timed_out = true; break; }
              a[r] = ld_volatile_u4(cell0 + r * slot_bytes); b[r] = ld_volatile_u4(cell0 + r * slot_bytes + 16);
            }
            const uint32_t words[4] = {a[r].x, a[r].z, b[r].x, b[r].z};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const T lo = *reinterpret_cast<const T*>(&words[q]);
              const T hi = *(reinterpret_cast<const T*>(&words[q]) + 1);
              acc[2 * q] += ElemTraits<T>::to_f(lo);
              acc[2 * q + 1] += ElemTraits<T>::to_f(hi);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < VN; ++k) {
          const float x = ElemTraits<T>::to_f(ElemTraits<T>::from_f(acc[k]));      // the all-reduce result, rounded as a stored tensor would be
          c[i].v[k] = ElemTraits<T>::from_f(x + ElemTraits<T>::to_f(res[i].v[k]));
        }
        st16(residual_out + row * n + size_t(v) * VN, c[i]);
#pragma unroll
        for (int k = 0; k < VN; ++k) { float f = ElemTraits<T>::to_f(c[i].v[k]); ss += f * f; }
      }
    }
    if (trace && blockIdx.x == 0 && threadIdx.x == 0) trace[14] = elementwise_global_ns();     // this thread's cells of every rank have arrived
    ss = warp_sum(ss);
    if (WPR > 1) {
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      ss = 0.f;
#pragma unroll
      for (int k = 0; k < WPR; ++k) ss += red[row_in_block * WPR + k];
      __syncthreads();
    }
    const float rs = rsqrtf(ss / float(n) + eps);
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const uint32_t v = wsub * 32 + lane + i * (32 * WPR);
      if (valid && v < nvec) {
        Vec16<T> o;
#pragma unroll
        for (int k = 0; k < VN; ++k) {
          float nx = ElemTraits<T>::to_f(ElemTraits<T>::from_f(ElemTraits<T>::to_f(c[i].v[k]) * rs));
          o.v[k] = ElemTraits<T>::from_f(nx * ElemTraits<T>::to_f(wv[i].v[k]));
        }
        st16(y + row * n + size_t(v) * VN, o);
      }
    }
  }
  if (timed_out) atomicExch(err, 30u);
  // every CTA read the epoch before it got here; the last one moves it on for the next exchange
  __syncthreads();
  if (trace && blockIdx.x == 0 && threadIdx.x == 0) trace[15] = elementwise_global_ns();       // rows summed, normalised, stored
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      atomicExch(ticket, 0u);
      atomicAdd(epoch, 1u);
    }
  }
}

// silu(gate) * up over a fused [m, 2n] gate|up activation
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(uint64_t m, uint32_t n, const T* __restrict__ gu, T* __restrict__ y) {
  pdl_wait();
  pdl_trigger();
  constexpr int VN = Vec16<T>::N;
  const uint32_t nvec = n / VN;
  const uint64_t total = m * nvec;
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t t = gt; t < total; t += gs) {
    const uint64_t row = t / nvec, v = t % nvec;
    Vec16<T> g = ld16(gu + row * 2 * n + v * VN), u = ld16(gu + row * 2 * n + n + v * VN), o;
#pragma unroll
    for (int e = 0; e < VN; ++e) {
      float gf = ElemTraits<T>::to_f(g.v[e]);
      float s = ElemTraits<T>::to_f(ElemTraits<T>::from_f(__fdividef(gf, 1.f + __expf(-gf))));   // silu rounded as eager does
      o.v[e] = ElemTraits<T>::from_f(s * ElemTraits<T>::to_f(u.v[e]));
    }
    st16(y + row * n + v * VN, o);
  }
}

// Rotary embedding on the q and k heads of packed qkv rows, plus the KV-cache append.
// One thread handles the (i, i + d/2) pair group of 8 elements from each half of `hpt` consecutive
// heads of one row: the angles depend only on (row, i), so their sines and cosines (the expensive
// part: accurate range reduction for positions in the thousands) are computed once and reused over
// those heads.  hpt is 1 for decode-sized calls (parallelism matters) and 8 for prefill.
template <typename T>
__global__ void __launch_bounds__(256)
rope_qkv_kernel(uint64_t rows, uint32_t hq, uint32_t hk, uint32_t d, T* qkv, int64_t row_stride,
                const int64_t* __restrict__ positions, float log2_theta, T* k_cache, T* v_cache,
                uint64_t cache_cap, uint32_t rows_per_seq, uint32_t hpt) {
  pdl_wait();
  pdl_trigger();
  constexpr int VN = Vec16<T>::N;
  const uint32_t half = d / 2, vec_per_half = half / VN;
  const uint32_t heads = hq + 2 * hk;                 // q heads, k heads, v heads
  const uint32_t groups = (heads + hpt - 1) / hpt;
  const uint64_t total = rows * groups * vec_per_half;
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t t = gt; t < total; t += gs) {
    const uint32_t v = t % vec_per_half;
    const uint32_t group = (t / vec_per_half) % groups;
    const uint64_t row = t / (uint64_t(vec_per_half) * groups);
    const int64_t pos = positions[row];
    const uint32_t h0 = group * hpt, h1 = min(h0 + hpt, heads);
    // eager computes cos / sin in fp32 and rounds them to the element type
    float csr[VN], snr[VN];
    if (h0 < hq + hk) {
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        const float fi = float(v * VN + e);
        // inv_freq = theta^(-2i/d); angle = pos * inv_freq
        const float inv_freq = exp2f(-log2_theta * (2.f * fi / float(d)));
        float sn, cs;
        sincosf(float(pos) * inv_freq, &sn, &cs);
        csr[e] = ElemTraits<T>::to_f(ElemTraits<T>::from_f(cs));
        snr[e] = ElemTraits<T>::to_f(ElemTraits<T>::from_f(sn));
      }
    }
    for (uint32_t head = h0; head < h1; ++head) {
      T* base = qkv + row * row_stride + size_t(head) * d;
      Vec16<T> lo = ld16(base + v * VN), hi = ld16(base + half + v * VN);
      if (head < hq + hk) {
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          // eager computes q*cos and rotate_half(q)*sin in the element type, then adds
          const float a = ElemTraits<T>::to_f(lo.v[e]), b = ElemTraits<T>::to_f(hi.v[e]);
          const float a_c = ElemTraits<T>::to_f(ElemTraits<T>::from_f(a * csr[e]));
          const float b_s = ElemTraits<T>::to_f(ElemTraits<T>::from_f(-b * snr[e]));
          const float b_c = ElemTraits<T>::to_f(ElemTraits<T>::from_f(b * csr[e]));
          const float a_s = ElemTraits<T>::to_f(ElemTraits<T>::from_f(a * snr[e]));
          lo.v[e] = ElemTraits<T>::from_f(a_c + b_s);
          hi.v[e] = ElemTraits<T>::from_f(b_c + a_s);
        }
        if (head < hq || k_cache == nullptr) {
          st16(base + v * VN, lo);
          st16(base + half + v * VN, hi);
        }
      }
      if (head >= hq && k_cache != nullptr) {
        const bool is_k = head < hq + hk;
        const uint32_t kvh = is_k ? head - hq : head - hq - hk;
        const uint64_t seq = row / rows_per_seq;
        T* dst = (is_k ? k_cache : v_cache) + ((seq * hk + kvh) * cache_cap + uint64_t(pos)) * d;
        if (uint64_t(pos) < cache_cap) {
          st16(dst + v * VN, lo);
          st16(dst + half + v * VN, hi);
        }
        if (is_k) {   // keep the packed row consistent too (prefill attention reads it)
          st16(base + v * VN, lo);
          st16(base + half + v * VN, hi);
        }
      }
    }
  }
}

template <typename P>
__global__ void __launch_bounds__(256)
embedding_kernel(uint64_t rows, uint64_t width_p, uint64_t vocab, const P* __restrict__ table,
                 const int64_t* __restrict__ ids, P* __restrict__ out, int32_t* status) {
  pdl_wait();
  pdl_trigger();
  const uint64_t total = rows * width_p;
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t t = gt; t < total; t += gs) {
    const uint64_t row = t / width_p, c = t % width_p;
    const int64_t id = ids[row];
    if (id < 0 || uint64_t(id) >= vocab) {
      if (status && c == 0) atomicExch(status, 1);
      continue;
    }
    out[t] = table[uint64_t(id) * width_p + c];
  }
}

// x[i] += delta over int64 (position counters kept on the device between captured decode steps)
__global__ void __launch_bounds__(256)
add_i64_kernel(uint64_t len, long long* x, long long delta) {
  pdl_wait();
  pdl_trigger();
  const uint64_t gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < len; i += gs) x[i] += delta;
}

}  // namespace kuiops

using namespace kuiops;

extern "C" {

int kuiops_map(int dtype, int op, uint64_t len, const void* X, void* Y, double c0, double c1, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_F32: return map_launch<float, false>(op, len, X, nullptr, Y, c0, c1, as_stream(s));
    case KUIOPS_BF16: return map_launch<__nv_bfloat16, false>(op, len, X, nullptr, Y, c0, c1, as_stream(s));
    case KUIOPS_F16: return map_launch<__half, false>(op, len, X, nullptr, Y, c0, c1, as_stream(s));
  }
  return KUIOPS_EINVAL;
}

int kuiops_add_i64(uint64_t len, int64_t* x, int64_t delta, kuiops_stream_t s) {
  if (len == 0 || !x) return KUIOPS_EINVAL;
  return launch_pdl(add_i64_kernel, dim3(stream_grid(len, 256, 8)), dim3(256), 0, as_stream(s), len, reinterpret_cast<long long*>(x), (long long)delta);
}

int kuiops_map2(int dtype, int op, uint64_t len, const void* X, const void* B, void* Y, double c1, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_F32: return map_launch<float, true>(op, len, X, B, Y, 0.0, c1, as_stream(s));
    case KUIOPS_BF16: return map_launch<__nv_bfloat16, true>(op, len, X, B, Y, 0.0, c1, as_stream(s));
    case KUIOPS_F16: return map_launch<__half, true>(op, len, X, B, Y, 0.0, c1, as_stream(s));
  }
  return KUIOPS_EINVAL;
}

int kuiops_map_u8(int op, uint64_t len, const void* X, const void* B, void* Y, kuiops_stream_t s) {
  if (len == 0 || !X || !Y) return KUIOPS_EINVAL;
  if (op != KUIOPS_MAP_BNOT && !B) return KUIOPS_EINVAL;
  const int vec_ok = aligned16(X) && aligned16(Y) && (op == KUIOPS_MAP_BNOT || aligned16(B));
  unsigned grid = stream_grid((len + 15) / 16, 256 * 2, 16);
  auto* x = static_cast<const uint8_t*>(X);
  auto* b = static_cast<const uint8_t*>(B);
  auto* y = static_cast<uint8_t*>(Y);
  switch (op) {
    case KUIOPS_MAP_BNOT: map_u8_kernel<KUIOPS_MAP_BNOT><<<grid, 256, 0, as_stream(s)>>>(len, x, b, y, vec_ok); break;
    case KUIOPS_MAP_BAND: map_u8_kernel<KUIOPS_MAP_BAND><<<grid, 256, 0, as_stream(s)>>>(len, x, b, y, vec_ok); break;
    case KUIOPS_MAP_BOR: map_u8_kernel<KUIOPS_MAP_BOR><<<grid, 256, 0, as_stream(s)>>>(len, x, b, y, vec_ok); break;
    default: return KUIOPS_EUNSUPPORTED;
  }
  return check_launch();
}

int kuiops_map_nip(int dtype, int op, uint64_t len, const void* X, void* Y, double c0, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_F32: return map_nip_launch<float>(op, len, X, Y, c0, as_stream(s));
    case KUIOPS_BF16: return map_nip_launch<__nv_bfloat16>(op, len, X, Y, c0, as_stream(s));
    case KUIOPS_F16: return map_nip_launch<__half>(op, len, X, Y, c0, as_stream(s));
  }
  return KUIOPS_EINVAL;
}

int kuiops_map3(uint32_t elem_bytes, uint64_t len, const void* cond, const void* A, const void* B, void* Y,
                kuiops_stream_t s) {
  if (len == 0 || !cond || !A || !B || !Y) return KUIOPS_EINVAL;
  unsigned grid = stream_grid(len, 256 * 4, 16);
  auto* c = static_cast<const uint8_t*>(cond);
  cudaStream_t st = as_stream(s);
  switch (elem_bytes) {
    case 1: where_kernel<uint8_t><<<grid, 256, 0, st>>>(len, c, (const uint8_t*)A, (const uint8_t*)B, (uint8_t*)Y); break;
    case 2: where_kernel<uint16_t><<<grid, 256, 0, st>>>(len, c, (const uint16_t*)A, (const uint16_t*)B, (uint16_t*)Y); break;
    case 4: where_kernel<uint32_t><<<grid, 256, 0, st>>>(len, c, (const uint32_t*)A, (const uint32_t*)B, (uint32_t*)Y); break;
    case 8: where_kernel<uint64_t><<<grid, 256, 0, st>>>(len, c, (const uint64_t*)A, (const uint64_t*)B, (uint64_t*)Y); break;
    default: return KUIOPS_EINVAL;
  }
  return check_launch();
}

}  // extern "C"
template <typename T>
static int rmsnorm_launch(uint64_t m, uint32_t n, const void* x, const void* res, const void* w, float eps, void* y,
                          void* res_out, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  if (m == 0 || n == 0 || !x || !w || !y) return KUIOPS_EINVAL;
  if (res && !res_out) return KUIOPS_EINVAL;
  if (n % VN || !aligned16(x) || !aligned16(w) || !aligned16(y) || (res && (!aligned16(res) || !aligned16(res_out))))
    return KUIOPS_EUNSUPPORTED;
  const uint32_t nvec = n / VN;
  auto X = static_cast<const T*>(x); auto R = static_cast<const T*>(res); auto W = static_cast<const T*>(w);
  auto Y = static_cast<T*>(y); auto RO = static_cast<T*>(res_out);
  // warps per row so that a thread holds at most 4 vectors
  if (nvec <= 128) return launch_pdl(rmsnorm_kernel<T, 1>, dim3(stream_grid(m, 8, 16)), dim3(256), 0, st, m, n, X, R, W, eps, Y, RO);
  if (nvec <= 256) return launch_pdl(rmsnorm_kernel<T, 2>, dim3(stream_grid(m, 4, 16)), dim3(256), 0, st, m, n, X, R, W, eps, Y, RO);
  if (nvec <= 512) return launch_pdl(rmsnorm_kernel<T, 4>, dim3(stream_grid(m, 2, 16)), dim3(256), 0, st, m, n, X, R, W, eps, Y, RO);
  if (nvec <= 1024) return launch_pdl(rmsnorm_kernel<T, 8>, dim3(stream_grid(m, 1, 16)), dim3(256), 0, st, m, n, X, R, W, eps, Y, RO);
  return KUIOPS_EUNSUPPORTED;
}

template <typename T>
static int rmsnorm_gather_launch(uint64_t m, uint32_t n, uint32_t n_ranks, const void* base, uint64_t slot_bytes,
                                 uint32_t* epoch, uint32_t* ticket, const void* res, const void* w, float eps, void* y,
                                 void* res_out, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  if (m == 0 || n == 0 || !base || !epoch || !ticket || !res || !w || !y || !res_out) return KUIOPS_EINVAL;
  if (n_ranks < 2 || n_ranks > KUIOPS_MAX_PEERS) return KUIOPS_EINVAL;
  if (slot_bytes < m * n * 4 || (slot_bytes & 15u)) return KUIOPS_EINVAL;
  if (n % VN || !aligned16(base) || !aligned16(res) || !aligned16(w) || !aligned16(y) || !aligned16(res_out)) return KUIOPS_EUNSUPPORTED;
  unsigned int* err = tc_error_word_device();
  if (!err) return KUIOPS_ELAUNCH;
  const uint32_t nvec = n / VN;
  auto B = static_cast<const unsigned char*>(base);
  auto R = static_cast<const T*>(res); auto W = static_cast<const T*>(w);
  auto Y = static_cast<T*>(y); auto RO = static_cast<T*>(res_out);
#define KUIOPS_RG(WPRV, RPBV) \
  return launch_pdl(rmsnorm_gather_kernel<T, WPRV>, dim3(stream_grid(m, RPBV, 16)), dim3(256), 0, st, m, n, n_ranks, B, slot_bytes, \
                    epoch, ticket, err, g_peer_wait_ns.load(std::memory_order_relaxed), \
                    g_gemm_trace.load(std::memory_order_relaxed), R, W, eps, Y, RO)
  // decode-sized steps are latency bound: spread a row over as many warps as it has vectors for, one row per CTA
  if (m <= 128 && nvec > 128 && nvec <= 1024) KUIOPS_RG(8, 1);
  if (nvec <= 128) KUIOPS_RG(1, 8);
  if (nvec <= 256) KUIOPS_RG(2, 4);
  if (nvec <= 512) KUIOPS_RG(4, 2);
  if (nvec <= 1024) KUIOPS_RG(8, 1);
#undef KUIOPS_RG
  return KUIOPS_EUNSUPPORTED;
}

extern "C" {
int kuiops_rmsnorm_gather(int dtype, uint64_t m, uint32_t n, uint32_t n_ranks, const void* recv_base, uint64_t slot_bytes,
                          uint32_t* epoch, uint32_t* ticket, const void* residual, const void* weight,
                          float eps, void* y, void* residual_out, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_BF16: return rmsnorm_gather_launch<__nv_bfloat16>(m, n, n_ranks, recv_base, slot_bytes, epoch, ticket,
                                                                  residual, weight, eps, y, residual_out, as_stream(s));
    case KUIOPS_F16: return rmsnorm_gather_launch<__half>(m, n, n_ranks, recv_base, slot_bytes, epoch, ticket,
                                                          residual, weight, eps, y, residual_out, as_stream(s));
  }
  return KUIOPS_EUNSUPPORTED;
}
}  // extern "C"

extern "C" {
int kuiops_rmsnorm(int dtype, uint64_t m, uint32_t n, const void* x, const void* residual, const void* weight,
                   float eps, void* y, void* residual_out, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_F32: return rmsnorm_launch<float>(m, n, x, residual, weight, eps, y, residual_out, as_stream(s));
    case KUIOPS_BF16: return rmsnorm_launch<__nv_bfloat16>(m, n, x, residual, weight, eps, y, residual_out, as_stream(s));
    case KUIOPS_F16: return rmsnorm_launch<__half>(m, n, x, residual, weight, eps, y, residual_out, as_stream(s));
  }
  return KUIOPS_EINVAL;
}

}  // extern "C"
template <typename T>
static int swiglu_launch(uint64_t m, uint32_t n, const void* gu, void* y, cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  if (m == 0 || n == 0 || !gu || !y) return KUIOPS_EINVAL;
  if (n % VN || !aligned16(gu) || !aligned16(y)) return KUIOPS_EUNSUPPORTED;
  unsigned grid = stream_grid(m * (n / VN), 256 * 2, 16);
  return launch_pdl(swiglu_kernel<T>, dim3(grid), dim3(256), 0, st, m, n, static_cast<const T*>(gu), static_cast<T*>(y));
}

extern "C" {
int kuiops_swiglu(int dtype, uint64_t m, uint32_t n, const void* gate_up, void* y, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_F32: return swiglu_launch<float>(m, n, gate_up, y, as_stream(s));
    case KUIOPS_BF16: return swiglu_launch<__nv_bfloat16>(m, n, gate_up, y, as_stream(s));
    case KUIOPS_F16: return swiglu_launch<__half>(m, n, gate_up, y, as_stream(s));
  }
  return KUIOPS_EINVAL;
}

}  // extern "C"
template <typename T>
static int rope_launch(uint64_t rows, uint32_t hq, uint32_t hk, uint32_t d, void* qkv, int64_t row_stride,
                       const int64_t* positions, float theta, void* kc, void* vc, uint64_t cap, uint32_t rps,
                       cudaStream_t st) {
  constexpr int VN = Vec16<T>::N;
  if (rows == 0 || hq == 0 || d == 0 || !qkv || !positions || theta <= 0.f) return KUIOPS_EINVAL;
  if ((kc == nullptr) != (vc == nullptr)) return KUIOPS_EINVAL;
  if (kc && (rps == 0 || cap == 0)) return KUIOPS_EINVAL;
  if (row_stride < int64_t(hq + 2 * hk) * d) return KUIOPS_EINVAL;
  if ((d / 2) % VN || d % 2 || row_stride % VN || !aligned16(qkv) || (kc && (!aligned16(kc) || !aligned16(vc))))
    return KUIOPS_EUNSUPPORTED;
  // heads per thread: share the sines and cosines of a row over eight heads once there are rows enough to fill the machine
  const uint32_t heads = hq + 2 * hk;
  const uint32_t hpt = rows * (heads / 8) * (d / 2 / VN) >= uint64_t(num_sms()) * 2048 ? 8u : 1u;
  const uint64_t total = rows * ((heads + hpt - 1) / hpt) * (d / 2 / VN);
  unsigned grid = stream_grid(total, 256, 16);
  return launch_pdl(rope_qkv_kernel<T>, dim3(grid), dim3(256), 0, st, rows, hq, hk, d, static_cast<T*>(qkv), row_stride,
                    positions, log2f(theta), static_cast<T*>(kc), static_cast<T*>(vc), cap, rps ? rps : 1u, hpt);
}

extern "C" {
int kuiops_rope_qkv(int dtype, uint64_t rows, uint32_t hq, uint32_t hk, uint32_t d, void* qkv, int64_t row_stride,
                    const int64_t* positions, float theta, void* k_cache, void* v_cache, uint64_t cache_cap,
                    uint32_t rows_per_seq, kuiops_stream_t s) {
  switch (dtype) {
    case KUIOPS_F32: return rope_launch<float>(rows, hq, hk, d, qkv, row_stride, positions, theta, k_cache, v_cache, cache_cap, rows_per_seq, as_stream(s));
    case KUIOPS_BF16: return rope_launch<__nv_bfloat16>(rows, hq, hk, d, qkv, row_stride, positions, theta, k_cache, v_cache, cache_cap, rows_per_seq, as_stream(s));
    case KUIOPS_F16: return rope_launch<__half>(rows, hq, hk, d, qkv, row_stride, positions, theta, k_cache, v_cache, cache_cap, rows_per_seq, as_stream(s));
  }
  return KUIOPS_EINVAL;
}

int kuiops_embedding(uint32_t elem_bytes, uint64_t rows, uint64_t width, uint64_t vocab, const void* table,
                     const int64_t* ids, void* out, int32_t* status, kuiops_stream_t s) {
  if (rows == 0 || width == 0 || vocab == 0 || !table || !ids || !out) return KUIOPS_EINVAL;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) return KUIOPS_EINVAL;
  const uint64_t row_bytes = width * elem_bytes;
  cudaStream_t st = as_stream(s);
  if (row_bytes % 16 == 0 && aligned16(table) && aligned16(out)) {
    const uint64_t wp = row_bytes / 16;
    unsigned grid = stream_grid(rows * wp, 256, 16);
    return launch_pdl(embedding_kernel<int4>, dim3(grid), dim3(256), 0, st, rows, wp, vocab, (const int4*)table, ids, (int4*)out, status);
  } else {
    unsigned grid = stream_grid(rows * row_bytes, 256, 16);
    return launch_pdl(embedding_kernel<uint8_t>, dim3(grid), dim3(256), 0, st, rows, row_bytes, vocab, (const uint8_t*)table, ids, (uint8_t*)out, status);
  }
}

}  // extern "C"

// --------------------------------------------------------------------------------------
// Data movement the dispatcher sees on every token next to the compute ops: dtype casts
// (aten._to_copy between the float types, aten.clone as the identity cast) and masked_fill with a
// scalar.  The reference lists them as backlog (KERNELS.md:46-48,68-90) and has no kernel.
// --------------------------------------------------------------------------------------
namespace kuiops {

template <typename TS, typename TD>
__global__ void __launch_bounds__(256)
cast_kernel(uint64_t len, const TS* __restrict__ X, TD* __restrict__ Y, int vec_ok) {
  // 8 elements per thread step: 16 or 32 bytes in, 16 or 32 bytes out, whichever type is wider
  const uint64_t gt = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x, gs = uint64_t(gridDim.x) * blockDim.x;
  uint64_t start = 0;
  if (vec_ok) {
    const uint64_t ngrp = len / 8;
    for (uint64_t g = gt; g < ngrp; g += gs) {
      TS in[8];
      TD out[8];
      if (sizeof(TS) == 2) *reinterpret_cast<int4*>(in) = __ldcs(reinterpret_cast<const int4*>(X + g * 8));
      else { reinterpret_cast<int4*>(in)[0] = __ldcs(reinterpret_cast<const int4*>(X + g * 8)); reinterpret_cast<int4*>(in)[1] = __ldcs(reinterpret_cast<const int4*>(X + g * 8) + 1); }
#pragma unroll
      for (int e = 0; e < 8; ++e) out[e] = ElemTraits<TD>::from_f(ElemTraits<TS>::to_f(in[e]));
      if (sizeof(TD) == 2) *reinterpret_cast<int4*>(Y + g * 8) = *reinterpret_cast<int4*>(out);
      else { reinterpret_cast<int4*>(Y + g * 8)[0] = reinterpret_cast<int4*>(out)[0]; reinterpret_cast<int4*>(Y + g * 8)[1] = reinterpret_cast<int4*>(out)[1]; }
    }
    start = ngrp * 8;
  }
  for (uint64_t i = start + gt; i < len; i += gs) Y[i] = ElemTraits<TD>::from_f(ElemTraits<TS>::to_f(X[i]));
}

template <typename TS, typename TD>
static int cast_launch(uint64_t len, const void* X, void* Y, cudaStream_t st) {
  const int vec_ok = aligned16(X) && aligned16(Y);
  const unsigned grid = stream_grid((len + 7) / 8, 256, 16);
  cast_kernel<TS, TD><<<grid, 256, 0, st>>>(len, static_cast<const TS*>(X), static_cast<TD*>(Y), vec_ok);
  return check_launch();
}

template <typename T>
__global__ void __launch_bounds__(256)
masked_fill_kernel(uint64_t len, const T* __restrict__ X, const uint8_t* __restrict__ mask, T value, T* __restrict__ Y) {
  const uint64_t gs = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < len; i += gs) Y[i] = mask[i] ? value : X[i];
}

}  // namespace kuiops

extern "C" {

int kuiops_cast(int src_dtype, int dst_dtype, uint64_t len, const void* X, void* Y, kuiops_stream_t s) {
  if (len == 0 || !X || !Y) return KUIOPS_EINVAL;
  cudaStream_t st = as_stream(s);
#define KUIOPS_CAST(SD, ST, DD, DT) if (src_dtype == SD && dst_dtype == DD) return cast_launch<ST, DT>(len, X, Y, st);
  KUIOPS_CAST(KUIOPS_F32, float, KUIOPS_F32, float)
  KUIOPS_CAST(KUIOPS_F32, float, KUIOPS_BF16, __nv_bfloat16)
  KUIOPS_CAST(KUIOPS_F32, float, KUIOPS_F16, __half)
  KUIOPS_CAST(KUIOPS_BF16, __nv_bfloat16, KUIOPS_F32, float)
  KUIOPS_CAST(KUIOPS_BF16, __nv_bfloat16, KUIOPS_BF16, __nv_bfloat16)
  KUIOPS_CAST(KUIOPS_BF16, __nv_bfloat16, KUIOPS_F16, __half)
  KUIOPS_CAST(KUIOPS_F16, __half, KUIOPS_F32, float)
  KUIOPS_CAST(KUIOPS_F16, __half, KUIOPS_BF16, __nv_bfloat16)
  KUIOPS_CAST(KUIOPS_F16, __half, KUIOPS_F16, __half)
#undef KUIOPS_CAST
  return KUIOPS_EINVAL;
}

int kuiops_masked_fill(int dtype, uint64_t len, const void* X, const void* mask, double value, void* Y, kuiops_stream_t s) {
  if (len == 0 || !X || !mask || !Y) return KUIOPS_EINVAL;
  const unsigned grid = stream_grid(len, 256 * 4, 16);
  cudaStream_t st = as_stream(s);
  auto M = static_cast<const uint8_t*>(mask);
  switch (dtype) {
    case KUIOPS_F32: masked_fill_kernel<float><<<grid, 256, 0, st>>>(len, static_cast<const float*>(X), M, float(value), static_cast<float*>(Y)); break;
    case KUIOPS_BF16: masked_fill_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(len, static_cast<const __nv_bfloat16*>(X), M, __float2bfloat16_rn(float(value)), static_cast<__nv_bfloat16*>(Y)); break;
    case KUIOPS_F16: masked_fill_kernel<__half><<<grid, 256, 0, st>>>(len, static_cast<const __half*>(X), M, __float2half_rn(float(value)), static_cast<__half*>(Y)); break;
    default: return KUIOPS_EINVAL;
  }
  return check_launch();
}

}  // extern "C"

