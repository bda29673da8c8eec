// Shared device/host helpers for the kuiops sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <atomic>
#include "../../include/kuiops.h"

namespace kuiops {

constexpr int kDefaultSMs = 148;       // B200: 2 dies x 74 SMs; used only when no device can be queried

// Number of SMs of the current device, asked once per device.  Grid sizes, split-K plans and the
// workspace sizes derived from them all go through this, so a query and the launch that follows it
// agree as long as the same device is current for both.
inline int num_sms() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return kDefaultSMs;
  }
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
    cudaGetLastError();
    return kDefaultSMs;
  }
  cache[dev].store(v, std::memory_order_relaxed);
  return v;
}
constexpr int kWarp = 32;

extern std::atomic<uint64_t> g_launches;
// How long a kernel polls a flag that another GPU raises before it gives up, records error word 30
// and carries on (nanoseconds; kuiops_debug_set_peer_wait_ns).
constexpr uint64_t kPeerWaitDefaultNs = 2000000000ull;
extern std::atomic<uint64_t> g_peer_wait_ns;

inline int check_launch() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaPeekAtLastError() == cudaSuccess ? KUIOPS_OK : KUIOPS_ELAUNCH;
}

inline cudaStream_t as_stream(kuiops_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- programmatic dependent launch -----------------------------------------------------------
// Kernels on the decode path are a few microseconds long, so launch latency and prologue are a
// large share of a step.  A kernel launched with the programmatic-serialisation attribute may
// begin (block scheduling, barrier / TMEM set-up) while its predecessor in the stream is still
// running; it must execute pdl_wait() before it touches global memory, which blocks until the
// predecessor grid has completed and its writes are visible.  pdl_trigger() tells the scheduler
// that this block no longer minds dependents being scheduled next to it; it is called after the
// block has claimed everything it will ever allocate (shared memory, TMEM), so a dependent that
// parks on an SM can never starve the grid it is waiting for.  Without the launch attribute both
// are no-ops.
extern std::atomic<int> g_pdl_enabled;
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch `kern` (which calls pdl_wait() first thing) with the attribute when enabled.
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled.load(std::memory_order_relaxed) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return e == cudaSuccess ? KUIOPS_OK : KUIOPS_ELAUNCH;
}

// Same, for a kernel whose CTAs form clusters of `cluster` along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
inline int launch_cluster_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              unsigned cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled.load(std::memory_order_relaxed) ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return e == cudaSuccess ? KUIOPS_OK : KUIOPS_ELAUNCH;
}

// 2^x by the special-function unit (relative error about 2^-22; results below 2^-126 become 0).
__device__ __forceinline__ float fast_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct ElemTraits<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

// Two floats rounded and packed into one 32-bit word of 16-bit elements (first value in the low half).
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 16-byte vector of T, the unit of every coalesced HBM access here.
template <typename T> struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
  return *reinterpret_cast<const Vec16<T>*>(p);
}
// Streaming load: data read exactly once, keep it out of L1.
template <typename T>
__device__ __forceinline__ Vec16<T> ld16_stream(const T* p) {
  Vec16<T> r;
  int4 raw = __ldcs(reinterpret_cast<const int4*>(p));
  *reinterpret_cast<int4*>(&r) = raw;
  return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<Vec16<T>*>(p) = v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions over <= 32 warps; `red` is a 32-float shared scratch.
// Every thread returns the full result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid size for grid-stride streaming kernels: whole multiples of the SM count.
inline unsigned stream_grid(uint64_t work_items, unsigned per_block, unsigned max_waves = 8) {
  uint64_t blocks = (work_items + per_block - 1) / per_block;
  uint64_t cap = uint64_t(num_sms()) * max_waves;
  if (blocks >= cap) return unsigned(cap);
  if (blocks > unsigned(num_sms())) blocks = ((blocks + num_sms() - 1) / num_sms()) * num_sms();
  return unsigned(blocks ? blocks : 1);
}

}  // namespace kuiops
