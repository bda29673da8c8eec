// SIMT GEMM: the path for fp32 operands and for bf16/f16 shapes the tensor-core kernels cannot
// take (leading dimensions that are not multiples of 8 elements, unaligned pointers).  Any M, N,
// K; fp32 accumulation; alpha/beta epilogue with a full or row-broadcast addend.
// Counterpart of Klas.GEMM.BlockTiling2D (kuiops/mm/Kuiops.Mm.Inst.fst.j2:12-15,
// kuiops/addmm/Kuiops.Addmm.Inst.fst.j2:11-12) and of the per-cell bmm kernel
// (kuiops/bmm/Kuiops.Bmm.fst:13-23), without their tile-divisibility preconditions.
#include "common.cuh"
#include "gemm.cuh"

namespace kuiops {

constexpr int SBM = 64, SBN = 64, SBK = 16;

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(GemmArgs a) {
  __shared__ float As[SBK][SBM + 4];
  __shared__ float Bs[SBK][SBN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, 4 x 4 outputs each
  const uint32_t m0 = blockIdx.y * SBM, n0 = blockIdx.x * SBN;
  const uint32_t b = blockIdx.z;
  const T* A = static_cast<const T*>(a.A) + size_t(b) * a.stride_a;
  const T* B = static_cast<const T*>(a.B) + size_t(b) * a.stride_b;
  float acc[4][4] = {};
  for (uint32_t k0 = 0; k0 < a.K; k0 += SBK) {
    // A tile: SBM x SBK, read along K (contiguous in memory)
    for (int i = tid; i < SBM * SBK; i += 256) {
      const int r = i / SBK, c = i % SBK;
      const uint32_t gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < a.M && gk < a.K) ? ElemTraits<T>::to_f(A[size_t(gm) * a.lda + gk]) : 0.f;
    }
    if (a.trans_b) {
      // B stored [N, K]: contiguous along K
      for (int i = tid; i < SBN * SBK; i += 256) {
        const int r = i / SBK, c = i % SBK;
        const uint32_t gn = n0 + r, gk = k0 + c;
        Bs[c][r] = (gn < a.N && gk < a.K) ? ElemTraits<T>::to_f(B[size_t(gn) * a.ldb + gk]) : 0.f;
      }
    } else {
      // B stored [K, N]: contiguous along N
      for (int i = tid; i < SBN * SBK; i += 256) {
        const int r = i / SBN, c = i % SBN;
        const uint32_t gk = k0 + r, gn = n0 + c;
        Bs[r][c] = (gn < a.N && gk < a.K) ? ElemTraits<T>::to_f(B[size_t(gk) * a.ldb + gn]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SBK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  TO* C = static_cast<TO*>(a.C) + size_t(b) * a.stride_c;
  const T* Cin = a.Cin ? static_cast<const T*>(a.Cin) + size_t(b) * a.stride_cin : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t gm = m0 + ty * 4 + i;
    if (gm >= a.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t gn = n0 + tx * 4 + j;
      if (gn >= a.N) continue;
      float v = a.alpha * acc[i][j];
      if (Cin) v += a.beta * ElemTraits<T>::to_f(Cin[size_t(gm) * a.ldcin + gn]);
      C[size_t(gm) * a.ldc + gn] = ElemTraits<TO>::from_f(v);
    }
  }
}

int gemm_simt(const GemmArgs& a, cudaStream_t st) {
  dim3 grid((a.N + SBN - 1) / SBN, (a.M + SBM - 1) / SBM, a.batch);
  if (grid.y > 65535 || grid.z > 65535) return KUIOPS_EUNSUPPORTED;
  const bool f32out = a.out_dtype == KUIOPS_F32;
  switch (a.dtype) {
    case KUIOPS_F32: gemm_simt_kernel<float, float><<<grid, 256, 0, st>>>(a); break;
    case KUIOPS_BF16:
      if (f32out) gemm_simt_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(a);
      else gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(a);
      break;
    case KUIOPS_F16:
      if (f32out) gemm_simt_kernel<__half, float><<<grid, 256, 0, st>>>(a);
      else gemm_simt_kernel<__half, __half><<<grid, 256, 0, st>>>(a);
      break;
    default: return KUIOPS_EINVAL;
  }
  return check_launch();
}

}  // namespace kuiops
