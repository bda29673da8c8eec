// Argument block shared by the GEMM kernels.
#pragma once
#include "common.cuh"

namespace kuiops {

// Tensor-parallel "push" epilogue: see kuiops_gemm_push.
struct GemmPush {
  uint32_t n_ranks, rank;
  uint64_t peer_base[KUIOPS_MAX_PEERS];
  uint64_t slot_bytes;
  const unsigned int* epoch;
};

// Rotary embedding + KV-cache append fused into the packed QKV projection: see kuiops_gemm_rope_qkv.
struct GemmRope {
  const int64_t* positions;
  float theta;
  void* k_cache; void* v_cache;
  uint64_t cache_cap;
  uint32_t hq, hk, rows_per_seq;
};

struct GemmArgs {
  int dtype, out_dtype;
  uint32_t batch, M, N, K;
  const void* A; int64_t lda, stride_a;
  const void* B; int64_t ldb, stride_b; int trans_b;
  const void* Cin; int64_t ldcin, stride_cin;
  float alpha, beta;
  void* C; int64_t ldc, stride_c;
  float* ssq_out;            // producer half of a folded RMSNorm: per (128-feature tile, row) sums of squares of C as stored
  const float* ssq_in;       // consumer half: those partials for the rows of A; row m of the product is scaled by rsqrt(sum / K + eps)
  uint32_t ssq_tiles;
  float ssq_eps;
  const GemmRope* rope;   // epilogue 2 only
  const GemmPush* push;   // non-null: partial sums go to every rank's receive area instead of C
  int epilogue;   // 0: C = alpha*acc + beta*Cin;  1: C[m, j] = silu(acc[m, 2j]) * acc[m, 2j+1] (gate/up rows interleaved in B);  2: rotary embedding + cache append (rope)
};

// SIMT kernel: any dtype / shape / stride.
int gemm_simt(const GemmArgs& a, cudaStream_t st);
// tcgen05 kernel: bf16 / f16, 16-byte aligned operands.  Returns KUIOPS_EUNSUPPORTED when the
// operands do not meet the TMA alignment rules so the caller can fall back to gemm_simt.
bool gemm_tc_eligible(const GemmArgs& a);
size_t gemm_tc_workspace_bytes(uint32_t batch, uint32_t M, uint32_t N, uint32_t K);
int gemm_tc(const GemmArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st);
extern std::atomic<unsigned long long*> g_gemm_trace;
// SMs the persistent (normal-placement) GEMM leaves free, for kernels that must run beside it (see kuiops_gemm_set_sm_reserve).
extern std::atomic<int> g_gemm_sm_reserve;
// Tuned-plan table of the tcgen05 kernel (see kuiops_gemm_tune_set).
int gemm_tune_set(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K, int splits, int bn);
void gemm_tune_clear();
int gemm_tune_query(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K, int* splits, int* bn, int* swapped);

}  // namespace kuiops
