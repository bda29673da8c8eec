// C-ABI entry points of the GEMM family and the library-wide helpers.
#include "gemm.cuh"
#include "tc_ptx.cuh"
#include <cstdlib>

namespace kuiops {
std::atomic<uint64_t> g_launches{0};
static int pdl_default() {
  const char* e = getenv("KUIOPS_PDL");
  return (e && e[0] == '0') ? 0 : 1;
}
std::atomic<int> g_pdl_enabled{pdl_default()};
std::atomic<uint64_t> g_peer_wait_ns{kPeerWaitDefaultNs};
}
using namespace kuiops;

extern "C" {

int kuiops_abi_version(void) { return KUIOPS_ABI_VERSION; }

int kuiops_set_pdl(int enabled) {
  return g_pdl_enabled.exchange(enabled ? 1 : 0);
}

uint64_t kuiops_debug_set_peer_wait_ns(uint64_t ns) {
  return g_peer_wait_ns.exchange(ns ? ns : kPeerWaitDefaultNs);
}

int kuiops_debug_gemm_trace(uint64_t* device_buffer) {
  g_gemm_trace.store(reinterpret_cast<unsigned long long*>(device_buffer), std::memory_order_relaxed);
  return KUIOPS_OK;
}

uint64_t kuiops_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* kuiops_strerror(int code) {
  switch (code) {
    case KUIOPS_OK: return "ok";
    case KUIOPS_EINVAL: return "kuiops: a shape, stride or dtype contract does not hold";
    case KUIOPS_EUNSUPPORTED: return "kuiops: request outside what the kernels cover";
    case KUIOPS_EWORKSPACE: return "kuiops: workspace missing or too small";
    case KUIOPS_ELAUNCH: return "kuiops: CUDA launch failed";
    case KUIOPS_EDRIVER: return "kuiops: TMA descriptor encoding failed";
    case KUIOPS_ELIMIT: return "kuiops: size beyond a fixed maximum";
  }
  return "kuiops: unknown error";
}

int kuiops_debug_tc_error(unsigned int* host_out, int reset) {
  unsigned int* dev = tc_error_word_device();
  if (!dev || !host_out) return KUIOPS_EINVAL;
  if (cudaMemcpy(host_out, dev, sizeof(unsigned int), cudaMemcpyDeviceToHost) != cudaSuccess) return KUIOPS_ELAUNCH;
  if (reset && *host_out) {
    unsigned int zero = 0;
    if (cudaMemcpy(dev, &zero, sizeof(zero), cudaMemcpyHostToDevice) != cudaSuccess) return KUIOPS_ELAUNCH;
  }
  return KUIOPS_OK;
}

size_t kuiops_gemm_workspace_bytes(int dtype, uint32_t batch, uint32_t M, uint32_t N, uint32_t K) {
  if (dtype == KUIOPS_F32) return KUIOPS_GEMM_COUNTER_BYTES;
  return gemm_tc_workspace_bytes(batch, M, N, K);
}

int kuiops_gemm(int dtype, int out_dtype, uint32_t batch, uint32_t M, uint32_t N, uint32_t K,
                const void* A, int64_t lda, int64_t stride_a,
                const void* B, int64_t ldb, int64_t stride_b, int trans_b,
                const void* Cin, int64_t ldcin, int64_t stride_cin,
                float alpha, float beta,
                void* C, int64_t ldc, int64_t stride_c,
                void* workspace, size_t workspace_bytes, kuiops_stream_t stream) {
  if (dtype != KUIOPS_F32 && dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EINVAL;
  if (out_dtype != dtype && out_dtype != KUIOPS_F32) return KUIOPS_EINVAL;
  if (batch == 0 || M == 0 || N == 0 || K == 0) return KUIOPS_EINVAL;
  if (!A || !B || !C) return KUIOPS_EINVAL;
  if (lda < int64_t(K) || ldc < int64_t(N)) return KUIOPS_EINVAL;
  if (ldb < int64_t(trans_b ? K : N)) return KUIOPS_EINVAL;
  if (Cin && ldcin != 0 && ldcin < int64_t(N)) return KUIOPS_EINVAL;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = out_dtype; a.batch = batch; a.M = M; a.N = N; a.K = K;
  a.A = A; a.lda = lda; a.stride_a = stride_a;
  a.B = B; a.ldb = ldb; a.stride_b = stride_b; a.trans_b = trans_b ? 1 : 0;
  a.Cin = Cin; a.ldcin = ldcin; a.stride_cin = stride_cin;
  a.alpha = alpha; a.beta = Cin ? beta : 0.f;
  a.C = C; a.ldc = ldc; a.stride_c = stride_c; a.epilogue = 0;
  cudaStream_t st = as_stream(stream);
  if (gemm_tc_eligible(a)) return gemm_tc(a, workspace, workspace_bytes, st);
  return gemm_simt(a, st);
}

int kuiops_gemm_tune_set(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K, int splits, int bn) {
  return gemm_tune_set(dtype, epilogue, trans_b, M, N, K, splits, bn);
}
int kuiops_gemm_tune_clear(void) { gemm_tune_clear(); return KUIOPS_OK; }
int kuiops_gemm_set_sm_reserve(int sms) {
  if (sms < 0) sms = 0;
  if (sms > 64) sms = 64;
  return g_gemm_sm_reserve.exchange(sms);
}
int kuiops_gemm_tune_query(int dtype, int epilogue, int trans_b, uint32_t M, uint32_t N, uint32_t K, int* splits, int* bn,
                           int* swapped) {
  return gemm_tune_query(dtype, epilogue, trans_b, M, N, K, splits, bn, swapped);
}

int kuiops_gemm_swiglu(int dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, int64_t lda,
                       const void* W, int64_t ldw, void* Y, int64_t ldy,
                       void* workspace, size_t workspace_bytes, kuiops_stream_t stream) {
  if (dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EUNSUPPORTED;
  if (M == 0 || N == 0 || K == 0 || !A || !W || !Y) return KUIOPS_EINVAL;
  if (lda < int64_t(K) || ldw < int64_t(K) || ldy < int64_t(N) || N > 0x7FFFFFFFu) return KUIOPS_EINVAL;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = dtype; a.batch = 1; a.M = M; a.N = 2 * N; a.K = K;
  a.A = A; a.lda = lda; a.B = W; a.ldb = ldw; a.trans_b = 1;
  a.alpha = 1.f; a.beta = 0.f; a.C = Y; a.ldc = ldy; a.epilogue = 1;
  if (!gemm_tc_eligible(a)) return KUIOPS_EUNSUPPORTED;
  return gemm_tc(a, workspace, workspace_bytes, as_stream(stream));
}

int kuiops_gemm_rope_qkv(int dtype, uint32_t M, uint32_t hq, uint32_t hk, uint32_t d, uint32_t K,
                         const void* A, int64_t lda, const void* W, int64_t ldw, void* qkv, int64_t ldq,
                         const int64_t* positions, float theta, void* k_cache, void* v_cache, uint64_t cache_cap,
                         uint32_t rows_per_seq, kuiops_stream_t stream) {
  if (dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EUNSUPPORTED;
  if (M == 0 || hq == 0 || K == 0 || !A || !W || !qkv || !positions || !(theta > 0.f)) return KUIOPS_EINVAL;
  if ((k_cache == nullptr) != (v_cache == nullptr) || (k_cache && cache_cap == 0)) return KUIOPS_EINVAL;
  if (d != 128 || M > 128) return KUIOPS_EUNSUPPORTED;         // one 128-feature tile per head, decode-sized steps
  const uint64_t N = uint64_t(hq + 2 * hk) * d;
  if (N > 0x7FFFFFFFull || lda < int64_t(K) || ldw < int64_t(K) || ldq < int64_t(N)) return KUIOPS_EINVAL;
  GemmRope rope = {};
  rope.positions = positions; rope.theta = theta; rope.k_cache = k_cache; rope.v_cache = v_cache;
  rope.cache_cap = cache_cap; rope.hq = hq; rope.hk = hk; rope.rows_per_seq = rows_per_seq ? rows_per_seq : 1u;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = dtype; a.batch = 1; a.M = M; a.N = uint32_t(N); a.K = K;
  a.A = A; a.lda = lda; a.B = W; a.ldb = ldw; a.trans_b = 1;
  a.alpha = 1.f; a.beta = 0.f; a.C = qkv; a.ldc = ldq; a.epilogue = 2; a.rope = &rope;
  if (!gemm_tc_eligible(a)) return KUIOPS_EUNSUPPORTED;
  return gemm_tc(a, nullptr, 0, as_stream(stream));
}

int kuiops_gemm_residual_ssq(int dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, int64_t lda, const void* W, int64_t ldw,
                             void* resid, int64_t ldr, float* ssq_out, kuiops_stream_t stream) {
  if (dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EUNSUPPORTED;
  if (M == 0 || N == 0 || K == 0 || !A || !W || !resid || !ssq_out) return KUIOPS_EINVAL;
  if (M > 128) return KUIOPS_EUNSUPPORTED;
  if (lda < int64_t(K) || ldw < int64_t(K) || ldr < int64_t(N)) return KUIOPS_EINVAL;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = dtype; a.batch = 1; a.M = M; a.N = N; a.K = K;
  a.A = A; a.lda = lda; a.B = W; a.ldb = ldw; a.trans_b = 1;
  a.Cin = resid; a.ldcin = ldr; a.alpha = 1.f; a.beta = 1.f; a.C = resid; a.ldc = ldr; a.epilogue = 0;
  a.ssq_out = ssq_out;
  if (!gemm_tc_eligible(a)) return KUIOPS_EUNSUPPORTED;
  return gemm_tc(a, nullptr, 0, as_stream(stream));
}

int kuiops_gemm_swiglu_rms(int dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, int64_t lda,
                           const void* W, int64_t ldw, void* Y, int64_t ldy, const float* ssq, uint32_t ssq_tiles, float eps,
                           kuiops_stream_t stream) {
  if (dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EUNSUPPORTED;
  if (M == 0 || N == 0 || K == 0 || !A || !W || !Y || !ssq || ssq_tiles == 0 || !(eps >= 0.f)) return KUIOPS_EINVAL;
  if (M > 128) return KUIOPS_EUNSUPPORTED;
  if (lda < int64_t(K) || ldw < int64_t(K) || ldy < int64_t(N) || N > 0x7FFFFFFFu) return KUIOPS_EINVAL;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = dtype; a.batch = 1; a.M = M; a.N = 2 * N; a.K = K;
  a.A = A; a.lda = lda; a.B = W; a.ldb = ldw; a.trans_b = 1;
  a.alpha = 1.f; a.beta = 0.f; a.C = Y; a.ldc = ldy; a.epilogue = 1;
  a.ssq_in = ssq; a.ssq_tiles = ssq_tiles; a.ssq_eps = eps;
  if (!gemm_tc_eligible(a)) return KUIOPS_EUNSUPPORTED;
  return gemm_tc(a, nullptr, 0, as_stream(stream));
}

int kuiops_gemm_rope_qkv_rms(int dtype, uint32_t M, uint32_t hq, uint32_t hk, uint32_t d, uint32_t K,
                             const void* A, int64_t lda, const void* W, int64_t ldw, void* qkv, int64_t ldq,
                             const int64_t* positions, float theta, void* k_cache, void* v_cache, uint64_t cache_cap,
                             uint32_t rows_per_seq, const float* ssq, uint32_t ssq_tiles, float eps, kuiops_stream_t stream) {
  if (dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EUNSUPPORTED;
  if (M == 0 || hq == 0 || K == 0 || !A || !W || !qkv || !positions || !(theta > 0.f)) return KUIOPS_EINVAL;
  if (!ssq || ssq_tiles == 0 || !(eps >= 0.f)) return KUIOPS_EINVAL;
  if ((k_cache == nullptr) != (v_cache == nullptr) || (k_cache && cache_cap == 0)) return KUIOPS_EINVAL;
  if (d != 128 || M > 128) return KUIOPS_EUNSUPPORTED;
  const uint64_t N = uint64_t(hq + 2 * hk) * d;
  if (N > 0x7FFFFFFFull || lda < int64_t(K) || ldw < int64_t(K) || ldq < int64_t(N)) return KUIOPS_EINVAL;
  GemmRope rope = {};
  rope.positions = positions; rope.theta = theta; rope.k_cache = k_cache; rope.v_cache = v_cache;
  rope.cache_cap = cache_cap; rope.hq = hq; rope.hk = hk; rope.rows_per_seq = rows_per_seq ? rows_per_seq : 1u;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = dtype; a.batch = 1; a.M = M; a.N = uint32_t(N); a.K = K;
  a.A = A; a.lda = lda; a.B = W; a.ldb = ldw; a.trans_b = 1;
  a.alpha = 1.f; a.beta = 0.f; a.C = qkv; a.ldc = ldq; a.epilogue = 2; a.rope = &rope;
  a.ssq_in = ssq; a.ssq_tiles = ssq_tiles; a.ssq_eps = eps;
  if (!gemm_tc_eligible(a)) return KUIOPS_EUNSUPPORTED;
  return gemm_tc(a, nullptr, 0, as_stream(stream));
}

int kuiops_gemm_push(int dtype, uint32_t M, uint32_t N, uint32_t K, const void* A, int64_t lda,
                     const void* B, int64_t ldb, int trans_b, uint32_t n_ranks, uint32_t rank,
                     const uint64_t* peer_base, uint64_t slot_bytes, const uint32_t* epoch, kuiops_stream_t stream) {
  if (dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EUNSUPPORTED;
  if (M == 0 || N == 0 || K == 0 || !A || !B || !peer_base || !epoch) return KUIOPS_EINVAL;
  if (n_ranks < 2 || n_ranks > KUIOPS_MAX_PEERS || rank >= n_ranks) return KUIOPS_EINVAL;
  if (M > 128 || N % 4) return KUIOPS_EUNSUPPORTED;            // the weight-streaming placement only; cells hold element pairs
  if (lda < int64_t(K) || ldb < int64_t(trans_b ? K : N)) return KUIOPS_EINVAL;
  if (slot_bytes < uint64_t(M) * N * 4 || (slot_bytes & 15u)) return KUIOPS_EINVAL;   // 4 bytes per element: value + half a stamp
  GemmPush push = {};
  push.n_ranks = n_ranks; push.rank = rank;
  for (uint32_t r = 0; r < n_ranks; ++r) {
    if (!peer_base[r] || (peer_base[r] & 15u)) return KUIOPS_EINVAL;
    push.peer_base[r] = peer_base[r];
  }
  push.slot_bytes = slot_bytes;
  push.epoch = epoch;
  GemmArgs a = {};
  a.dtype = dtype; a.out_dtype = dtype; a.batch = 1; a.M = M; a.N = N; a.K = K;
  a.A = A; a.lda = lda; a.B = B; a.ldb = ldb; a.trans_b = trans_b ? 1 : 0;
  a.alpha = 1.f; a.beta = 0.f; a.C = nullptr; a.ldc = N; a.epilogue = 0; a.push = &push;
  if (!gemm_tc_eligible(a)) return KUIOPS_EUNSUPPORTED;
  return gemm_tc(a, nullptr, 0, as_stream(stream));
}

#define KUIOPS_GEMM_ENTRIES(SUFFIX, DT)                                                                             \
  int kuiops_mm_##SUFFIX(uint32_t M, uint32_t N, uint32_t K, const void* A, const void* B, void* C, void* ws,       \
                         size_t wsb, kuiops_stream_t s) {                                                           \
    return kuiops_gemm(DT, DT, 1, M, N, K, A, K, 0, B, N, 0, 0, nullptr, 0, 0, 1.f, 0.f, C, N, 0, ws, wsb, s);      \
  }                                                                                                                 \
  int kuiops_addmm_##SUFFIX(uint32_t M, uint32_t K, uint32_t N, float alpha, float beta, const void* A,             \
                            const void* B, void* C, void* ws, size_t wsb, kuiops_stream_t s) {                      \
    return kuiops_gemm(DT, DT, 1, M, N, K, A, K, 0, B, N, 0, 0, C, N, 0, alpha, beta, C, N, 0, ws, wsb, s);         \
  }                                                                                                                 \
  int kuiops_bmm_##SUFFIX(uint32_t batch, uint32_t M, uint32_t K, uint32_t N, const void* A, const void* B,         \
                          void* C, void* ws, size_t wsb, kuiops_stream_t s) {                                       \
    return kuiops_gemm(DT, DT, batch, M, N, K, A, K, int64_t(M) * K, B, N, int64_t(K) * N, 0, nullptr, 0, 0, 1.f,   \
                       0.f, C, N, int64_t(M) * N, ws, wsb, s);                                                      \
  }

KUIOPS_GEMM_ENTRIES(f32, KUIOPS_F32)
KUIOPS_GEMM_ENTRIES(bf16, KUIOPS_BF16)
KUIOPS_GEMM_ENTRIES(f16, KUIOPS_F16)

}  // extern "C"
