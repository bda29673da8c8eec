// C-ABI entry point of scaled dot-product attention: contract checks and kernel choice.
#include "sdpa.cuh"
#include <mutex>

using namespace kuiops;

static int fill_args(SdpaArgs& a, int dtype, uint32_t n, uint32_t h, uint32_t h_kv, uint32_t l, uint32_t s, uint32_t e,
                     uint32_t ev) {
  if (dtype != KUIOPS_F32 && dtype != KUIOPS_BF16 && dtype != KUIOPS_F16) return KUIOPS_EINVAL;
  if (n == 0 || h == 0 || h_kv == 0 || l == 0 || s == 0 || e == 0 || ev == 0) return KUIOPS_EINVAL;
  if (h % h_kv) return KUIOPS_EINVAL;
  a.dtype = dtype; a.n = n; a.h = h; a.h_kv = h_kv; a.l = l; a.s = s; a.e = e; a.ev = ev;
  return KUIOPS_OK;
}

// Scratch for kuiops_sdpa_noalloc: lives in the library image, one copy per GPU that loads it.
// In host code the name below is only a handle; the device address comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char g_sdpa_static_scratch[KUIOPS_SDPA_NOALLOC_SCRATCH_BYTES];

// Address of the array on device `dev`, which must be the current device.
static int sdpa_static_scratch(int dev, void** out) {
  static std::mutex mu;
  static void* per_device[64] = {};
  if (dev < 0 || dev >= 64) return KUIOPS_ELAUNCH;
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_sdpa_static_scratch) != cudaSuccess || !ptr) return KUIOPS_ELAUNCH;
    per_device[dev] = ptr;
  }
  *out = per_device[dev];
  return KUIOPS_OK;
}

// Makes `dev` the current device for its lifetime and puts the previous one back afterwards.
struct DeviceScope {
  int prev = -1;
  bool switched = false, ok = true;
  explicit DeviceScope(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev) {
      if (cudaSetDevice(dev) != cudaSuccess) { ok = false; return; }
      switched = true;
    }
  }
  ~DeviceScope() { if (switched) cudaSetDevice(prev); }
};

enum SdpaKernel { kSdpaFlash, kSdpaDecodeTc, kSdpaRows };

// The kernel kuiops_sdpa* runs for these arguments (pointer alignment included).
static SdpaKernel choose_kernel(const SdpaArgs& a) {
  if (sdpa_flash_eligible(a)) return kSdpaFlash;
  if (sdpa_decode_tc_eligible(a)) return kSdpaDecodeTc;
  return kSdpaRows;
}

static int check_and_fill_ptrs(SdpaArgs& a,
                               const void* Q, int64_t q_sn, int64_t q_sh, int64_t q_sl,
                               const void* K, int64_t k_sn, int64_t k_sh, int64_t k_ss,
                               const void* V, int64_t v_sn, int64_t v_sh, int64_t v_ss,
                               const void* bias, float scale, int is_causal,
                               void* out, int64_t o_sn, int64_t o_sh, int64_t o_sl, float* lse, const int64_t* kv_lens) {
  if (!Q || !K || !V || !out) return KUIOPS_EINVAL;
  if (q_sl < int64_t(a.e) || k_ss < int64_t(a.e) || v_ss < int64_t(a.ev) || o_sl < int64_t(a.ev)) return KUIOPS_EINVAL;
  a.Q = Q; a.q_sn = q_sn; a.q_sh = q_sh; a.q_sl = q_sl;
  a.K = K; a.k_sn = k_sn; a.k_sh = k_sh; a.k_ss = k_ss;
  a.V = V; a.v_sn = v_sn; a.v_sh = v_sh; a.v_ss = v_ss;
  a.bias = bias; a.scale = scale; a.is_causal = is_causal ? 1 : 0;
  a.out = out; a.o_sn = o_sn; a.o_sh = o_sh; a.o_sl = o_sl; a.lse = lse; a.kv_lens = kv_lens;
  return KUIOPS_OK;
}

extern "C" {

int kuiops_debug_sdpa_splits(int splits) {
  sdpa_decode_tc_force_splits(splits);
  return KUIOPS_OK;
}

size_t kuiops_sdpa_workspace_bytes(int dtype, uint32_t n, uint32_t h, uint32_t h_kv, uint32_t l, uint32_t s,
                                   uint32_t e, uint32_t ev) {
  SdpaArgs a = {};
  if (fill_args(a, dtype, n, h, h_kv, l, s, e, ev) != KUIOPS_OK) return 0;
  // which kernel runs also depends on pointer alignment, unknown here: cover both
  size_t need = sdpa_rows_workspace_bytes(a);
  if (dtype != KUIOPS_F32 && e == 128 && ev == 128 && uint64_t(h / h_kv) * l <= 128 && l <= 16) {
    const size_t t = sdpa_decode_tc_workspace_bytes(a);
    if (t > need) need = t;
  }
  return need;
}

int kuiops_sdpa_varlen(int dtype, uint32_t n, uint32_t h, uint32_t h_kv, uint32_t l, uint32_t s, uint32_t e, uint32_t ev,
                const void* Q, int64_t q_sn, int64_t q_sh, int64_t q_sl,
                const void* K, int64_t k_sn, int64_t k_sh, int64_t k_ss,
                const void* V, int64_t v_sn, int64_t v_sh, int64_t v_ss,
                const void* bias, float scale, int is_causal,
                void* out, int64_t o_sn, int64_t o_sh, int64_t o_sl, float* lse,
                const int64_t* kv_lens,
                void* workspace, size_t workspace_bytes, kuiops_stream_t stream) {
  SdpaArgs a = {};
  int rc = fill_args(a, dtype, n, h, h_kv, l, s, e, ev);
  if (rc != KUIOPS_OK) return rc;
  rc = check_and_fill_ptrs(a, Q, q_sn, q_sh, q_sl, K, k_sn, k_sh, k_ss, V, v_sn, v_sh, v_ss, bias, scale, is_causal,
                           out, o_sn, o_sh, o_sl, lse, kv_lens);
  if (rc != KUIOPS_OK) return rc;
  cudaStream_t st = as_stream(stream);
  switch (choose_kernel(a)) {
    case kSdpaFlash: return sdpa_flash(a, st);
    case kSdpaDecodeTc: return sdpa_decode_tc(a, workspace, workspace_bytes, st);
    default: return sdpa_rows(a, workspace, workspace_bytes, st);
  }
}

int kuiops_sdpa(int dtype, uint32_t n, uint32_t h, uint32_t h_kv, uint32_t l, uint32_t s, uint32_t e, uint32_t ev,
                const void* Q, int64_t q_sn, int64_t q_sh, int64_t q_sl,
                const void* K, int64_t k_sn, int64_t k_sh, int64_t k_ss,
                const void* V, int64_t v_sn, int64_t v_sh, int64_t v_ss,
                const void* bias, float scale, int is_causal,
                void* out, int64_t o_sn, int64_t o_sh, int64_t o_sl, float* lse,
                void* workspace, size_t workspace_bytes, kuiops_stream_t stream) {
  return kuiops_sdpa_varlen(dtype, n, h, h_kv, l, s, e, ev, Q, q_sn, q_sh, q_sl, K, k_sn, k_sh, k_ss, V, v_sn, v_sh, v_ss,
                            bias, scale, is_causal, out, o_sn, o_sh, o_sl, lse, nullptr, workspace, workspace_bytes, stream);
}

int kuiops_sdpa_noalloc(int dtype, uint32_t n, uint32_t h, uint32_t h_kv, uint32_t l, uint32_t s, uint32_t e, uint32_t ev,
                        const void* Q, int64_t q_sn, int64_t q_sh, int64_t q_sl,
                        const void* K, int64_t k_sn, int64_t k_sh, int64_t k_ss,
                        const void* V, int64_t v_sn, int64_t v_sh, int64_t v_ss,
                        const void* bias, float scale, int is_causal,
                        void* out, int64_t o_sn, int64_t o_sh, int64_t o_sl, float* lse,
                        const int64_t* kv_lens, kuiops_stream_t stream) {
  SdpaArgs a = {};
  int rc = fill_args(a, dtype, n, h, h_kv, l, s, e, ev);
  if (rc != KUIOPS_OK) return rc;
  rc = check_and_fill_ptrs(a, Q, q_sn, q_sh, q_sl, K, k_sn, k_sh, k_ss, V, v_sn, v_sh, v_ss, bias, scale, is_causal,
                           out, o_sn, o_sh, o_sl, lse, kv_lens);
  if (rc != KUIOPS_OK) return rc;
  // size the refusal on the kernel that will run for these arguments, not on the largest of all
  const SdpaKernel which = choose_kernel(a);
  size_t need = 0, head = 0;
  if (which == kSdpaDecodeTc) { need = sdpa_decode_tc_workspace_bytes(a); head = sdpa_decode_tc_counter_bytes(a); }
  else if (which == kSdpaRows) { need = sdpa_rows_workspace_bytes(a); head = sdpa_rows_counter_bytes(a); }
  if (need > size_t(KUIOPS_SDPA_NOALLOC_SCRATCH_BYTES)) return KUIOPS_ELIMIT;   // beyond the built-in scratch
  // The array to use is the copy on the GPU that holds Q, whichever device the calling thread
  // has current; that device is made current for the set-up, the clearing and the launch.
  cudaPointerAttributes attr = {};
  if (cudaPointerGetAttributes(&attr, Q) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
    cudaGetLastError();
    return KUIOPS_EINVAL;
  }
  DeviceScope scope(attr.device);
  if (!scope.ok) return KUIOPS_ELAUNCH;
  void* scratch = nullptr;
  rc = sdpa_static_scratch(attr.device, &scratch);
  if (rc != KUIOPS_OK) return rc;
  cudaStream_t st = as_stream(stream);
  if (need) {
    // every call shares the array and it keeps the previous call's contents (possibly another
    // kernel's records): the ticket words at its head have to be zero when the kernel starts
    if (cudaMemsetAsync(scratch, 0, head, st) != cudaSuccess) return KUIOPS_ELAUNCH;
  }
  switch (which) {
    case kSdpaFlash: return sdpa_flash(a, st);
    case kSdpaDecodeTc: return sdpa_decode_tc(a, scratch, size_t(KUIOPS_SDPA_NOALLOC_SCRATCH_BYTES), st);
    default: return sdpa_rows(a, scratch, size_t(KUIOPS_SDPA_NOALLOC_SCRATCH_BYTES), st);
  }
}

}  // extern "C"
