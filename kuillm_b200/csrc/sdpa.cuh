// Argument blocks shared by the attention kernels.
#pragma once
#include "common.cuh"

namespace kuiops {

struct SdpaArgs {
  int dtype;
  uint32_t n, h, h_kv, l, s, e, ev;
  const void* Q; int64_t q_sn, q_sh, q_sl;
  const void* K; int64_t k_sn, k_sh, k_ss;
  const void* V; int64_t v_sn, v_sh, v_ss;
  const void* bias;
  float scale;
  int is_causal;
  void* out; int64_t o_sn, o_sh, o_sl;
  float* lse;
  const int64_t* kv_lens;   // optional per-batch key counts on the device (<= s)
};

struct SdpaRowsPlan {
  uint32_t rows_h, rows_l;      // query heads x query positions handled by one CTA
  uint32_t hgroups, lblocks;
  uint64_t units;
  uint32_t splits, e_pad, r_pad, dv;
  int k_vec, v_vec;
  int* counters; float* partials;
};

SdpaRowsPlan sdpa_rows_plan(const SdpaArgs& a);
size_t sdpa_rows_workspace_bytes(const SdpaArgs& a);
size_t sdpa_rows_counter_bytes(const SdpaArgs& a);   // leading ticket words of that workspace
int sdpa_rows(const SdpaArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st);

// tcgen05 flash-attention forward (bf16 / f16, head dim 128, no bias).
bool sdpa_flash_eligible(const SdpaArgs& a);
int sdpa_flash(const SdpaArgs& a, cudaStream_t st);

// tcgen05 split-KV decode attention (bf16 / f16, head dim 128, G * l <= 128 query rows per KV head).
bool sdpa_decode_tc_eligible(const SdpaArgs& a);
size_t sdpa_decode_tc_workspace_bytes(const SdpaArgs& a);
size_t sdpa_decode_tc_counter_bytes(const SdpaArgs& a);
int sdpa_decode_tc(const SdpaArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t st);
void sdpa_decode_tc_force_splits(int splits);   // debug: 0 restores the rule

}  // namespace kuiops
