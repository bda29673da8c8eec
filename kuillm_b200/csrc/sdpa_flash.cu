// tcgen05 flash-attention forward (placeholder until the kernel lands: nothing is eligible, so
// every call takes the SIMT kernel).
#include "sdpa.cuh"
namespace kuiops {
bool sdpa_flash_eligible(const SdpaArgs&) { return false; }
int sdpa_flash(const SdpaArgs&, cudaStream_t) { return KUIOPS_EUNSUPPORTED; }
}  // namespace kuiops
