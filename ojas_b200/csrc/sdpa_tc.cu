// bf16 tensor-core attention tier (placeholder until the kernels land: nothing is eligible yet).
#include "sdpa.cuh"
bool sdpa_tc_eligible(const ojc_tensor*, const ojc_tensor*, const ojc_tensor*, const ojc_tensor*, const SdpaDims&) { return false; }
ojc_status sdpa_forward_tc(ojc_backend*, const ojc_tensor*, const ojc_tensor*, const ojc_tensor*, int64_t, ojc_tensor*, float*, const SdpaDims&) {
  return ojc_fail(OJC_ERR_UNSUPPORTED, "causal_sdpa_forward", "tensor-core tier not built");
}
ojc_status sdpa_backward_tc(ojc_backend*, const ojc_tensor*, const ojc_tensor*, const ojc_tensor*, const ojc_tensor*, const float*, const ojc_tensor*, int64_t,
                            ojc_tensor*, ojc_tensor*, ojc_tensor*, const SdpaDims&, float*) {
  return ojc_fail(OJC_ERR_UNSUPPORTED, "causal_sdpa_backward", "tensor-core tier not built");
}
