// Shared declarations of the attention kernels.
#pragma once
#include "common.cuh"

template <class P>
struct SdpaView {  // [B, H, T, dh] through strides; the dh axis is contiguous
  P* ptr;
  int64_t sb, sh, st;
  __host__ __device__ __forceinline__ P* row(int b, int h, int t) const { return ptr + b * sb + h * sh + t * st; }
};

struct SdpaDims { int batch, heads, kv_heads, time, dim; float scale; };

ojc_status sdpa_check(const char* op, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, SdpaDims* d);
ojc_status sdpa_forward_f32tier(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, int64_t window, ojc_tensor* out,
                                float* lse, const SdpaDims& d);
ojc_status sdpa_backward_f32tier(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const float* lse,
                                 const ojc_tensor* gout, int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const SdpaDims& d, float* dr);
// bf16 tensor-core tier (head_dim 64 or 128, full causal attention)
bool sdpa_tc_eligible(const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const SdpaDims& d);
ojc_status sdpa_forward_tc(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, int64_t window, ojc_tensor* out, float* lse,
                           const SdpaDims& d);
ojc_status sdpa_backward_tc(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const float* lse,
                            const ojc_tensor* gout, int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const SdpaDims& d, float* dr);
// tcgen05 / TMEM forward (head_dim 64, bf16, full causal)
bool sdpa_tcgen05_eligible(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, int64_t window, const SdpaDims& d);
ojc_status sdpa_forward_tcgen05(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, ojc_tensor* out, float* lse, const SdpaDims& d);
bool sdpa_tcgen05_bwd_eligible(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* gout, const ojc_tensor* gq,
                               const ojc_tensor* gk, const ojc_tensor* gv, int64_t window, const SdpaDims& d);
ojc_status sdpa_backward_tcgen05(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const float* lse,
                                 const ojc_tensor* gout, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const SdpaDims& d, float* work, const float* dr_given = nullptr);
// causal_sdpa_backward for a caller that already holds Dr = rowsum(dO . O) as F32 [B, H, T] (the gate's backward forms the same dot product): `*taken`
// says whether the tensor-core path used it; when it did not, nothing was launched and the caller runs the plain op.
ojc_status sdpa_backward_with_dr(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const ojc_tensor* lse,
                                 const ojc_tensor* gout, int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const float* dr, bool* taken);
bool sdpa_backward_takes_dr(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const ojc_tensor* gout,
                            const ojc_tensor* gq, const ojc_tensor* gk, const ojc_tensor* gv, int64_t window);
ojc_status sdpa_dr(ojc_backend* be, const ojc_tensor* out, const ojc_tensor* gout, float* dr, const SdpaDims& d);
