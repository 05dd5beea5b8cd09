// Device-side optimizer pieces shared by the C ABI and the step driver.
#pragma once
#include "common.cuh"

int64_t norm_partials(int64_t n);
// norm_and_scale_dev[0] = global L2 norm, [1] = clip scale (1 when max_norm < 0). No host sync.
ojc_status grad_norm_device(ojc_backend* be, const float* const* ptrs, const int64_t* lens, int64_t count, float max_norm, float* norm_and_scale_dev);
ojc_status scale_by_device(ojc_backend* be, float* x, int64_t n, const float* scale_dev);
// grad_scale_dev (optional): device scalar folded into the gradient when it is < 1 (the clip coefficient).
ojc_status adamw_device(ojc_backend* be, float* p, const float* g, float* m, float* v, bf16* mirror, int64_t n, uint64_t step_before,
                        const ojc_adamw_config& cfg, const float* grad_scale_dev);
ojc_status muon_device(ojc_backend* be, float* p, const float* g, float* mom, bf16* mirror, int64_t rows, int64_t cols, const ojc_muon_config& cfg,
                       const float* grad_scale_dev);
uint64_t muon_scratch_bytes(int64_t rows, int64_t cols, bool bf16_mode);
// the same step for up to 48 matrices of one shape at once (pointer tables of length `batch`; mirror may be null)
ojc_status muon_group_device(ojc_backend* be, float* const* p, const float* const* g, float* const* mom, bf16* const* mirror, int64_t batch, int64_t rows,
                             int64_t cols, const ojc_muon_config& cfg, const float* grad_scale_dev);
