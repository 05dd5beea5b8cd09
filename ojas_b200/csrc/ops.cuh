// Internal entry points of the memory-bound kernels, shared with the step driver.
#pragma once
#include "common.cuh"

ojc_status embedding_backward_impl(ojc_backend* be, const uint32_t* ids, const void* grad, int32_t grad_dtype, float* out, int64_t tokens, int64_t vocab,
                                   int64_t dim, bool accumulate);
// copy (optional, F32 rows like x): also receives the input rows
ojc_status rms_forward_impl(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, float eps, ojc_tensor* y, float* copy = nullptr);
ojc_status rms_backward_impl(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, const ojc_tensor* gy, float eps, ojc_tensor* gx, ojc_tensor* gw,
                             bool accumulate_gw, bool accumulate_gx, bf16* gx_b = nullptr);   // gx_b (optional): a bf16 copy of grad_x
ojc_status rope_impl(ojc_backend* be, const char* op, const ojc_tensor* x, const ojc_tensor* cos_t, const ojc_tensor* sin_t, ojc_tensor* y, int backward);
ojc_status vres_backward_impl(ojc_backend* be, const ojc_tensor* v, const ojc_tensor* v0, const ojc_tensor* lambda, const ojc_tensor* gy, ojc_tensor* gv,
                              ojc_tensor* gv0, float* glambda, bool accumulate_lambda);
ojc_status gate_backward_impl(ojc_backend* be, const ojc_tensor* input, const ojc_tensor* weight, const ojc_tensor* bias, const ojc_tensor* attn,
                              const ojc_tensor* gout, const ojc_tensor* saved, ojc_tensor* ginput, float* gweight, float* gbias, ojc_tensor* gattn,
                              bool accumulate_w);
ojc_status swiglu_forward_impl(ojc_backend* be, const void* a, const void* u, void* m, int32_t dt, int64_t n);
ojc_status swiglu_backward_impl(ojc_backend* be, const void* a, const void* u, const void* gm, void* ga, void* gu, int32_t dt, int64_t n);

// fused.cu (bf16 storage)
bool qk_norm_rope_supported(int dh);
ojc_status qk_norm_rope_forward(ojc_backend* be, const bf16* x, int64_t xs, const float* w, const float* cos_t, const float* sin_t, bf16* y, int64_t ys,
                                int64_t tokens, int heads, int dh, int time, float eps);
ojc_status qk_norm_rope_backward(ojc_backend* be, const bf16* x, int64_t xs, const float* w, const float* cos_t, const float* sin_t, const bf16* gy, int64_t gys,
                                 bf16* gx, int64_t gxs, float* gw, int64_t tokens, int heads, int dh, int time, float eps);
ojc_status gate_apply_forward(ojc_backend* be, const bf16* z, int zld, const float* bias, const bf16* attn, bf16* out, float* scales, int64_t rows, int heads, int dh);
ojc_status gate_apply_backward(ojc_backend* be, const float* scales, const bf16* attn, const bf16* gout, bf16* gattn, bf16* gz, int zld, float* gbias, int64_t rows,
                               int heads, int dh, float* dr = nullptr, int time = 0);   // dr: also Dr[b, h, t] of the attention backward, rows = b * time + t
// row-strided forms for column slices of a [rows, ld] buffer
ojc_status swiglu_rows_forward(ojc_backend* be, const bf16* au, int64_t ld, bf16* m, int64_t rows, int64_t f);
ojc_status swiglu_rows_backward(ojc_backend* be, const bf16* au, const bf16* gm, bf16* gau, int64_t ld, int64_t rows, int64_t f);
ojc_status vres_rows_forward(ojc_backend* be, const bf16* v, int64_t ldv, const bf16* v0, int64_t ld0, const float* lambda, bf16* y, int64_t rows, int64_t cols);
ojc_status vres_rows_backward(ojc_backend* be, const bf16* v, int64_t ldv, const bf16* v0, int64_t ld0, const float* lambda, const bf16* gy, bf16* gv, int64_t ldg,
                              float* acc, bool first, float* glambda, int64_t rows, int64_t cols);
ojc_status vres_root_backward(ojc_backend* be, const float* acc, const bf16* g, bf16* out, int64_t ldo, int64_t rows, int64_t cols);
bool rms_backward_rows_supported(int64_t dim);
ojc_status rms_backward_rows(ojc_backend* be, const float* x, const float* w, const float* gy, float* gx, bf16* gx_b, float* part, int64_t rows, int64_t dim,
                             float eps, bool accumulate_gx, int blocks);
ojc_status rms_forward_rows(ojc_backend* be, const float* x, const float* w, bf16* y, float* copy, int64_t rows, int64_t dim, float eps);
