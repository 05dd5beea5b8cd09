#pragma once
#include "common.cuh"
// y[rows, out] (+)= x[rows, in] W[out, in]^T (+ residual[rows, out], F32); accumulate needs an F32 y
ojc_status linear_forward_impl(ojc_backend* be, const void* x, int32_t x_dt, const void* w, int32_t w_dt, void* y, int32_t y_dt, int64_t rows, int64_t kin,
                               int64_t nout, const float* residual, bool accumulate = false);
// gx[rows, in] (+)= gy[rows, out] W[out, in]
ojc_status linear_backward_input_impl(ojc_backend* be, const void* w, int32_t w_dt, const void* gy, int32_t g_dt, void* gx, int32_t gx_dt, int64_t rows,
                                      int64_t kin, int64_t nout, bool accumulate);
// gw[out, in] (+)= gy[rows, out]^T x[rows, in]
ojc_status linear_backward_weight_impl(ojc_backend* be, const void* x, int32_t x_dt, const void* gy, int32_t g_dt, float* gw, int64_t rows, int64_t kin,
                                       int64_t nout, bool accumulate);
// The MLP down projection's input gradient with SwiGLU's backward folded into the product's epilogue (bf16 tier): with
// g = gy[rows, out] W[out, in] rounded to bf16, gau[rows, 0:in] = g_a and gau[rows, in:2 in] = g_u from au[rows, 0:in] = a and
// au[rows, in:2 in] = u (both buffers in rows `ld` wide). The same bits as linear_backward_input_impl followed by swiglu_rows_backward.
// Two-SM tiles only: ask linear_backward_input_swiglu_eligible first.
bool linear_backward_input_swiglu_eligible(ojc_backend* be, const void* w, const void* gy, const void* au, const void* gau, int64_t ld, int64_t rows, int64_t kin, int64_t nout);
ojc_status linear_backward_input_swiglu_impl(ojc_backend* be, const void* w, const void* gy, const void* au, void* gau, int64_t ld, int64_t rows, int64_t kin,
                                             int64_t nout);
// The MLP's gate/up product with SwiGLU's forward folded into its epilogue (bf16 tier): au[rows, 0:hidden] = a = x Wg^T,
// au[rows, hidden:2 hidden] = u = x Wu^T (w = [Wg; Wu], [2 hidden, in]) and m[rows, hidden] = bf16(silu(a)) * u. The same bits as
// linear_forward_impl followed by swiglu_rows_forward. Two-SM tiles only: ask linear_forward_swiglu_eligible first.
bool linear_forward_swiglu_eligible(ojc_backend* be, const void* x, const void* w, const void* au, const void* m, int64_t ld, int64_t rows, int64_t kin, int64_t hidden);
ojc_status linear_forward_swiglu_impl(ojc_backend* be, const void* x, const void* w, void* au, void* m, int64_t ld, int64_t rows, int64_t kin, int64_t hidden);
