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
