// linear_forward / linear_backward / linear_backward_input: y = x W^T, dX = dY W, dW = dY^T x
// (ojas-cpu/src/linalg.rs:69-210). BF16 operands run on the tcgen05 kernel, F32 operands on the f32 tier.
#include "common.cuh"
#include "gemm.cuh"
#include "linear.cuh"

static ojc_status linear_dims(const char* op, const ojc_tensor* x, const ojc_tensor* w, int64_t* rows, int64_t* kin, int64_t* nout) {
  if (w->rank != 2 || x->rank < 1 || x->shape[x->rank - 1] != w->shape[1]) return ojc_fail(OJC_ERR_SHAPE, op, "x [..., in] against weight [out, in]");
  *kin = w->shape[1]; *nout = w->shape[0];
  if (*kin == 0 || *nout == 0 || numel(x) == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  *rows = numel(x) / *kin;
  return OJC_OK;
}

ojc_status linear_forward_impl(ojc_backend* be, const void* x, int32_t x_dt, const void* w, int32_t w_dt, void* y, int32_t y_dt, int64_t rows, int64_t kin,
                               int64_t nout, const float* residual, bool accumulate) {
  GemmOperand a{x, x_dt, kin, 1}, b{w, w_dt, 1, kin};
  return gemm_auto(be, "linear_forward", a, b, y, y_dt, nout, rows, nout, kin, 1.0f, accumulate, residual);
}
ojc_status linear_backward_input_impl(ojc_backend* be, const void* w, int32_t w_dt, const void* gy, int32_t g_dt, void* gx, int32_t gx_dt, int64_t rows,
                                      int64_t kin, int64_t nout, bool accumulate) {
  GemmOperand a{gy, g_dt, nout, 1}, b{w, w_dt, kin, 1};
  return gemm_auto(be, "linear_backward", a, b, gx, gx_dt, kin, rows, kin, nout, 1.0f, accumulate, nullptr);
}
bool linear_forward_swiglu_eligible(ojc_backend* be, const void* x, const void* w, const void* au, const void* m, int64_t ld, int64_t rows, int64_t kin, int64_t hidden) {
  GemmOperand a{x, OJC_BF16, kin, 1}, b{w, OJC_BF16, 1, kin};
  return ld == 2 * hidden && gemm_tc_eligible(a, b, au, OJC_BF16, ld, rows, 2 * hidden, kin) && gemm_tc_swiglu_forward_eligible(be, rows, 2 * hidden, hidden, m);
}
ojc_status linear_forward_swiglu_impl(ojc_backend* be, const void* x, const void* w, void* au, void* m, int64_t ld, int64_t rows, int64_t kin, int64_t hidden) {
  GemmOperand a{x, OJC_BF16, kin, 1}, b{w, OJC_BF16, 1, kin};
  const SwigluForward sw{m, hidden};
  return gemm_tc_batched(be, "linear_forward", a, b, au, OJC_BF16, ld, rows, 2 * hidden, kin, 1, 0, 0, 0, 1.0f, false, nullptr, nullptr, false, nullptr, &sw);
}
ojc_status linear_backward_input_swiglu_impl(ojc_backend* be, const void* w, const void* gy, const void* au, void* gau, int64_t ld, int64_t rows, int64_t kin,
                                             int64_t nout) {
  GemmOperand a{gy, OJC_BF16, nout, 1}, b{w, OJC_BF16, kin, 1};
  const SwigluGrad sw{au, ld};
  return gemm_tc_batched(be, "linear_backward", a, b, gau, OJC_BF16, ld, rows, kin, nout, 1, 0, 0, 0, 1.0f, false, nullptr, nullptr, false, &sw);
}
bool linear_backward_input_swiglu_eligible(ojc_backend* be, const void* w, const void* gy, const void* au, const void* gau, int64_t ld, int64_t rows, int64_t kin, int64_t nout) {
  GemmOperand a{gy, OJC_BF16, nout, 1}, b{w, OJC_BF16, kin, 1};
  return kin % 64 == 0 && ld % 8 == 0 && ld >= 2 * kin && (reinterpret_cast<uintptr_t>(au) & 15) == 0 && gemm_tc_eligible(a, b, gau, OJC_BF16, ld, rows, kin, nout) &&
         gemm_tc_swiglu_backward_eligible(be, rows, kin);
}
ojc_status linear_backward_weight_impl(ojc_backend* be, const void* x, int32_t x_dt, const void* gy, int32_t g_dt, float* gw, int64_t rows, int64_t kin,
                                       int64_t nout, bool accumulate) {
  GemmOperand a{gy, g_dt, 1, nout}, b{x, x_dt, kin, 1};
  return gemm_auto(be, "linear_backward", a, b, gw, OJC_F32, kin, nout, kin, rows, 1.0f, accumulate, nullptr);
}

extern "C" {

ojc_status ojc_linear_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, ojc_tensor* y) {
  const char* op = "linear_forward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "weight", w)); OJC_TRY(check_tensor(op, "y", y));
  int64_t rows, kin, nout;
  OJC_TRY(linear_dims(op, x, w, &rows, &kin, &nout));
  if (numel(y) != rows * nout || y->shape[y->rank - 1] != nout) return ojc_fail(OJC_ERR_SHAPE, op, "y must be [..., out]");
  if (!is_float(x) || !is_float(w) || !is_float(y)) return ojc_fail(OJC_ERR_DTYPE, op, "operands must be F32 or BF16");
  return linear_forward_impl(be, x->data, x->dtype, w->data, w->dtype, y->data, y->dtype, rows, kin, nout, nullptr);
}

ojc_status ojc_linear_backward_input(ojc_backend* be, const ojc_tensor* w, const ojc_tensor* gy, ojc_tensor* gx) {
  const char* op = "linear_backward_input";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "weight", w)); OJC_TRY(check_tensor(op, "grad_y", gy)); OJC_TRY(check_tensor(op, "grad_x", gx));
  if (w->rank != 2 || gy->rank < 1 || gy->shape[gy->rank - 1] != w->shape[0] || gx->rank < 1 || gx->shape[gx->rank - 1] != w->shape[1])
    return ojc_fail(OJC_ERR_SHAPE, op, "grad_y [..., out], weight [out, in], grad_x [..., in]");
  const int64_t nout = w->shape[0], kin = w->shape[1];
  if (nout == 0 || kin == 0 || numel(gy) == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  const int64_t rows = numel(gy) / nout;
  if (numel(gx) != rows * kin) return ojc_fail(OJC_ERR_SHAPE, op, "grad_x length differs");
  if (!is_float(w) || !is_float(gy) || !is_float(gx)) return ojc_fail(OJC_ERR_DTYPE, op, "operands must be F32 or BF16");
  return linear_backward_input_impl(be, w->data, w->dtype, gy->data, gy->dtype, gx->data, gx->dtype, rows, kin, nout, false);
}

ojc_status ojc_linear_backward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, const ojc_tensor* gy, ojc_tensor* gx, ojc_tensor* gw) {
  const char* op = "linear_backward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "weight", w)); OJC_TRY(check_tensor(op, "grad_y", gy));
  OJC_TRY(check_tensor(op, "grad_x", gx)); OJC_TRY(check_tensor(op, "grad_w", gw));
  int64_t rows, kin, nout;
  OJC_TRY(linear_dims(op, x, w, &rows, &kin, &nout));
  if (numel(gy) != rows * nout || !same_shape(x, gx) || !same_shape(w, gw)) return ojc_fail(OJC_ERR_SHAPE, op, "grad_y [..., out]; grad_x like x; grad_w like weight");
  if (gw->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "the weight gradient is F32");
  if (!is_float(x) || !is_float(w) || !is_float(gy) || !is_float(gx)) return ojc_fail(OJC_ERR_DTYPE, op, "operands must be F32 or BF16");
  OJC_TRY(linear_backward_input_impl(be, w->data, w->dtype, gy->data, gy->dtype, gx->data, gx->dtype, rows, kin, nout, false));
  return linear_backward_weight_impl(be, x->data, x->dtype, gy->data, gy->dtype, (float*)gw->data, rows, kin, nout, false);
}

}  // extern "C"
