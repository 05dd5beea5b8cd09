// Runtime dtype -> compile-time type dispatch for the float storage types.
#pragma once
#include "common.cuh"

template <class F>
static inline ojc_status dispatch_float(const char* op, int32_t dtype, F&& f) {
  if (dtype == OJC_F32) return f(float());
  if (dtype == OJC_BF16) return f(bf16());
  return ojc_fail(OJC_ERR_DTYPE, op, "operand must be F32 or BF16");
}
