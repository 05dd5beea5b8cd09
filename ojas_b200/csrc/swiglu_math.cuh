// SwiGLU arithmetic of the bf16 tier at one element, shared by the row kernels and by the GEMM epilogue that folds the
// backward pass into the down-projection's input gradient, so both produce the same bits:
//   m = bf16(silu(a)) * u        (silu_forward then mul_forward, each emitting bf16: ojas-core/src/autocast.rs)
//   g_u = g * bf16(silu(a)),  g_a = bf16(g * u) * silu'(a),  silu'(a) = s (1 + a (1 - s)),  s = sigmoid(a)
#pragma once
#include <cstdint>

namespace swiglu {
__device__ __forceinline__ uint32_t pack2(float lo, float hi) { uint32_t r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
__device__ __forceinline__ float round_bf16(float v) { return __uint_as_float(pack2(0.0f, v) & 0xffff0000u); }
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
// both values of a pair rounded to bf16 by one conversion (the conversions are the scarce pipe in the epilogues that use this)
__device__ __forceinline__ void round2_bf16(float& x0, float& x1) {
  const uint32_t r = pack2(x0, x1);
  x0 = __uint_as_float(r << 16); x1 = __uint_as_float(r & 0xffff0000u);
}
// two elements at a time
__device__ __forceinline__ void forward_pair(float a0, float a1, float u0, float u1, float& m0, float& m1) {
  float t0 = a0 * sigmoid_fast(a0), t1 = a1 * sigmoid_fast(a1);
  round2_bf16(t0, t1);
  m0 = t0 * u0; m1 = t1 * u1;
}
__device__ __forceinline__ void backward_pair(float a0, float a1, float u0, float u1, float g0, float g1, float& ga0, float& ga1, float& gu0, float& gu1) {
  const float s0 = sigmoid_fast(a0), s1 = sigmoid_fast(a1);
  float t0 = a0 * s0, t1 = a1 * s1, w0 = g0 * u0, w1 = g1 * u1;
  round2_bf16(t0, t1);
  round2_bf16(w0, w1);
  gu0 = g0 * t0; gu1 = g1 * t1;
  ga0 = w0 * s0 * (1.0f + a0 * (1.0f - s0)); ga1 = w1 * s1 * (1.0f + a1 * (1.0f - s1));
}
}  // namespace swiglu
