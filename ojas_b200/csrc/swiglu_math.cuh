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
__device__ __forceinline__ float forward_elem(float a, float u) { return round_bf16(a * sigmoid_fast(a)) * u; }
__device__ __forceinline__ void backward_elem(float a, float u, float g, float& ga, float& gu) {
  const float sg = sigmoid_fast(a);
  gu = g * round_bf16(a * sg);
  ga = round_bf16(g * u) * sg * (1.0f + a * (1.0f - sg));
}
}  // namespace swiglu
