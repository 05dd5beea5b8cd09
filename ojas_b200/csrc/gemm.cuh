// GEMM entry points shared by the linear, fused cross-entropy, gate and Muon code.
#pragma once
#include "common.cuh"

// A strided matrix view: element (i, j) lives at ptr[i * rs + j * cs].
struct GemmOperand {
  const void* ptr;
  int32_t dtype;
  int64_t rs, cs;
};

enum GemmOutMode { GEMM_STORE = 0, GEMM_ACCUMULATE = 1 };

// C[m,n] = alpha * A[m,k] . B[k,n] (+ residual[m,n]) (+ C when accumulate); C row-major with leading dimension ldc.
ojc_status gemm_f32(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                    int64_t n, int64_t k, float alpha, bool accumulate, const float* residual);
// bf16 x bf16 -> f32-accumulated tcgen05 kernel. OJC_ERR_UNSUPPORTED when the operands break the TMA alignment rules.
bool gemm_tc_eligible(const GemmOperand& a, const GemmOperand& b, const void* c, int32_t c_dtype, int64_t ldc, int64_t m, int64_t n, int64_t k);
ojc_status gemm_tc(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                   int64_t n, int64_t k, float alpha, bool accumulate, const float* residual);
// Tensor-core kernel when both operands are bf16 and eligible, the f32 tier otherwise.
ojc_status gemm_auto(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                     int64_t n, int64_t k, float alpha, bool accumulate, const float* residual);
// `batch` independent products of one shape on the tensor-core kernels: matrix i of A / B / C starts a_bs / b_bs / c_bs elements
// after matrix i - 1 (the operand views describe matrix 0). No residual operand; at least 64 output columns.
// An optional epilogue for the Newton-Schulz products in bf16 mode: C = bf16(bf16(src_mul * src) + bf16(acc_mul * bf16(A.B))), with `src`
// a bf16 matrix of C's shape (leading dimension src_ld, matrix stride src_bs). It is the combine step the iteration would otherwise run
// as a kernel of its own after the product, with the same rounding points (ojas-cpu/src/optim.rs:947-974). Needs a bf16 output,
// alpha 1, no accumulation or split, src_ld % 8 == 0 and a 16-byte aligned src; a non-finite result raises the Muon fault.
// allow_split = false keeps a single product's reduction in one piece too, so its bits equal those of the same product inside a batch.
struct NsCombine { const void* src; int64_t src_ld, src_bs; float src_mul, acc_mul; };
// A second optional epilogue, for the input gradient of the MLP's down projection under bf16 autocast: the product A.B is g, the
// gradient of m = bf16(silu(a)) * u, and what is stored is SwiGLU's backward of it, g_a in columns [0, n) and g_u in columns [n, 2n) of C's
// rows, with g rounded to bf16 first (the rounding a stored g would have had; ojas-core/src/autocast.rs emits bf16 from every linear).
// `au` holds a in columns [0, n) and u in columns [n, 2n) of bf16 rows `ld` wide. Single product, n % 64 == 0, alpha 1, no accumulation.
// Two-SM tiles only: gemm_tc_swiglu_backward_eligible says whether a shape qualifies (256 rows and 256 columns or more).
struct SwigluGrad { const void* au; int64_t ld; };
bool gemm_tc_swiglu_backward_eligible(ojc_backend* be, int64_t m, int64_t n);
// And its forward counterpart on the gate/up product, whose B operand is the [gate; up] weight (n = 2 F output columns, C = (a | u)):
// besides a and u the kernel stores m = bf16(silu(a)) * u into `m` (bf16 rows `ldm` wide), computed from the rounded a and u.
// Two-SM tiles only: gemm_tc_swiglu_forward_eligible says whether a shape qualifies (m >= 256 rows, F a multiple of 128).
struct SwigluForward { void* m; int64_t ldm; };
bool gemm_tc_swiglu_forward_eligible(ojc_backend* be, int64_t m, int64_t n, int64_t ldm, const void* mptr);
ojc_status gemm_tc_batched(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                           int64_t n, int64_t k, int64_t batch, int64_t a_bs, int64_t b_bs, int64_t c_bs, float alpha, bool accumulate, const float* residual,
                           const NsCombine* combine = nullptr, bool allow_split = true, const SwigluGrad* swiglu_grad = nullptr,
                           const SwigluForward* swiglu_fwd = nullptr);
