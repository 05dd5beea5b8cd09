// f32 GEMM tier on CUDA cores: C[m,n] (+)= alpha * sum_k A(i,k) B(k,j) over strided views. Every output is the reference's
// Exact chain ((0 + a0 b0) + a1 b1) + ... with k ascending and a separately rounded multiply and add per step
// (ojas-cpu/src/gemm.rs:11-16,1044-1083), so with alpha 1 a product here has the bits of the CPU reference's. This is the
// parity tier (and the fallback for shapes the tensor-core kernel's TMA alignment rules exclude); the bf16 performance
// path is gemm_tc.cu.
#include "common.cuh"
#include "dispatch.cuh"
#include "gemm.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <class TA, class TB, class TO>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const TA* __restrict__ A, int64_t ars, int64_t acs, const TB* __restrict__ B, int64_t brs,
                                                       int64_t bcs, TO* __restrict__ C, int64_t ldc, int m, int n, int k, float alpha, int accumulate,
                                                       const float* __restrict__ residual) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = tid / 16, tx = tid % 16;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
  // Load mappings: walk the contiguous axis with consecutive threads.
  const bool a_kfast = (acs == 1), b_nfast = (bcs == 1);
  for (int k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
    for (int l = 0; l < (BM * BK) / 256; ++l) {
      int idx = tid + l * 256;
      int kk = a_kfast ? idx % BK : idx / BM;
      int mm = a_kfast ? idx / BK : idx % BM;
      int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < m && gk < k) ? ldf(A, (int64_t)gm * ars + (int64_t)gk * acs) : 0.0f;
    }
#pragma unroll
    for (int l = 0; l < (BN * BK) / 256; ++l) {
      int idx = tid + l * 256;
      int kk = b_nfast ? idx / BN : idx % BK;
      int nn = b_nfast ? idx % BN : idx / BK;
      int gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < n && gk < k) ? ldf(B, (int64_t)gk * brs + (int64_t)gn * bcs) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));   // never contracted into an fma
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int gm = m0 + ty * TM + i;
    if (gm >= m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int gn = n0 + tx * TN + j;
      if (gn >= n) continue;
      int64_t o = (int64_t)gm * ldc + gn;
      float v = alpha == 1.0f ? acc[i][j] : alpha * acc[i][j];
      if (residual) v = __fadd_rn(v, residual[o]);
      if (accumulate) v = __fadd_rn(v, ldf(C, o));
      stf(C, o, v);
    }
  }
}
}  // namespace

ojc_status gemm_f32(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                    int64_t n, int64_t k, float alpha, bool accumulate, const float* residual) {
  if (m == 0 || n == 0) return OJC_OK;
  dim3 grid((unsigned)((n + BN - 1) / BN), (unsigned)((m + BM - 1) / BM));
  return dispatch_float(op, a.dtype, [&](auto ta) { return dispatch_float(op, b.dtype, [&](auto tb) { return dispatch_float(op, c_dtype, [&](auto to) {
    using TA = decltype(ta); using TB = decltype(tb); using TO = decltype(to);
    gemm_f32_kernel<TA, TB, TO><<<grid, 256, 0, be->stream>>>((const TA*)a.ptr, a.rs, a.cs, (const TB*)b.ptr, b.rs, b.cs, (TO*)c, ldc, (int)m, (int)n, (int)k,
                                                                alpha, accumulate ? 1 : 0, residual);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }); }); });
}
