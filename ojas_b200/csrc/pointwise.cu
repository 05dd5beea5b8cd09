// Memory-bound ops of the block: embedding gather / scatter-add, RMSNorm,
// RoPE, value-residual blend, permute, per-head sigmoid gate, SiLU, mul, add,
// casts, gradient accumulate / scale, argmax. All are coalesced warp-shuffle
// kernels with fixed-order reductions (no float atomics on any output), sized
// as grid-stride launches over a multiple of the SM count.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"
#include "dispatch.cuh"
#include "ops.cuh"

// ======================================================================== elementwise
enum EwOp { EW_SILU, EW_SILU_BWD, EW_MUL, EW_ADD, EW_COPY, EW_ROUND_BF16, EW_SCALE, EW_ACCUM };
// EW_ACCUM is accumulate_grad (ojas-cpu/src/accum.rs:33-115): acc + grad, where a sum that is not finite is not stored and raises the
// deferred fault word instead (the reference refuses the call with NonFinite and leaves acc untouched).

template <int OP, class TA, class TB, class TO>
__global__ void ew_kernel(const TA* __restrict__ a, const TB* __restrict__ b, TO* __restrict__ out, int64_t n, float s, uint32_t* fault) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float x = ldf(a, i), r;
    if (OP == EW_SILU) r = x * sigmoidf_(x);
    else if (OP == EW_SILU_BWD) { float g = ldf(b, i), sg = sigmoidf_(x); r = g * sg * (1.0f + x * (1.0f - sg)); }
    else if (OP == EW_MUL) r = x * ldf(b, i);
    else if (OP == EW_ADD) r = x + ldf(b, i);
    else if (OP == EW_ACCUM) { r = x + ldf(b, i); if (!isfinite(r)) { raise_fault(fault, OP_ACCUMULATE); continue; } }
    else if (OP == EW_ROUND_BF16) r = round_bf16(x);
    else if (OP == EW_SCALE) r = x * s;
    else r = x;
    stf(out, i, r);
  }
}

// 4 elements per thread with 128-bit (f32) / 64-bit (bf16) accesses when n % 4 == 0.
template <class T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void ld(const float* p, int64_t i4, float v[4]) { float4 t = reinterpret_cast<const float4*>(p)[i4]; v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  static __device__ __forceinline__ void st(float* p, int64_t i4, const float v[4]) { reinterpret_cast<float4*>(p)[i4] = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ void ld(const bf16* p, int64_t i4, float v[4]) {
    uint2 t = reinterpret_cast<const uint2*>(p)[i4];
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void st(bf16* p, int64_t i4, const float v[4]) {
    uint2 t;
    t.x = (uint32_t)f32_to_bf16_bits(v[0]) | ((uint32_t)f32_to_bf16_bits(v[1]) << 16);
    t.y = (uint32_t)f32_to_bf16_bits(v[2]) | ((uint32_t)f32_to_bf16_bits(v[3]) << 16);
    reinterpret_cast<uint2*>(p)[i4] = t;
  }
};

template <int OP, class TA, class TB, class TO>
__global__ void ew_kernel_v4(const TA* __restrict__ a, const TB* __restrict__ b, TO* __restrict__ out, int64_t n4, float s, uint32_t* fault) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float x[4], y[4], r[4];
    Vec4<TA>::ld(a, i, x);
    if (OP == EW_SILU_BWD || OP == EW_MUL || OP == EW_ADD || OP == EW_ACCUM) Vec4<TB>::ld(b, i, y);
    bool bad = false;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (OP == EW_SILU) r[k] = x[k] * sigmoidf_(x[k]);
      else if (OP == EW_SILU_BWD) { float sg = sigmoidf_(x[k]); r[k] = y[k] * sg * (1.0f + x[k] * (1.0f - sg)); }
      else if (OP == EW_MUL) r[k] = x[k] * y[k];
      else if (OP == EW_ADD) r[k] = x[k] + y[k];
      else if (OP == EW_ACCUM) { r[k] = x[k] + y[k]; if (!isfinite(r[k])) { bad = true; r[k] = x[k]; } }
      else if (OP == EW_ROUND_BF16) r[k] = round_bf16(x[k]);
      else if (OP == EW_SCALE) r[k] = x[k] * s;
      else r[k] = x[k];
    }
    if (OP == EW_ACCUM && bad) raise_fault(fault, OP_ACCUMULATE);
    Vec4<TO>::st(out, i, r);
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int OP>
static ojc_status launch_ew(ojc_backend* be, const char* op, const ojc_tensor* a, const ojc_tensor* b, ojc_tensor* out, float s = 1.0f) {
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "a", a));
  if (b) { OJC_TRY(check_tensor(op, "b", b)); if (numel(a) != numel(b)) return ojc_fail(OJC_ERR_SHAPE, op, "operand lengths differ"); }
  OJC_TRY(check_tensor(op, "out", out));
  const int64_t n = numel(a);
  if (numel(out) != n) return ojc_fail(OJC_ERR_SHAPE, op, "output length differs");
  if (n == 0) return OJC_OK;
  const ojc_tensor* bb = b ? b : a;
  return dispatch_float(op, a->dtype, [&](auto ta) {
    return dispatch_float(op, bb->dtype, [&](auto tb) {
      return dispatch_float(op, out->dtype, [&](auto to) {
        using TA = decltype(ta); using TB = decltype(tb); using TO = decltype(to);
        const TA* ap = (const TA*)a->data; const TB* bp = (const TB*)bb->data; TO* op_ = (TO*)out->data;
        bool vec = (n % 4 == 0) && aligned16(ap) && aligned16(bp) && aligned16(op_);
        if (vec) ew_kernel_v4<OP, TA, TB, TO><<<elementwise_grid(be, n / 4, 256), 256, 0, be->stream>>>(ap, bp, op_, n / 4, s, be->fault_dev);
        else ew_kernel<OP, TA, TB, TO><<<elementwise_grid(be, n, 256), 256, 0, be->stream>>>(ap, bp, op_, n, s, be->fault_dev);
        OJC_LAUNCHED(be, op);
        return OJC_OK;
      });
    });
  });
}

// ======================================================================== embedding
template <class TT, class TO>
__global__ void embedding_gather_kernel(const TT* __restrict__ table, const uint32_t* __restrict__ ids, TO* __restrict__ out,
                                        int64_t tokens, int64_t dim, int64_t vocab, uint32_t* fault) {
  pdl_trigger();
  // one warp per token row; the row is copied as bits (widened exactly when the table is bf16)
  const int lane = threadIdx.x & 31;
  int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t rstride = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (; row < tokens; row += rstride) {
    uint32_t id = ids[row];
    if (id >= vocab) { if (lane == 0) raise_fault(fault, OP_ID_RANGE); continue; }
    const TT* src = table + (int64_t)id * dim;
    TO* dst = out + row * dim;
    if (dim % 4 == 0) { for (int64_t c = lane; c < dim / 4; c += 32) { float v[4]; Vec4<TT>::ld(src, c, v); Vec4<TO>::st(dst, c, v); } }
    else for (int64_t c = lane; c < dim; c += 32) stf(dst, c, ldf(src, c));
  }
}

__global__ void iota_kernel(uint32_t* out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (uint32_t)i;
}

// One block per vocabulary row: find the row's run in the id-sorted token list
// (stable sort keeps ascending token order) and add the run's gradient rows in
// that order; rows no token selected are written as zero. Every output element
// has one writer, so there are no atomics and no separate zero-fill pass.
template <class TG>
__global__ void embedding_scatter_sorted_kernel(const uint32_t* __restrict__ sorted_ids, const uint32_t* __restrict__ sorted_tok,
                                                const TG* __restrict__ grad, float* __restrict__ out, int64_t tokens,
                                                int64_t dim, int accumulate) {
  const uint32_t v = blockIdx.x;
  int64_t lo = 0, hi = tokens;
  while (lo < hi) { int64_t mid = (lo + hi) >> 1; if (sorted_ids[mid] < v) lo = mid + 1; else hi = mid; }
  for (int64_t c = threadIdx.x; c < dim; c += blockDim.x) {
    float acc = 0.0f;
    for (int64_t p = lo; p < tokens && sorted_ids[p] == v; ++p) acc += ldf(grad, (int64_t)sorted_tok[p] * dim + c);
    float* dst = out + (int64_t)v * dim + c;
    *dst = accumulate ? (*dst + acc) : acc;
  }
}

// The same sums for F32 gradients of 16-byte rows, one warp per vocabulary row: lane 0 finds the row's run and the warp shares it,
// the columns move as float4, and a row no token selected is left alone when the result accumulates into `out` (adding zero to
// every element would only read and rewrite it). Same order of additions per element as the kernel above: the bits are the same.
__global__ void embedding_scatter_sorted_rows_kernel(const uint32_t* __restrict__ sorted_ids, const uint32_t* __restrict__ sorted_tok, const float* __restrict__ grad,
                                                     float* __restrict__ out, int64_t tokens, int64_t vocab, int dim4, int accumulate) {
  const int lane = threadIdx.x & 31;
  const int64_t v = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (v >= vocab) return;
  int64_t lo = 0, n = 0;
  if (lane == 0) {
    int64_t hi = tokens;
    while (lo < hi) { const int64_t mid = (lo + hi) >> 1; if (sorted_ids[mid] < (uint32_t)v) lo = mid + 1; else hi = mid; }
    while (lo + n < tokens && sorted_ids[lo + n] == (uint32_t)v) ++n;
  }
  lo = __shfl_sync(0xffffffffu, lo, 0);
  n = __shfl_sync(0xffffffffu, n, 0);
  if (n == 0 && accumulate) return;
  float4* dst = reinterpret_cast<float4*>(out) + v * dim4;
  for (int c = lane; c < dim4; c += 32) {
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int64_t p = lo; p < lo + n; ++p) {
      const float4 g = reinterpret_cast<const float4*>(grad)[(int64_t)sorted_tok[p] * dim4 + c];
      acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
    }
    if (accumulate) { const float4 o = dst[c]; acc.x = o.x + acc.x; acc.y = o.y + acc.y; acc.z = o.z + acc.z; acc.w = o.w + acc.w; }
    dst[c] = acc;
  }
}

ojc_status embedding_backward_impl(ojc_backend* be, const uint32_t* ids, const void* grad, int32_t grad_dtype, float* out,
                                   int64_t tokens, int64_t vocab, int64_t dim, bool accumulate) {
  const char* op = "embedding_backward";
  size_t cub_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const uint32_t*)nullptr, (uint32_t*)nullptr, (const uint32_t*)nullptr,
                                  (uint32_t*)nullptr, (int)tokens, 0, 32, be->stream);
  uint64_t tok_bytes = ((uint64_t)tokens * 4 + 255) & ~uint64_t(255);
  void* ws = nullptr;
  OJC_TRY(ojc_scratch(be, 3 * tok_bytes + cub_bytes + 256, &ws));
  uint32_t* iota = (uint32_t*)ws;
  uint32_t* sorted_ids = (uint32_t*)((char*)ws + tok_bytes);
  uint32_t* sorted_tok = (uint32_t*)((char*)ws + 2 * tok_bytes);
  void* cub_ws = (char*)ws + 3 * tok_bytes;
  iota_kernel<<<(unsigned)((tokens + 255) / 256), 256, 0, be->stream>>>(iota, tokens);
  OJC_LAUNCHED(be, op);
  int bits = 1; while ((1ll << bits) < vocab && bits < 32) ++bits;
  OJC_CUDA(be, cub::DeviceRadixSort::SortPairs(cub_ws, cub_bytes, ids, sorted_ids, iota, sorted_tok, (int)tokens, 0, bits, be->stream), op);
  be->launches += 2;
  int threads = dim >= 256 ? 256 : (dim >= 128 ? 128 : 64);
  if (grad_dtype == OJC_F32 && dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    embedding_scatter_sorted_rows_kernel<<<(unsigned)((vocab * 32 + 255) / 256), 256, 0, be->stream>>>(sorted_ids, sorted_tok, (const float*)grad, out, tokens, vocab,
                                                                                                      (int)(dim / 4), accumulate ? 1 : 0);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }
  if (grad_dtype == OJC_F32)
    embedding_scatter_sorted_kernel<float><<<(unsigned)vocab, threads, 0, be->stream>>>(sorted_ids, sorted_tok, (const float*)grad, out, tokens, dim, accumulate);
  else
    embedding_scatter_sorted_kernel<bf16><<<(unsigned)vocab, threads, 0, be->stream>>>(sorted_ids, sorted_tok, (const bf16*)grad, out, tokens, dim, accumulate);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

// ======================================================================== RMSNorm
// One warp per row; lane l owns columns l, l+32, ...  y = x * rstd * w with
// rstd = 1 / sqrt(mean(x^2) + eps)  (ojas-cpu/src/norm.rs:24-56,193-204).
template <int ITERS, class TX, class TO>
__global__ void rms_forward_kernel(const TX* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y, int64_t rows,
                                   int dim, float eps, uint32_t* fault, float* __restrict__ copy) {
  const int lane = threadIdx.x & 31;
  int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t rstride = ((int64_t)gridDim.x * blockDim.x) >> 5;
  float wv[ITERS];
#pragma unroll
  for (int j = 0; j < ITERS; ++j) { int c = lane + 32 * j; wv[j] = c < dim ? w[c] : 0.0f; }
  for (; row < rows; row += rstride) {
    const TX* src = x + row * dim;
    float xv[ITERS], ss = 0.0f;
#pragma unroll
    for (int j = 0; j < ITERS; ++j) { int c = lane + 32 * j; xv[j] = c < dim ? ldf(src, c) : 0.0f; ss += xv[j] * xv[j]; }
    ss = warp_sum(ss);
    float denom = ss / (float)dim + eps;
    float rstd = 1.0f / sqrtf(denom);
    if (!(isfinite(denom) && denom > 0.0f && isfinite(rstd))) { if (lane == 0) raise_fault(fault, OP_RMS_NORM); }
#pragma unroll
    for (int j = 0; j < ITERS; ++j) { int c = lane + 32 * j; if (c < dim) stf(y, row * dim + c, xv[j] * rstd * wv[j]); }
    if (copy) {   // the residual stream's next buffer starts as a copy of this one (the following projection adds into it)
#pragma unroll
      for (int j = 0; j < ITERS; ++j) { int c = lane + 32 * j; if (c < dim) copy[row * dim + c] = xv[j]; }
    }
  }
}

// dX per row and per-block partial column sums for dW (ojas-cpu/src/norm.rs:62-127):
// dot = sum (g w)(x rstd); dX = (g w - xhat dot/dim) rstd; dW[c] = sum_rows g xhat.
// Each block writes its partial dW to part[block, dim]; rms_dw_finish_kernel adds
// the partials in block order.
template <int ITERS, class TX, class TG, class TO>
__global__ void rms_backward_kernel(const TX* __restrict__ x, const float* __restrict__ w, const TG* __restrict__ gy,
                                    TO* __restrict__ gx, float* __restrict__ part, int64_t rows, int dim, float eps, int gx_accumulate, bf16* __restrict__ gx_b) {
  extern __shared__ float smem[];  // [warps][dim]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int64_t row = (int64_t)blockIdx.x * nwarps + warp;
  const int64_t rstride = (int64_t)gridDim.x * nwarps;
  float wv[ITERS], dw[ITERS];
#pragma unroll
  for (int j = 0; j < ITERS; ++j) { int c = lane + 32 * j; wv[j] = c < dim ? w[c] : 0.0f; dw[j] = 0.0f; }
  const float inv_dim = 1.0f / (float)dim;
  for (; row < rows; row += rstride) {
    float xv[ITERS], gv[ITERS], old[ITERS], ss = 0.0f;
#pragma unroll
    for (int j = 0; j < ITERS; ++j) {
      int c = lane + 32 * j;
      xv[j] = c < dim ? ldf(x, row * dim + c) : 0.0f;
      gv[j] = c < dim ? ldf(gy, row * dim + c) : 0.0f;
      old[j] = (gx_accumulate && c < dim) ? ldf(gx, row * dim + c) : 0.0f;  // issued with the other loads, not behind the stores
      ss += xv[j] * xv[j];
    }
    ss = warp_sum(ss);
    float rstd = 1.0f / sqrtf(ss * inv_dim + eps);
    float dot = 0.0f;
#pragma unroll
    for (int j = 0; j < ITERS; ++j) dot += (gv[j] * wv[j]) * (xv[j] * rstd);
    dot = warp_sum(dot);
    float mean = dot * inv_dim;
#pragma unroll
    for (int j = 0; j < ITERS; ++j) {
      int c = lane + 32 * j;
      float xhat = xv[j] * rstd;
      dw[j] += gv[j] * xhat;
      const float out = (gv[j] * wv[j] - xhat * mean) * rstd + old[j];
      if (c < dim) { stf(gx, row * dim + c, out); if (gx_b) gx_b[row * dim + c] = __float2bfloat16_rn(out); }   // gx_b: the matmul-operand copy
    }
  }
#pragma unroll
  for (int j = 0; j < ITERS; ++j) { int c = lane + 32 * j; if (c < dim) smem[warp * dim + c] = dw[j]; }
  __syncthreads();
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float acc = 0.0f;
    for (int wi = 0; wi < nwarps; ++wi) acc += smem[wi * dim + c];
    part[(int64_t)blockIdx.x * dim + c] = acc;
  }
}

// out[c] (+)= sum over parts of part[p, c]. Block = 32 columns x 8 part groups; group g adds parts g, g+8, ... in order,
// then the eight group sums are added in group order: a fixed order whatever the grid.
__global__ void column_sum_finish_kernel(const float* __restrict__ part, float* __restrict__ out, int nparts, int cols, int accumulate) {
  __shared__ float red[8][33];
  const int cl = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float acc = 0.0f;
  if (c < cols) for (int p = g; p < nparts; p += 8) acc += part[(int64_t)p * cols + c];
  red[g][cl] = acc;
  __syncthreads();
  if (g == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][cl];
    out[c] = accumulate ? out[c] + t : t;
  }
}

template <class F> static ojc_status dispatch_iters(const char* op, int dim, F&& f) {
  int iters = (dim + 31) / 32;
  if (iters <= 1) return f(std::integral_constant<int, 1>());
  if (iters <= 2) return f(std::integral_constant<int, 2>());
  if (iters <= 4) return f(std::integral_constant<int, 4>());
  if (iters <= 8) return f(std::integral_constant<int, 8>());
  if (iters <= 16) return f(std::integral_constant<int, 16>());
  if (iters <= 24) return f(std::integral_constant<int, 24>());
  if (iters <= 32) return f(std::integral_constant<int, 32>());
  if (iters <= 64) return f(std::integral_constant<int, 64>());
  return ojc_fail(OJC_ERR_UNSUPPORTED, op, "row width above 2048 is not supported");
}

ojc_status rms_forward_impl(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, float eps, ojc_tensor* y, float* copy) {
  const char* op = "rms_norm_forward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "weight", w)); OJC_TRY(check_tensor(op, "y", y));
  if (x->rank < 1 || w->rank != 1 || w->shape[0] != x->shape[x->rank - 1] || !same_shape(x, y)) return ojc_fail(OJC_ERR_SHAPE, op, "x [..., dim], weight [dim], y like x");
  if (w->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "weight must be F32");
  const int dim = (int)w->shape[0];
  const int64_t n = numel(x);
  if (n == 0 || dim == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  const int64_t rows = n / dim;
  if (copy && x->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "the row copy is F32 like its source");
  if (x->dtype == OJC_F32 && y->dtype == OJC_BF16 && rms_backward_rows_supported(dim) &&
      ((reinterpret_cast<uintptr_t>(x->data) | reinterpret_cast<uintptr_t>(y->data) | reinterpret_cast<uintptr_t>(w->data) | reinterpret_cast<uintptr_t>(copy)) & 15) == 0)
    return rms_forward_rows(be, (const float*)x->data, (const float*)w->data, (bf16*)y->data, copy, rows, dim, eps);   // the bf16 step's residual-stream form
  return dispatch_float(op, x->dtype, [&](auto tx) { return dispatch_float(op, y->dtype, [&](auto to) {
    return dispatch_iters(op, dim, [&](auto it) {
      using TX = decltype(tx); using TO = decltype(to); constexpr int IT = decltype(it)::value;
      int grid = elementwise_grid(be, rows * 32, 256);
      rms_forward_kernel<IT, TX, TO><<<grid, 256, 0, be->stream>>>((const TX*)x->data, (const float*)w->data, (TO*)y->data, rows, dim, eps, be->fault_dev, copy);
      OJC_LAUNCHED(be, op);
      return OJC_OK;
    }); }); });
}

ojc_status rms_backward_impl(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, const ojc_tensor* gy, float eps,
                             ojc_tensor* gx, ojc_tensor* gw, bool accumulate_gw, bool accumulate_gx, bf16* gx_b) {
  const char* op = "rms_norm_backward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "weight", w)); OJC_TRY(check_tensor(op, "grad_y", gy));
  OJC_TRY(check_tensor(op, "grad_x", gx)); OJC_TRY(check_tensor(op, "grad_w", gw));
  if (x->rank < 1 || w->rank != 1 || w->shape[0] != x->shape[x->rank - 1] || !same_shape(x, gy) || !same_shape(x, gx) || !same_shape(w, gw))
    return ojc_fail(OJC_ERR_SHAPE, op, "x, grad_y, grad_x [..., dim]; weight, grad_w [dim]");
  if (w->dtype != OJC_F32 || gw->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "weight and grad_w must be F32");
  const int dim = (int)w->shape[0];
  const int64_t n = numel(x);
  if (n == 0 || dim == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  const int64_t rows = n / dim;
  const int warps = dim > 512 ? 4 : 8;
  int64_t blocks = (rows + warps - 1) / warps;
  if (blocks > REDUCE_SMS * 4) blocks = REDUCE_SMS * 4;
  if (x->dtype != gy->dtype || x->dtype != gx->dtype) return ojc_fail(OJC_ERR_DTYPE, op, "x, grad_y and grad_x must share a dtype");
  void* part = nullptr;
  bool on_lane = false;
  cudaStream_t fs = nullptr;
  OJC_TRY(ojc_partials(be, (uint64_t)blocks * dim * 4, &part, &on_lane));
  const bool aligned = ((reinterpret_cast<uintptr_t>(x->data) | reinterpret_cast<uintptr_t>(gy->data) | reinterpret_cast<uintptr_t>(gx->data) |
                         reinterpret_cast<uintptr_t>(w->data) | reinterpret_cast<uintptr_t>(gx_b)) & 15) == 0;
  if (gx_b && x->dtype == OJC_F32 && aligned && rms_backward_rows_supported(dim)) {
    // the residual-stream form of the bf16 step: 128-bit accesses, same arithmetic
    OJC_TRY(rms_backward_rows(be, (const float*)x->data, (const float*)w->data, (const float*)gy->data, (float*)gx->data, gx_b, (float*)part, rows, dim, eps,
                              accumulate_gx, (int)blocks));
    OJC_TRY(ojc_finish_stream(be, on_lane, &fs));
    column_sum_finish_kernel<<<(dim + 31) / 32, 256, 0, fs>>>((const float*)part, (float*)gw->data, (int)blocks, dim, accumulate_gw ? 1 : 0);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }
  OJC_TRY(dispatch_float(op, x->dtype, [&](auto tx) {
    return dispatch_iters(op, dim, [&](auto it) {
      using TX = decltype(tx); constexpr int IT = decltype(it)::value;
      rms_backward_kernel<IT, TX, TX, TX><<<(unsigned)blocks, warps * 32, warps * dim * 4, be->stream>>>(
          (const TX*)x->data, (const float*)w->data, (const TX*)gy->data, (TX*)gx->data, (float*)part, rows, dim, eps, accumulate_gx ? 1 : 0, gx_b);
      OJC_LAUNCHED(be, op);
      return OJC_OK;
    }); }));
  OJC_TRY(ojc_finish_stream(be, on_lane, &fs));
  column_sum_finish_kernel<<<(dim + 31) / 32, 256, 0, fs>>>((const float*)part, (float*)gw->data, (int)blocks, dim, accumulate_gw ? 1 : 0);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

// ======================================================================== RoPE (half split)
// fwd y1 = a c1 + (-b) s1, y2 = b c2 + a s2; bwd d1 = a c1 + b s2, d2 = -a s1 + b c2
// (ojas-cpu/src/norm.rs:271-312); tables [T, dh], row -> (row / heads) % T.
template <class TX, class TO>
__global__ void rope_kernel(const TX* __restrict__ x, const float* __restrict__ cos_t, const float* __restrict__ sin_t, TO* __restrict__ y,
                            int64_t rows, int dim, int64_t time, int64_t heads, int backward) {
  const int half = dim / 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = rows * half, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int64_t row = i / half; int c = (int)(i % half);
    int64_t t = (row / heads) % time;
    float a = ldf(x, row * dim + c), b = ldf(x, row * dim + c + half);
    float c1 = cos_t[t * dim + c], s1 = sin_t[t * dim + c], c2 = cos_t[t * dim + c + half], s2 = sin_t[t * dim + c + half];
    float o1, o2;
    if (!backward) { o1 = a * c1 + (-b) * s1; o2 = b * c2 + a * s2; }
    else { o1 = a * c1 + b * s2; o2 = -a * s1 + b * c2; }
    stf(y, row * dim + c, o1); stf(y, row * dim + c + half, o2);
  }
}

ojc_status rope_impl(ojc_backend* be, const char* op, const ojc_tensor* x, const ojc_tensor* cos_t, const ojc_tensor* sin_t, ojc_tensor* y, int backward) {
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "cos", cos_t)); OJC_TRY(check_tensor(op, "sin", sin_t)); OJC_TRY(check_tensor(op, "y", y));
  if (x->rank != 4 || cos_t->rank != 2 || !same_shape(cos_t, sin_t) || !same_shape(x, y) || cos_t->shape[0] != x->shape[1] ||
      cos_t->shape[1] != x->shape[3] || x->shape[3] % 2 != 0)
    return ojc_fail(OJC_ERR_SHAPE, op, "x [B,T,H,dh] with even dh, tables [T,dh]");
  if (cos_t->dtype != OJC_F32 || sin_t->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "tables must be F32");
  const int64_t rows = x->shape[0] * x->shape[1] * x->shape[2];
  const int dim = (int)x->shape[3];
  if (rows == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  return dispatch_float(op, x->dtype, [&](auto tx) { return dispatch_float(op, y->dtype, [&](auto to) {
    using TX = decltype(tx); using TO = decltype(to);
    rope_kernel<TX, TO><<<elementwise_grid(be, rows * dim / 2, 256), 256, 0, be->stream>>>(
        (const TX*)x->data, (const float*)cos_t->data, (const float*)sin_t->data, (TO*)y->data, rows, dim, x->shape[1], x->shape[2], backward);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }); });
}

// ======================================================================== value residual blend
// s = sigmoid(lambda); y = (1-s) v + s v0; dv = (1-s) g, dv0 = s g,
// dlambda = s (1-s) sum (v0 - v) g   (ojas-cpu/src/pointwise.rs:2031-2146).
template <class TV, class T0, class TO>
__global__ void vres_forward_kernel(const TV* __restrict__ v, const T0* __restrict__ v0, const float* __restrict__ lambda, TO* __restrict__ y, int64_t n) {
  const float s = sigmoidf_(lambda[0]);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) stf(y, i, (1.0f - s) * ldf(v, i) + s * ldf(v0, i));
}

template <class TV, class T0, class TG, class TO>
__global__ void vres_backward_kernel(const TV* __restrict__ v, const T0* __restrict__ v0, const TG* __restrict__ gy, const float* __restrict__ lambda,
                                     TO* __restrict__ gv, TO* __restrict__ gv0, double* __restrict__ part, int64_t n) {
  __shared__ float red[32];
  const float s = sigmoidf_(lambda[0]);
  float acc = 0.0f;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) {
    float g = ldf(gy, i);
    stf(gv, i, (1.0f - s) * g); stf(gv0, i, s * g);
    acc += (ldf(v0, i) - ldf(v, i)) * g;
  }
  float t = block_sum(acc, red);
  if (threadIdx.x == 0) part[blockIdx.x] = (double)t;
}

__global__ void vres_lambda_finish_kernel(const double* __restrict__ part, int nparts, const float* __restrict__ lambda, float* __restrict__ out, int accumulate) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  double acc = 0.0;
  for (int p = 0; p < nparts; ++p) acc += part[p];
  float s = sigmoidf_(lambda[0]);
  float g = (float)(acc * (double)s * (double)(1.0f - s));
  out[0] = accumulate ? out[0] + g : g;
}

// ======================================================================== permute [0,2,1,3]
template <class T>
__global__ void permute_0213_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t d0, int64_t d1, int64_t d2, int64_t d3) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = d0 * d1 * d2 * d3, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {  // i indexes the output [d0, d2, d1, d3]
    int64_t e = i % d3, r = i / d3;
    int64_t b = r % d1; r /= d1;
    int64_t c = r % d2; int64_t a = r / d2;
    y[i] = x[((a * d1 + b) * d2 + c) * d3 + e];
  }
}

// ======================================================================== per-head sigmoid gate
// g = sigmoid(h . Wg^T + b) [rows, H]; out = attn * g broadcast over dh
// (ojas-cpu/src/pointwise.rs:1422-1508). One warp per row.
template <class TI, class TW, class TA, class TO>
__global__ void gate_forward_kernel(const TI* __restrict__ inp, const TW* __restrict__ weight, const float* __restrict__ bias, const TA* __restrict__ attn,
                                    TO* __restrict__ out, float* __restrict__ scales, int64_t rows, int din, int heads, int dh) {
  const int lane = threadIdx.x & 31;
  int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t rstride = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (; row < rows; row += rstride) {
    for (int h = 0; h < heads; ++h) {
      float acc = 0.0f;
      for (int c = lane; c < din; c += 32) acc += ldf(inp, row * din + c) * ldf(weight, (int64_t)h * din + c);
      acc = warp_sum(acc);
      float g = sigmoidf_(acc + bias[h]);
      if (scales && lane == 0) scales[row * heads + h] = g;
      const int64_t base = (row * heads + h) * dh;
      for (int d = lane; d < dh; d += 32) stf(out, base + d, ldf(attn, base + d) * g);
    }
  }
}

// dAttn = gOut * g; gz = (sum_dh gOut * attn) * g (1 - g); dInput = gz . Wg
// (ojas-cpu/src/pointwise.rs:1678-1781). gz is kept for the weight/bias pass.
template <class TI, class TW, class TA, class TG, class TO, class TOI>
__global__ void gate_backward_kernel(const TI* __restrict__ inp, const TW* __restrict__ weight, const float* __restrict__ bias, const TA* __restrict__ attn,
                                     const TG* __restrict__ gout, const float* __restrict__ saved, TO* __restrict__ gattn, TOI* __restrict__ ginp,
                                     float* __restrict__ gz, int64_t rows, int din, int heads, int dh) {
  extern __shared__ float gsm[];  // [warps][heads]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* gzrow = gsm + warp * heads;
  int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t rstride = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (; row < rows; row += rstride) {
    for (int h = 0; h < heads; ++h) {
      float g;
      if (saved) g = saved[row * heads + h];
      else {
        float acc = 0.0f;
        for (int c = lane; c < din; c += 32) acc += ldf(inp, row * din + c) * ldf(weight, (int64_t)h * din + c);
        g = sigmoidf_(warp_sum(acc) + bias[h]);
      }
      const int64_t base = (row * heads + h) * dh;
      float dot = 0.0f;
      for (int d = lane; d < dh; d += 32) { float go = ldf(gout, base + d); dot += go * ldf(attn, base + d); stf(gattn, base + d, go * g); }
      dot = warp_sum(dot);
      float z = dot * g * (1.0f - g);
      if (lane == 0) { gzrow[h] = z; gz[row * heads + h] = z; }
    }
    __syncwarp();
    for (int c = lane; c < din; c += 32) {
      float acc = 0.0f;
      for (int h = 0; h < heads; ++h) acc += gzrow[h] * ldf(weight, (int64_t)h * din + c);
      stf(ginp, row * din + c, acc);
    }
    __syncwarp();
  }
}

// dWg[h, c] = sum_rows gz[r, h] x[r, c]; db[h] = sum_rows gz[r, h]. Block (col tile of 32, row chunk):
// thread (h, c) walks its rows in ascending order; chunk partials are added in order by the finish kernel.
template <class TI>
__global__ void gate_weight_grad_kernel(const float* __restrict__ gz, const TI* __restrict__ inp, float* __restrict__ part, int64_t rows, int din,
                                        int heads, int64_t rows_per_chunk) {
  const int c = blockIdx.x * 32 + (threadIdx.x & 31);
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
  const int cols = din + 1;  // column din holds the bias gradient
  for (int h = threadIdx.x >> 5; h < heads; h += blockDim.x >> 5) {
    float acc = 0.0f;
    if (c < din) for (int64_t r = r0; r < r1; ++r) acc += gz[r * heads + h] * ldf(inp, r * din + c);
    else if (c == din) for (int64_t r = r0; r < r1; ++r) acc += gz[r * heads + h];
    if (c < cols) part[((int64_t)blockIdx.y * heads + h) * cols + c] = acc;
  }
}

__global__ void gate_weight_finish_kernel(const float* __restrict__ part, float* __restrict__ gw, float* __restrict__ gb, int nparts, int din, int heads, int accumulate) {
  const int cols = din + 1;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= heads * cols) return;
  int h = i / cols, c = i % cols;
  float acc = 0.0f;
  for (int p = 0; p < nparts; ++p) acc += part[((int64_t)p * heads + h) * cols + c];
  float* dst = c < din ? &gw[(int64_t)h * din + c] : &gb[h];
  *dst = accumulate ? *dst + acc : acc;
}

// ======================================================================== argmax
__global__ void argmax_rows_kernel(const float* __restrict__ x, uint32_t* __restrict__ out, int64_t rows, int64_t cols, uint32_t* fault) {
  __shared__ float bv[32]; __shared__ int64_t bi[32];
  const int64_t row = blockIdx.x;
  float best = -INFINITY; int64_t idx = INT64_MAX; bool bad = false;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = x[row * cols + c];
    if (!isfinite(v)) bad = true;
    if (v > best || (v == best && c < idx)) { best = v; idx = c; }
  }
  if (bad) raise_fault(fault, OP_ARGMAX);
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o); int64_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
    out[row] = (uint32_t)(idx == INT64_MAX ? 0 : idx);
  }
}

// ======================================================================== SwiGLU (silu . mul fused)
// m = silu(a) * u and its backward in one pass each; equal to silu_forward + mul_forward (and mul_backward +
// silu_backward) including the bf16 rounding of the intermediate when the storage is bf16.
template <class T>
__global__ void swiglu_forward_kernel(const T* __restrict__ a, const T* __restrict__ u, T* __restrict__ m, int64_t n4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n4; i += stride) {
    float av[4], uv[4], r[4];
    Vec4<T>::ld(a, i, av); Vec4<T>::ld(u, i, uv);
#pragma unroll
    for (int k = 0; k < 4; ++k) { float s = av[k] * sigmoidf_(av[k]); if (sizeof(T) == 2) s = round_bf16(s); r[k] = s * uv[k]; }
    Vec4<T>::st(m, i, r);
  }
}
template <class T>
__global__ void swiglu_backward_kernel(const T* __restrict__ a, const T* __restrict__ u, const T* __restrict__ gm, T* __restrict__ ga, T* __restrict__ gu, int64_t n4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n4; i += stride) {
    float av[4], uv[4], gv[4], ra[4], ru[4];
    Vec4<T>::ld(a, i, av); Vec4<T>::ld(u, i, uv); Vec4<T>::ld(gm, i, gv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float sg = sigmoidf_(av[k]);
      float s = av[k] * sg; if (sizeof(T) == 2) s = round_bf16(s);
      ru[k] = gv[k] * s;
      float gs = gv[k] * uv[k]; if (sizeof(T) == 2) gs = round_bf16(gs);
      ra[k] = gs * sg * (1.0f + av[k] * (1.0f - sg));
    }
    Vec4<T>::st(ga, i, ra); Vec4<T>::st(gu, i, ru);
  }
}

ojc_status swiglu_forward_impl(ojc_backend* be, const void* a, const void* u, void* m, int32_t dt, int64_t n) {
  const char* op = "swiglu_forward";
  if (n % 4 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "length must be a multiple of 4");
  return dispatch_float(op, dt, [&](auto t) {
    using T = decltype(t);
    swiglu_forward_kernel<T><<<elementwise_grid(be, n / 4, 256), 256, 0, be->stream>>>((const T*)a, (const T*)u, (T*)m, n / 4);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  });
}
ojc_status swiglu_backward_impl(ojc_backend* be, const void* a, const void* u, const void* gm, void* ga, void* gu, int32_t dt, int64_t n) {
  const char* op = "swiglu_backward";
  if (n % 4 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "length must be a multiple of 4");
  return dispatch_float(op, dt, [&](auto t) {
    using T = decltype(t);
    swiglu_backward_kernel<T><<<elementwise_grid(be, n / 4, 256), 256, 0, be->stream>>>((const T*)a, (const T*)u, (const T*)gm, (T*)ga, (T*)gu, n / 4);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  });
}

// ======================================================================== C ABI
extern "C" {

ojc_status ojc_silu_forward(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y) { return launch_ew<EW_SILU>(be, "silu_forward", x, nullptr, y); }
ojc_status ojc_silu_backward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* gy, ojc_tensor* gx) { return launch_ew<EW_SILU_BWD>(be, "silu_backward", x, gy, gx); }
ojc_status ojc_mul_forward(ojc_backend* be, const ojc_tensor* a, const ojc_tensor* b, ojc_tensor* y) { return launch_ew<EW_MUL>(be, "mul_forward", a, b, y); }
ojc_status ojc_mul_backward(ojc_backend* be, const ojc_tensor* a, const ojc_tensor* b, const ojc_tensor* gy, ojc_tensor* ga, ojc_tensor* gb) {
  OJC_TRY(launch_ew<EW_MUL>(be, "mul_backward", gy, b, ga));
  return launch_ew<EW_MUL>(be, "mul_backward", gy, a, gb);
}
ojc_status ojc_residual_add_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* y, ojc_tensor* out) { return launch_ew<EW_ADD>(be, "residual_add_forward", x, y, out); }
ojc_status ojc_residual_add_backward(ojc_backend* be, const ojc_tensor* g, ojc_tensor* gx, ojc_tensor* gy) {
  OJC_TRY(launch_ew<EW_COPY>(be, "residual_add_backward", g, nullptr, gx));
  return launch_ew<EW_COPY>(be, "residual_add_backward", g, nullptr, gy);
}
ojc_status ojc_accumulate_grad(ojc_backend* be, ojc_tensor* acc, const ojc_tensor* grad) {
  if (acc && grad && !same_shape(acc, grad)) return ojc_fail(OJC_ERR_SHAPE, "accumulate_grad", "shapes differ");
  return launch_ew<EW_ACCUM>(be, "accumulate_grad", acc, grad, acc);
}
ojc_status ojc_scale_grad(ojc_backend* be, ojc_tensor* grad, float scale) {
  if (!isfinite(scale)) return ojc_fail(OJC_ERR_NON_FINITE, "scale_grad", "scale is not finite");
  return launch_ew<EW_SCALE>(be, "scale_grad", grad, nullptr, grad, scale);
}
ojc_status ojc_cast_bf16(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y) {
  if (x && y && (x->dtype != OJC_F32 || y->dtype != OJC_F32)) return ojc_fail(OJC_ERR_DTYPE, "cast_bf16", "F32 storage in and out");
  return launch_ew<EW_ROUND_BF16>(be, "cast_bf16", x, nullptr, y);
}
ojc_status ojc_to_bf16(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y) {
  if (x && y && (x->dtype != OJC_F32 || y->dtype != OJC_BF16)) return ojc_fail(OJC_ERR_DTYPE, "to_bf16", "F32 in, BF16 out");
  return launch_ew<EW_COPY>(be, "to_bf16", x, nullptr, y);
}
ojc_status ojc_to_f32(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y) {
  if (x && y && (x->dtype != OJC_BF16 || y->dtype != OJC_F32)) return ojc_fail(OJC_ERR_DTYPE, "to_f32", "BF16 in, F32 out");
  return launch_ew<EW_COPY>(be, "to_f32", x, nullptr, y);
}

ojc_status ojc_embedding_forward(ojc_backend* be, const ojc_tensor* table, const ojc_tensor* ids, ojc_tensor* out) {
  const char* op = "embedding_forward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "table", table)); OJC_TRY(check_tensor(op, "ids", ids)); OJC_TRY(check_tensor(op, "out", out));
  if (table->rank != 2 || out->rank != ids->rank + 1 || out->shape[out->rank - 1] != table->shape[1]) return ojc_fail(OJC_ERR_SHAPE, op, "table [V,d], ids [...], out [..., d]");
  if (ids->dtype != OJC_U32) return ojc_fail(OJC_ERR_DTYPE, op, "ids must be U32");
  const int64_t tokens = numel(ids), dim = table->shape[1], vocab = table->shape[0];
  if (numel(out) != tokens * dim) return ojc_fail(OJC_ERR_SHAPE, op, "out length differs");
  if (tokens == 0 || dim == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  return dispatch_float(op, table->dtype, [&](auto tt) { return dispatch_float(op, out->dtype, [&](auto to) {
    using TT = decltype(tt); using TO = decltype(to);
    embedding_gather_kernel<TT, TO><<<elementwise_grid(be, tokens * 32, 256), 256, 0, be->stream>>>(
        (const TT*)table->data, (const uint32_t*)ids->data, (TO*)out->data, tokens, dim, vocab, be->fault_dev);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }); });
}

ojc_status ojc_embedding_backward(ojc_backend* be, const ojc_tensor* table, const ojc_tensor* ids, const ojc_tensor* grad_out, ojc_tensor* grad_table) {
  const char* op = "embedding_backward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "ids", ids)); OJC_TRY(check_tensor(op, "grad_out", grad_out)); OJC_TRY(check_tensor(op, "grad_table", grad_table));
  if (!table || table->rank != 2 || !same_shape(table, grad_table) || grad_out->shape[grad_out->rank - 1] != table->shape[1] ||
      numel(grad_out) != numel(ids) * table->shape[1])
    return ojc_fail(OJC_ERR_SHAPE, op, "table [V,d], ids [...], grad_out [..., d], grad_table [V,d]");
  if (ids->dtype != OJC_U32 || grad_table->dtype != OJC_F32 || !is_float(grad_out)) return ojc_fail(OJC_ERR_DTYPE, op, "ids U32, grad_table F32");
  if (numel(ids) == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  return embedding_backward_impl(be, (const uint32_t*)ids->data, grad_out->data, grad_out->dtype, (float*)grad_table->data,
                                 numel(ids), table->shape[0], table->shape[1], false);
}

ojc_status ojc_rms_norm_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, float eps, ojc_tensor* y) { return rms_forward_impl(be, x, w, eps, y); }
ojc_status ojc_rms_norm_backward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, const ojc_tensor* gy, float eps, ojc_tensor* gx, ojc_tensor* gw) {
  return rms_backward_impl(be, x, w, gy, eps, gx, gw, false, false);
}
ojc_status ojc_rms_qk_norm_forward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* qw, const ojc_tensor* kw, float eps, ojc_tensor* qo, ojc_tensor* ko) {
  OJC_TRY(rms_forward_impl(be, q, qw, eps, qo));
  return rms_forward_impl(be, k, kw, eps, ko);
}
ojc_status ojc_rms_qk_norm_backward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* qw, const ojc_tensor* kw, const ojc_tensor* gq,
                                    const ojc_tensor* gk, float eps, ojc_tensor* gqi, ojc_tensor* gki, ojc_tensor* gqw, ojc_tensor* gkw) {
  OJC_TRY(rms_backward_impl(be, q, qw, gq, eps, gqi, gqw, false, false));
  return rms_backward_impl(be, k, kw, gk, eps, gki, gkw, false, false);
}
ojc_status ojc_rope_half_split_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* c, const ojc_tensor* s, ojc_tensor* y) { return rope_impl(be, "rope_half_split_forward", x, c, s, y, 0); }
ojc_status ojc_rope_half_split_backward(ojc_backend* be, const ojc_tensor* g, const ojc_tensor* c, const ojc_tensor* s, ojc_tensor* gx) { return rope_impl(be, "rope_half_split_backward", g, c, s, gx, 1); }

ojc_status ojc_value_residual_blend_forward(ojc_backend* be, const ojc_tensor* v, const ojc_tensor* v0, const ojc_tensor* lambda, ojc_tensor* y) {
  const char* op = "value_residual_blend_forward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "v", v)); OJC_TRY(check_tensor(op, "v0", v0)); OJC_TRY(check_tensor(op, "lambda", lambda)); OJC_TRY(check_tensor(op, "y", y));
  if (!same_shape(v, v0) || !same_shape(v, y) || numel(lambda) != 1) return ojc_fail(OJC_ERR_SHAPE, op, "v, v0, y alike; lambda [1]");
  if (lambda->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "lambda must be F32");
  const int64_t n = numel(v);
  if (n == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  if (v->dtype != v0->dtype) return ojc_fail(OJC_ERR_DTYPE, op, "v and v0 must share a dtype");
  return dispatch_float(op, v->dtype, [&](auto tv) { return dispatch_float(op, y->dtype, [&](auto to) {
    using TV = decltype(tv); using TO = decltype(to);
    vres_forward_kernel<TV, TV, TO><<<elementwise_grid(be, n, 256), 256, 0, be->stream>>>((const TV*)v->data, (const TV*)v0->data, (const float*)lambda->data, (TO*)y->data, n);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }); });
}

}  // extern "C"

ojc_status vres_backward_impl(ojc_backend* be, const ojc_tensor* v, const ojc_tensor* v0, const ojc_tensor* lambda, const ojc_tensor* gy, ojc_tensor* gv,
                              ojc_tensor* gv0, float* glambda, bool accumulate_lambda) {
  const char* op = "value_residual_blend_backward";
  const int64_t n = numel(v);
  int blocks = REDUCE_SMS * 4;
  void* part = nullptr;
  OJC_TRY(ojc_scratch(be, (uint64_t)blocks * 8, &part));
  if (v->dtype != v0->dtype || gy->dtype != gv->dtype) return ojc_fail(OJC_ERR_DTYPE, op, "v/v0 and grad_y/grad_v must pair up in dtype");
  OJC_TRY(dispatch_float(op, v->dtype, [&](auto tv) { return dispatch_float(op, gy->dtype, [&](auto tg) {
    using TV = decltype(tv); using TG = decltype(tg);
    vres_backward_kernel<TV, TV, TG, TG><<<blocks, 256, 0, be->stream>>>((const TV*)v->data, (const TV*)v0->data, (const TG*)gy->data, (const float*)lambda->data,
                                                                        (TG*)gv->data, (TG*)gv0->data, (double*)part, n);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }); }));
  vres_lambda_finish_kernel<<<1, 32, 0, be->stream>>>((const double*)part, blocks, (const float*)lambda->data, glambda, accumulate_lambda ? 1 : 0);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

extern "C" {

ojc_status ojc_value_residual_blend_backward(ojc_backend* be, const ojc_tensor* v, const ojc_tensor* v0, const ojc_tensor* lambda, const ojc_tensor* gy,
                                             ojc_tensor* gv, ojc_tensor* gv0, ojc_tensor* glambda) {
  const char* op = "value_residual_blend_backward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "v", v)); OJC_TRY(check_tensor(op, "v0", v0)); OJC_TRY(check_tensor(op, "lambda", lambda)); OJC_TRY(check_tensor(op, "grad_y", gy));
  OJC_TRY(check_tensor(op, "grad_v", gv)); OJC_TRY(check_tensor(op, "grad_v0", gv0)); OJC_TRY(check_tensor(op, "grad_lambda", glambda));
  if (!same_shape(v, v0) || !same_shape(v, gy) || !same_shape(v, gv) || !same_shape(v, gv0) || numel(lambda) != 1 || numel(glambda) != 1)
    return ojc_fail(OJC_ERR_SHAPE, op, "v, v0, grads alike; lambda [1]");
  if (lambda->dtype != OJC_F32 || glambda->dtype != OJC_F32 || gv->dtype != gv0->dtype) return ojc_fail(OJC_ERR_DTYPE, op, "lambda F32; grad_v and grad_v0 share a dtype");
  if (numel(v) == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  return vres_backward_impl(be, v, v0, lambda, gy, gv, gv0, (float*)glambda->data, false);
}

ojc_status ojc_permute(ojc_backend* be, const ojc_tensor* x, const int32_t* dims, int32_t ndims, ojc_tensor* y) {
  const char* op = "permute";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "y", y));
  if (ndims != 4 || x->rank != 4 || y->rank != 4 || dims[0] != 0 || dims[1] != 2 || dims[2] != 1 || dims[3] != 3)
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "only the [0,2,1,3] permutation of a rank-4 tensor is on this path");
  if (y->shape[0] != x->shape[0] || y->shape[1] != x->shape[2] || y->shape[2] != x->shape[1] || y->shape[3] != x->shape[3]) return ojc_fail(OJC_ERR_SHAPE, op, "y must be x with axes 1 and 2 swapped");
  if (x->dtype != y->dtype) return ojc_fail(OJC_ERR_DTYPE, op, "permute keeps the dtype");
  const int64_t n = numel(x);
  if (n == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  if (dtype_size(x->dtype) == 4)
    permute_0213_kernel<uint32_t><<<elementwise_grid(be, n, 256), 256, 0, be->stream>>>((const uint32_t*)x->data, (uint32_t*)y->data, x->shape[0], x->shape[1], x->shape[2], x->shape[3]);
  else
    permute_0213_kernel<uint16_t><<<elementwise_grid(be, n, 256), 256, 0, be->stream>>>((const uint16_t*)x->data, (uint16_t*)y->data, x->shape[0], x->shape[1], x->shape[2], x->shape[3]);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

static ojc_status gate_dims(const char* op, const ojc_tensor* input, const ojc_tensor* weight, const ojc_tensor* bias, const ojc_tensor* attn, int64_t* rows, int* din, int* heads, int* dh) {
  OJC_TRY(check_tensor(op, "input", input)); OJC_TRY(check_tensor(op, "weight", weight)); OJC_TRY(check_tensor(op, "bias", bias)); OJC_TRY(check_tensor(op, "attn", attn));
  if (weight->rank != 2 || bias->rank != 1 || bias->shape[0] != weight->shape[0] || input->rank < 1 || input->shape[input->rank - 1] != weight->shape[1])
    return ojc_fail(OJC_ERR_SHAPE, op, "input [..., d], weight [H, d], bias [H]");
  *din = (int)weight->shape[1]; *heads = (int)weight->shape[0];
  if (*din == 0 || *heads == 0 || numel(input) == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  *rows = numel(input) / *din;
  int64_t per = numel(attn) / (*rows * *heads);
  if (per * *rows * *heads != numel(attn) || per == 0) return ojc_fail(OJC_ERR_SHAPE, op, "attn must be [rows, H, dh]");
  *dh = (int)per;
  if (bias->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "bias must be F32");
  return OJC_OK;
}

ojc_status ojc_per_head_sigmoid_gate_forward(ojc_backend* be, const ojc_tensor* input, const ojc_tensor* weight, const ojc_tensor* bias, const ojc_tensor* attn,
                                             ojc_tensor* out, ojc_tensor* scales) {
  const char* op = "per_head_sigmoid_gate_forward";
  OJC_ALIVE(be, op);
  int64_t rows = 0; int din = 0, heads = 0, dh = 0;
  OJC_TRY(gate_dims(op, input, weight, bias, attn, &rows, &din, &heads, &dh));
  OJC_TRY(check_tensor(op, "out", out));
  if (numel(out) != numel(attn)) return ojc_fail(OJC_ERR_SHAPE, op, "out must match attn");
  if (scales && (numel(scales) != rows * heads || scales->dtype != OJC_F32)) return ojc_fail(OJC_ERR_SHAPE, op, "scales must be F32 [rows, H]");
  if (input->dtype != weight->dtype || input->dtype != attn->dtype || input->dtype != out->dtype) return ojc_fail(OJC_ERR_DTYPE, op, "input, weight, attn and out must share a dtype");
  return dispatch_float(op, input->dtype, [&](auto ti) {
    using T = decltype(ti);
    gate_forward_kernel<T, T, T, T><<<elementwise_grid(be, rows * 32, 256), 256, 0, be->stream>>>(
        (const T*)input->data, (const T*)weight->data, (const float*)bias->data, (const T*)attn->data, (T*)out->data,
        scales ? (float*)scales->data : nullptr, rows, din, heads, dh);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  });
}

}  // extern "C"

ojc_status gate_backward_impl(ojc_backend* be, const ojc_tensor* input, const ojc_tensor* weight, const ojc_tensor* bias, const ojc_tensor* attn, const ojc_tensor* gout,
                              const ojc_tensor* saved, ojc_tensor* ginput, float* gweight, float* gbias, ojc_tensor* gattn, bool accumulate_w) {
  const char* op = "per_head_sigmoid_gate_backward";
  int64_t rows = 0; int din = 0, heads = 0, dh = 0;
  OJC_TRY(gate_dims(op, input, weight, bias, attn, &rows, &din, &heads, &dh));
  if (heads > 64) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "more than 64 heads");
  const int64_t rows_per_chunk = 256;
  const int64_t chunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
  const uint64_t gz_bytes = ((uint64_t)rows * heads * 4 + 255) & ~uint64_t(255);
  void* ws = nullptr;
  OJC_TRY(ojc_scratch(be, gz_bytes + (uint64_t)chunks * heads * (din + 1) * 4, &ws));
  float* gz = (float*)ws;
  float* part = (float*)((char*)ws + gz_bytes);
  if (input->dtype != weight->dtype || input->dtype != attn->dtype || input->dtype != gout->dtype || input->dtype != gattn->dtype)
    return ojc_fail(OJC_ERR_DTYPE, op, "input, weight, attn, grad_out and grad_attn must share a dtype");
  OJC_TRY(dispatch_float(op, input->dtype, [&](auto ti) { return dispatch_float(op, ginput->dtype, [&](auto toi) {
      using T = decltype(ti); using TOI = decltype(toi);
      const int warps = 8;
      gate_backward_kernel<T, T, T, T, T, TOI><<<elementwise_grid(be, rows * 32, warps * 32), warps * 32, warps * heads * 4, be->stream>>>(
          (const T*)input->data, (const T*)weight->data, (const float*)bias->data, (const T*)attn->data, (const T*)gout->data,
          saved ? (const float*)saved->data : nullptr, (T*)gattn->data, (TOI*)ginput->data, gz, rows, din, heads, dh);
      OJC_LAUNCHED(be, op);
      dim3 grid((din + 1 + 31) / 32, (unsigned)chunks);
      gate_weight_grad_kernel<T><<<grid, 32 * (heads < 8 ? heads : 8), 0, be->stream>>>(gz, (const T*)input->data, part, rows, din, heads, rows_per_chunk);
      OJC_LAUNCHED(be, op);
      return OJC_OK;
    }); }));
  gate_weight_finish_kernel<<<(heads * (din + 1) + 127) / 128, 128, 0, be->stream>>>(part, gweight, gbias, (int)chunks, din, heads, accumulate_w ? 1 : 0);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

extern "C" {

ojc_status ojc_per_head_sigmoid_gate_backward(ojc_backend* be, const ojc_tensor* input, const ojc_tensor* weight, const ojc_tensor* bias, const ojc_tensor* attn,
                                              const ojc_tensor* gout, const ojc_tensor* saved, ojc_tensor* ginput, ojc_tensor* gweight, ojc_tensor* gbias, ojc_tensor* gattn) {
  const char* op = "per_head_sigmoid_gate_backward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "grad_out", gout)); OJC_TRY(check_tensor(op, "grad_input", ginput)); OJC_TRY(check_tensor(op, "grad_weight", gweight));
  OJC_TRY(check_tensor(op, "grad_bias", gbias)); OJC_TRY(check_tensor(op, "grad_attn", gattn));
  if (!same_shape(input, ginput) || !same_shape(weight, gweight) || !same_shape(bias, gbias) || numel(attn) != numel(gattn) || numel(attn) != numel(gout))
    return ojc_fail(OJC_ERR_SHAPE, op, "each gradient must match its operand");
  if (gweight->dtype != OJC_F32 || gbias->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "weight and bias gradients are F32");
  if (saved && saved->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "saved scales are F32");
  return gate_backward_impl(be, input, weight, bias, attn, gout, saved, ginput, (float*)gweight->data, (float*)gbias->data, gattn, false);
}

ojc_status ojc_argmax_rows(ojc_backend* be, const ojc_tensor* x, ojc_tensor* out) {
  const char* op = "argmax_rows";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "out", out));
  if (x->rank != 2 || out->rank != 1 || out->shape[0] != x->shape[0]) return ojc_fail(OJC_ERR_SHAPE, op, "x [rows, cols], out [rows]");
  if (x->dtype != OJC_F32 || out->dtype != OJC_U32) return ojc_fail(OJC_ERR_DTYPE, op, "x F32, out U32");
  if (x->shape[0] == 0 || x->shape[1] == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  argmax_rows_kernel<<<(unsigned)x->shape[0], 256, 0, be->stream>>>((const float*)x->data, (uint32_t*)out->data, x->shape[0], x->shape[1], be->fault_dev);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

}  // extern "C"

// ======================================================================== RMSNorm backward without any allocation
// Workspace for ojc_rms_norm_backward_noalloc: the per-block partial column sums of dW live in this fixed array instead
// of the backend's growable workspace. Every GPU that loads the library holds these 2 MiB until the process exits.
constexpr int64_t NOALLOC_PART_FLOATS = 1 << 19;
static __device__ __align__(256) float g_rms_noalloc_part[NOALLOC_PART_FLOATS];
// In host code the array's name is only a stand-in for the symbol: the device address is looked up once per device.
static float* g_rms_noalloc_ptr[64] = {nullptr};

extern "C" ojc_status ojc_rms_norm_backward_noalloc(void* cuda_stream, const float* x, const float* weight, const float* grad_y, int64_t rows, int64_t dim,
                                                    float eps, float* grad_x, float* grad_w) {
  const char* op = "rms_norm_backward_noalloc";
  if (!x || !weight || !grad_y || !grad_x || !grad_w) return ojc_fail(OJC_ERR_PLACEMENT, op, "every operand must be a device pointer");
  if (rows <= 0 || dim <= 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  if (dim > 2048) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "row width above 2048 is not supported");
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) { cudaGetLastError(); return ojc_fail(OJC_ERR_NO_DEVICE, op, "no current CUDA device"); }
  if (!g_rms_noalloc_ptr[device]) {
    // first call on this device: resolve the symbol with this device current (do this before any stream capture)
    float* p = nullptr;
    cudaError_t err = cudaGetSymbolAddress((void**)&p, g_rms_noalloc_part);
    if (err != cudaSuccess || !p) { cudaGetLastError(); return ojc_fail(OJC_ERR_BACKEND, op, std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(err)); }
    g_rms_noalloc_ptr[device] = p;
  }
  float* part = g_rms_noalloc_ptr[device];
  const int warps = dim > 512 ? 4 : 8;
  int64_t blocks = (rows + warps - 1) / warps;
  if (blocks > (int64_t)REDUCE_SMS * 4) blocks = (int64_t)REDUCE_SMS * 4;
  if (blocks * dim > NOALLOC_PART_FLOATS) blocks = NOALLOC_PART_FLOATS / dim;  // fewer, longer blocks rather than a larger workspace
  if (blocks < 1 || rows > (int64_t)INT32_MAX * warps) return ojc_fail(OJC_ERR_CAPACITY_EXCEEDED, op, "the problem does not fit the fixed 2 MiB workspace");
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  ojc_status st = dispatch_iters(op, (int)dim, [&](auto it) {
    constexpr int IT = decltype(it)::value;
    // every launched block overwrites its own row of the workspace and the finish kernel reads exactly those rows,
    // so nothing left by an earlier call is ever read and nothing needs clearing
    rms_backward_kernel<IT, float, float, float><<<(unsigned)blocks, warps * 32, warps * (int)dim * 4, stream>>>(x, weight, grad_y, grad_x, part, rows, (int)dim, eps, 0, nullptr);
    return OJC_OK;
  });
  if (st != OJC_OK) return st;
  column_sum_finish_kernel<<<(unsigned)((dim + 31) / 32), 256, 0, stream>>>(part, grad_w, (int)blocks, (int)dim, 0);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return ojc_fail(OJC_ERR_BACKEND, op, std::string(cudaGetErrorName(err)) + ": " + cudaGetErrorString(err));
  return OJC_OK;
}
