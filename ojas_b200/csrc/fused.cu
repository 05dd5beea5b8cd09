// Fused forms the step driver uses under bf16 autocast, each equal to a short chain of the per-op entry points:
//   qk_norm_rope_forward / backward   rms_norm (per head, weight [dh]) followed by rope_half_split, one pass over q or k
//   gate_apply_forward / backward     the pointwise half of per_head_sigmoid_gate once the [rows, H] logits come from a GEMM
// 128-bit accesses throughout; per-column weight-gradient sums are two-stage with a fixed order (no float atomics).
#include "common.cuh"
#include "ops.cuh"
#include "swiglu_math.cuh"

namespace {

// hardware round-to-nearest-even conversions and approximate sigmoid: these kernels only run in the bf16 tier
using swiglu::pack2;
using swiglu::sigmoid_fast;
__device__ __forceinline__ float rbf(float v) { return swiglu::round_bf16(v); }

__device__ __forceinline__ void load8(const bf16* p, float v[8]) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
__device__ __forceinline__ void store8(bf16* p, const float v[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
}
__device__ __forceinline__ void load8f(const float* p, float v[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <int TPR> __device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// y = rope(rms_norm(x) * w). x, y: [tokens, heads, dh] with a token stride (so a column slice of a wider buffer works);
// cos_t / sin_t: [time, dh] tables whose second half of columns repeats the first, as the step driver builds them (block.rs:62-85).
// TPR = dh / 16 threads per (token, head lane), each owning columns [8 part, 8 part + 8) of both halves, i.e. whole rotation
// pairs, and walking every HL-th head: the weight, cosine and sine values it needs are the same for every head of its token,
// and the HL heads side by side make one warp load cover HL * 128 contiguous bytes of a token's row (DRAM page locality).
template <int TPR, int HL>
__global__ void qk_norm_rope_forward_kernel(const bf16* __restrict__ x, int64_t xs, const float* __restrict__ w, const float* __restrict__ cos_t,
                                            const float* __restrict__ sin_t, bf16* __restrict__ y, int64_t ys, int64_t tokens, int heads, int time, float eps) {
  pdl_trigger();
  constexpr int DH = 16 * TPR, HALF = 8 * TPR;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int part = (int)(gid % TPR), hsub = (int)((gid / TPR) % HL);   // HL heads side by side in a warp: one load covers HL * 128 contiguous bytes per token
  const int64_t tok_raw = gid / (TPR * HL);
  const bool live = tok_raw < tokens;
  const int64_t token = live ? tok_raw : tokens - 1;
  const int t = (int)(token % time), c0 = part * 8;
  // the rotation tables repeat their first half in their second (one frequency per pair of columns i, i + HALF): one load serves both
  float wa[8], wb[8], c1[8], s1[8];
  load8f(w + c0, wa); load8f(w + HALF + c0, wb);
  load8f(cos_t + (int64_t)t * DH + c0, c1);
  load8f(sin_t + (int64_t)t * DH + c0, s1);
  const bf16* src = x + token * xs + c0;
  bf16* dst = y + token * ys + c0;
#pragma unroll 4
  for (int head = hsub; head < heads; head += HL) {
    float a[8], b[8];
    load8(src + head * DH, a); load8(src + head * DH + HALF, b);
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
    ss = row_sum<TPR>(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)DH + eps);
    float y1[8], y2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float an = a[i] * rstd * wa[i], bn = b[i] * rstd * wb[i];
      y1[i] = an * c1[i] - bn * s1[i];
      y2[i] = bn * c1[i] + an * s1[i];
    }
    if (live) { store8(dst + head * DH, y1); store8(dst + head * DH + HALF, y2); }
  }
}

// Backward of the above from the saved pre-norm x: rope backward, then RMSNorm backward; dW partials per block. The same
// thread-per-(token, part) walk over the heads; the weight-gradient terms accumulate in registers across heads and tokens.
template <int TPR, int HL>
__global__ void __launch_bounds__(128, 4) qk_norm_rope_backward_kernel(const bf16* __restrict__ x, int64_t xs, const float* __restrict__ w, const float* __restrict__ cos_t,
                                             const float* __restrict__ sin_t, const bf16* __restrict__ gy, int64_t gys, bf16* __restrict__ gx, int64_t gxs,
                                             float* __restrict__ part_out, int64_t tokens, int heads, int time, float eps) {
  pdl_trigger();
  constexpr int DH = 16 * TPR, HALF = 8 * TPR;
  extern __shared__ float red[];  // [threads][16]
  const int part = threadIdx.x % TPR, hsub = (threadIdx.x / TPR) % HL, tok_in_block = threadIdx.x / (TPR * HL);
  const int c0 = part * 8;
  float wa[8], wb[8], dwa[8], dwb[8];
  load8f(w + c0, wa); load8f(w + HALF + c0, wb);
#pragma unroll
  for (int i = 0; i < 8; ++i) { dwa[i] = 0.0f; dwb[i] = 0.0f; }
  const int64_t tok_per_pass = (int64_t)gridDim.x * (blockDim.x / (TPR * HL));
  const int64_t passes = (tokens + tok_per_pass - 1) / tok_per_pass;
  for (int64_t pass = 0; pass < passes; ++pass) {
    const int64_t tok_raw = pass * tok_per_pass + (int64_t)blockIdx.x * (blockDim.x / (TPR * HL)) + tok_in_block;
    const bool live = tok_raw < tokens;
    const int64_t token = live ? tok_raw : tokens - 1;
    const int t = (int)(token % time);
    float c1[8], s1[8];                        // both halves of the tables hold the same values
    load8f(cos_t + (int64_t)t * DH + c0, c1);
    load8f(sin_t + (int64_t)t * DH + c0, s1);
    const bf16* xsrc = x + token * xs + c0;
    const bf16* gsrc = gy + token * gys + c0;
    bf16* dst = gx + token * gxs + c0;
#pragma unroll 2
    for (int head = hsub; head < heads; head += HL) {
      float a[8], b[8], ga[8], gb[8];
      load8(xsrc + head * DH, a); load8(xsrc + head * DH + HALF, b);
      load8(gsrc + head * DH, ga); load8(gsrc + head * DH + HALF, gb);
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
      ss = row_sum<TPR>(ss);
      const float rstd = 1.0f / sqrtf(ss / (float)DH + eps);
      float da[8], db[8], dot = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        da[i] = ga[i] * c1[i] + gb[i] * s1[i];    // d/d(an): rope backward (ojas-cpu/src/norm.rs:303-306)
        db[i] = -ga[i] * s1[i] + gb[i] * c1[i];
        a[i] *= rstd; b[i] *= rstd;               // x hat
        dot += (da[i] * wa[i]) * a[i] + (db[i] * wb[i]) * b[i];
      }
      dot = row_sum<TPR>(dot);
      const float mean = dot / (float)DH;
      float oa[8], ob[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        oa[i] = (da[i] * wa[i] - a[i] * mean) * rstd;
        ob[i] = (db[i] * wb[i] - b[i] * mean) * rstd;
        if (live) { dwa[i] += da[i] * a[i]; dwb[i] += db[i] * b[i]; }
      }
      if (live) { store8(dst + head * DH, oa); store8(dst + head * DH + HALF, ob); }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) { red[threadIdx.x * 16 + i] = dwa[i]; red[threadIdx.x * 16 + 8 + i] = dwb[i]; }
  __syncthreads();
  if (threadIdx.x < DH) {
    const int c = threadIdx.x, p = (c % HALF) / 8, slot = (c / HALF) * 8 + (c % 8);
    float acc = 0.0f;
    for (int th = p; th < (int)blockDim.x; th += TPR) acc += red[th * 16 + slot];
    part_out[(int64_t)blockIdx.x * DH + c] = acc;
  }
}

__global__ void fused_column_sum_kernel(const float* __restrict__ part, float* __restrict__ out, int nparts, int cols) {
  __shared__ float red[8][33];
  const int cl = threadIdx.x & 31, g = threadIdx.x >> 5, c = blockIdx.x * 32 + cl;
  float acc = 0.0f;
  if (c < cols) for (int p = g; p < nparts; p += 8) acc += part[(int64_t)p * cols + c];
  red[g][cl] = acc;
  __syncthreads();
  if (g == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][cl];
    out[c] = t;
  }
}

// out = attn * sigmoid(z + b) per head; z: [rows, zld] logits (zld >= heads), scales (optional) keeps the sigmoid.
// One thread per 8 contiguous values of one (row, head).
__global__ void gate_apply_forward_kernel(const bf16* __restrict__ z, int zld, const bf16* __restrict__ attn, const float* __restrict__ bias, bf16* __restrict__ out,
                                          float* __restrict__ scales, int64_t rows, int heads, int dh) {
  pdl_trigger();
  // threadIdx.x walks the 16-byte chunks of a token's row, threadIdx.y the tokens: a thread's head is fixed, no division per element
  const int per = dh / 8, chunks = heads * per;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const int h = c / per;
    const bool first = c % per == 0;
    const float bh = bias[h];
    for (int64_t row = (int64_t)blockIdx.x * blockDim.y + threadIdx.y; row < rows; row += (int64_t)gridDim.x * blockDim.y) {
      const float g = sigmoid_fast(__bfloat162float(z[row * zld + h]) + bh);
      if (scales && first) scales[row * heads + h] = g;
      const int64_t off = (row * chunks + c) * 8;
      float v[8];
      load8(attn + off, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= g;
      store8(out + off, v);
    }
  }
}

// dAttn = gOut * g; gz[row, h] = (sum_dh gOut * attn) * g (1 - g), written as bf16 [rows, zld] with zero padding columns
// (the operand of the two gate GEMMs) and as f32 partial column sums for the bias gradient. One warp per row.
// With `dr`: also Dr[b, h, t] = sum_dh dAttn * attn = g * (sum_dh gOut * attn), the row statistic the attention backward needs
// (rows are tokens b * time + t), which saves that op a pass over attn and dAttn.
__global__ void gate_apply_backward_kernel(const float* __restrict__ scales, const bf16* __restrict__ attn, const bf16* __restrict__ gout, bf16* __restrict__ gattn,
                                           bf16* __restrict__ gz, int zld, float* __restrict__ part_out, int64_t rows, int heads, int dh, float* __restrict__ dr, int time) {
  pdl_trigger();
  extern __shared__ float red[];  // [warps][heads]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int per = dh / 8;                 // 16-byte chunks per head
  float* mine = red + warp * heads;
  for (int h = lane; h < heads; h += 32) mine[h] = 0.0f;
  __syncwarp();
  const int per_shift = 31 - __clz(per);    // per is a power of two: head and piece of a chunk by shift and mask
  const int chunks = heads * per;
  for (int64_t row = (int64_t)blockIdx.x * nwarps + warp; row < rows; row += (int64_t)gridDim.x * nwarps) {
    // once per row, not per head: the token's batch and time step (64-bit divisions cost this kernel its issue slots otherwise)
    const int64_t rb = dr ? row / time : 0, rt = row - rb * time;
    const float* srow = scales + row * heads;
    const int64_t base = row * heads * (int64_t)dh;
    for (int c = lane; c < ((chunks + 31) / 32) * 32; c += 32) {
      const bool ok = c < chunks;
      const int h = ok ? c >> per_shift : 0;
      float dot = 0.0f, g = 0.0f;
      if (ok) {
        g = srow[h];
        float a[8], go[8];
        const int64_t off = base + c * 8;
        load8(attn + off, a); load8(gout + off, go);
#pragma unroll
        for (int k = 0; k < 8; ++k) { dot += go[k] * a[k]; go[k] *= g; }
        store8(gattn + off, go);
      }
      // the `per` lanes of one head are contiguous (per divides 32 for head_dim 64 / 128 / 256)
      for (int o = per / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (ok && (c & (per - 1)) == 0) {
        const float zg = dot * g * (1.0f - g);
        gz[row * zld + h] = __float2bfloat16_rn(zg);
        mine[h] += zg;
        if (dr) dr[(rb * heads + h) * (int64_t)time + rt] = dot * g;
      }
    }
    for (int h = heads + lane; h < zld; h += 32) gz[row * zld + h] = __float2bfloat16_rn(0.0f);
    __syncwarp();
  }
  __syncthreads();
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    float acc = 0.0f;
    for (int wi = 0; wi < nwarps; ++wi) acc += red[wi * heads + h];
    part_out[(int64_t)blockIdx.x * heads + h] = acc;
  }
}

// ---- row-strided forms for column slices of a wider [rows, ld] buffer (the outputs of one GEMM over concatenated weights)
// SwiGLU: a = au[:, 0:F], u = au[:, F:2F]; same arithmetic (and bf16 rounding of silu(a)) as swiglu_forward / backward.
__global__ void swiglu_rows_forward_kernel(const bf16* __restrict__ au, int64_t ld, bf16* __restrict__ m, int64_t rows, int f8) {
  pdl_trigger();
  const int64_t total = rows * f8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / f8; const int c = (int)(i % f8) * 8;
    float a[8], u[8], r[8];
    load8(au + row * ld + c, a); load8(au + row * ld + (int64_t)f8 * 8 + c, u);
#pragma unroll
    for (int k = 0; k < 8; k += 2) swiglu::forward_pair(a[k], a[k + 1], u[k], u[k + 1], r[k], r[k + 1]);
    store8(m + row * (int64_t)f8 * 8 + c, r);
  }
}
__global__ void swiglu_rows_backward_kernel(const bf16* __restrict__ au, const bf16* __restrict__ gm, bf16* __restrict__ gau, int64_t ld, int64_t rows, int f8) {
  pdl_trigger();
  const int64_t total = rows * f8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / f8; const int c = (int)(i % f8) * 8;
    float a[8], u[8], g[8], ra[8], ru[8];
    load8(au + row * ld + c, a); load8(au + row * ld + (int64_t)f8 * 8 + c, u); load8(gm + row * (int64_t)f8 * 8 + c, g);
#pragma unroll
    for (int k = 0; k < 8; k += 2) swiglu::backward_pair(a[k], a[k + 1], u[k], u[k + 1], g[k], g[k + 1], ra[k], ra[k + 1], ru[k], ru[k + 1]);
    store8(gau + row * ld + c, ra); store8(gau + row * ld + (int64_t)f8 * 8 + c, ru);
  }
}

// Value-residual blend over strided rows: y = (1-s) v + s v0, s = sigmoid(lambda).
__global__ void vres_rows_forward_kernel(const bf16* __restrict__ v, int64_t ldv, const bf16* __restrict__ v0, int64_t ld0, const float* __restrict__ lambda,
                                         bf16* __restrict__ y, int64_t rows, int c8) {
  pdl_trigger();
  const float s = sigmoidf_(lambda[0]);
  const int64_t total = rows * c8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / c8; const int c = (int)(i % c8) * 8;
    float a[8], b[8], r[8];
    load8(v + row * ldv + c, a); load8(v0 + row * ld0 + c, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) r[k] = (1.0f - s) * a[k] + s * b[k];
    store8(y + row * (int64_t)c8 * 8 + c, r);
  }
}
// Backward of the blend, with the layer-0 accumulation folded in: gv = (1-s) g (strided), acc (+)= bf16(s g) in f32,
// part[block] = sum (v0 - v) g  (finished by vres_rows_lambda_kernel in block order).
__global__ void vres_rows_backward_kernel(const bf16* __restrict__ v, int64_t ldv, const bf16* __restrict__ v0, int64_t ld0, const float* __restrict__ lambda,
                                          const bf16* __restrict__ gy, bf16* __restrict__ gv, int64_t ldg, float* __restrict__ acc, int first,
                                          double* __restrict__ part, int64_t rows, int c8) {
  pdl_trigger();
  __shared__ float red[32];
  const float s = sigmoidf_(lambda[0]);
  const int64_t total = rows * c8;
  float sum = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / c8; const int c = (int)(i % c8) * 8;
    float a[8], b[8], g[8], r[8], o[8];
    load8(v + row * ldv + c, a); load8(v0 + row * ld0 + c, b); load8(gy + row * (int64_t)c8 * 8 + c, g);
    float* ap = acc + row * (int64_t)c8 * 8 + c;
    if (first) {
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = 0.0f;
    } else load8f(ap, o);
#pragma unroll
    for (int k = 0; k < 8; ++k) { r[k] = (1.0f - s) * g[k]; o[k] += rbf(s * g[k]); sum += (b[k] - a[k]) * g[k]; }
    store8(gv + row * ldg + c, r);
    *reinterpret_cast<float4*>(ap) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4*>(ap + 4) = make_float4(o[4], o[5], o[6], o[7]);
  }
  const float t = block_sum(sum, red);
  if (threadIdx.x == 0) part[blockIdx.x] = (double)t;
}
__global__ void vres_rows_lambda_kernel(const double* __restrict__ part, int nparts, const float* __restrict__ lambda, float* __restrict__ out) {
  double a = 0.0;
  for (int p = threadIdx.x; p < nparts; p += 32) a += part[p];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
  if (threadIdx.x == 0) { const float s = sigmoidf_(lambda[0]); out[0] = (float)(a * (double)s * (double)(1.0f - s)); }
}
// Layer 0's raw value gradient: out (strided) = bf16(acc + g), acc = the later layers' contributions (null: a plain strided copy).
__global__ void vres_root_backward_kernel(const float* __restrict__ acc, const bf16* __restrict__ g, bf16* __restrict__ out, int64_t ldo, int64_t rows, int c8) {
  pdl_trigger();
  const int64_t total = rows * c8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / c8; const int c = (int)(i % c8) * 8;
    float a[8], r[8];
    load8(g + row * (int64_t)c8 * 8 + c, r);
    if (acc) {
      load8f(acc + row * (int64_t)c8 * 8 + c, a);
#pragma unroll
      for (int k = 0; k < 8; ++k) r[k] += a[k];
    }
    store8(out + row * ldo + c, r);
  }
}

// ---- RMSNorm backward over the f32 residual stream, 128-bit accesses: a warp per row, lane l owns float4 columns
// 4 (l + 32 j). Same arithmetic as rms_backward_kernel (dot = sum (g w)(x rstd); dX = (g w - xhat dot/dim) rstd; per-block
// partial dW in shared memory, finished by the fixed-order column sum). Optional second f32 output accumulation and a
// bf16 copy of dX (the operand of the next matmul).
template <int J>
__global__ void rms_backward_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ gy, float* __restrict__ gx,
                                         bf16* __restrict__ gx_b, float* __restrict__ part, int64_t rows, float eps, int gx_accumulate) {
  pdl_trigger();
  constexpr int DIM = 128 * J;
  extern __shared__ float smem[];  // [warps][DIM]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float4 wv[J], dw[J];
#pragma unroll
  for (int j = 0; j < J; ++j) { wv[j] = *reinterpret_cast<const float4*>(w + 4 * (lane + 32 * j)); dw[j] = make_float4(0.f, 0.f, 0.f, 0.f); }
  const float inv_dim = 1.0f / (float)DIM;
  for (int64_t row = (int64_t)blockIdx.x * nwarps + warp; row < rows; row += (int64_t)gridDim.x * nwarps) {
    const float* xr = x + row * DIM; const float* gr = gy + row * DIM; float* or_ = gx + row * DIM;
    float4 xv[J], gv[J], old[J];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = 4 * (lane + 32 * j);
      xv[j] = *reinterpret_cast<const float4*>(xr + c);
      gv[j] = *reinterpret_cast<const float4*>(gr + c);
      old[j] = gx_accumulate ? *reinterpret_cast<const float4*>(or_ + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
    }
    ss = row_sum<32>(ss);
    const float rstd = 1.0f / sqrtf(ss * inv_dim + eps);
    float dot = 0.0f;
#pragma unroll
    for (int j = 0; j < J; ++j)
      dot += (gv[j].x * wv[j].x) * (xv[j].x * rstd) + (gv[j].y * wv[j].y) * (xv[j].y * rstd) + (gv[j].z * wv[j].z) * (xv[j].z * rstd) + (gv[j].w * wv[j].w) * (xv[j].w * rstd);
    dot = row_sum<32>(dot);
    const float mean = dot * inv_dim;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = 4 * (lane + 32 * j);
      const float4 xh = make_float4(xv[j].x * rstd, xv[j].y * rstd, xv[j].z * rstd, xv[j].w * rstd);
      dw[j].x += gv[j].x * xh.x; dw[j].y += gv[j].y * xh.y; dw[j].z += gv[j].z * xh.z; dw[j].w += gv[j].w * xh.w;
      const float4 o = make_float4((gv[j].x * wv[j].x - xh.x * mean) * rstd + old[j].x, (gv[j].y * wv[j].y - xh.y * mean) * rstd + old[j].y,
                                   (gv[j].z * wv[j].z - xh.z * mean) * rstd + old[j].z, (gv[j].w * wv[j].w - xh.w * mean) * rstd + old[j].w);
      *reinterpret_cast<float4*>(or_ + c) = o;
      if (gx_b) *reinterpret_cast<uint2*>(gx_b + row * DIM + c) = make_uint2(pack2(o.x, o.y), pack2(o.z, o.w));
    }
  }
#pragma unroll
  for (int j = 0; j < J; ++j) *reinterpret_cast<float4*>(smem + warp * DIM + 4 * (lane + 32 * j)) = dw[j];
  __syncthreads();
  for (int c = threadIdx.x; c < DIM; c += blockDim.x) {
    float acc = 0.0f;
    for (int wi = 0; wi < nwarps; ++wi) acc += smem[wi * DIM + c];
    part[(int64_t)blockIdx.x * DIM + c] = acc;
  }
}

// ---- RMSNorm forward over the f32 residual stream to a bf16 operand, 128-bit accesses (a warp per row, lane l owns float4
// columns 4 (l + 32 j)); optionally also copies the row into the stream's next buffer.
template <int J>
__global__ void rms_forward_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, bf16* __restrict__ y, float* __restrict__ copy, int64_t rows,
                                        float eps, uint32_t* fault) {
  pdl_trigger();
  constexpr int DIM = 128 * J;
  const int lane = threadIdx.x & 31;
  float4 wv[J];
#pragma unroll
  for (int j = 0; j < J; ++j) wv[j] = *reinterpret_cast<const float4*>(w + 4 * (lane + 32 * j));
  const int64_t rstride = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += rstride) {
    const float* xr = x + row * DIM;
    float4 xv[J];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      xv[j] = *reinterpret_cast<const float4*>(xr + 4 * (lane + 32 * j));
      ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
    }
    ss = row_sum<32>(ss);
    const float denom = ss / (float)DIM + eps;
    const float rstd = 1.0f / sqrtf(denom);
    if (!(isfinite(denom) && denom > 0.0f && isfinite(rstd))) { if (lane == 0) raise_fault(fault, OP_RMS_NORM); }
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = 4 * (lane + 32 * j);
      *reinterpret_cast<uint2*>(y + row * DIM + c) = make_uint2(pack2(xv[j].x * rstd * wv[j].x, xv[j].y * rstd * wv[j].y), pack2(xv[j].z * rstd * wv[j].z, xv[j].w * rstd * wv[j].w));
      if (copy) *reinterpret_cast<float4*>(copy + row * DIM + c) = xv[j];
    }
  }
}

template <class F> ojc_status dispatch_tpr(const char* op, int dh, F&& f) {
  switch (dh) {
    case 16: return f(std::integral_constant<int, 1>());
    case 32: return f(std::integral_constant<int, 2>());
    case 64: return f(std::integral_constant<int, 4>());
    case 128: return f(std::integral_constant<int, 8>());
    case 256: return f(std::integral_constant<int, 16>());
    default: return ojc_fail(OJC_ERR_UNSUPPORTED_HEAD_DIM, op, "the fused norm + rope kernel wants head_dim in {16, 32, 64, 128, 256}");
  }
}

}  // namespace

bool qk_norm_rope_supported(int dh) { return dh == 16 || dh == 32 || dh == 64 || dh == 128 || dh == 256; }

ojc_status qk_norm_rope_forward(ojc_backend* be, const bf16* x, int64_t xs, const float* w, const float* cos_t, const float* sin_t, bf16* y, int64_t ys,
                                int64_t tokens, int heads, int dh, int time, float eps) {
  const char* op = "qk_norm_rope_forward";
  const int64_t rows = tokens * heads;
  if (rows == 0) return OJC_OK;
  return dispatch_tpr(op, dh, [&](auto tpr) {
    constexpr int TPR = decltype(tpr)::value;
    // one thread per (token, head lane, 16-column part), walking every HL-th head
    if (TPR <= 8 && heads % 4 == 0) {
      const int64_t threads = tokens * TPR * 4;
      qk_norm_rope_forward_kernel<TPR, 4><<<(unsigned)((threads + 127) / 128), 128, 0, be->stream>>>(x, xs, w, cos_t, sin_t, y, ys, tokens, heads, time, eps);
    } else {
      const int64_t threads = tokens * TPR;
      qk_norm_rope_forward_kernel<TPR, 1><<<(unsigned)((threads + 127) / 128), 128, 0, be->stream>>>(x, xs, w, cos_t, sin_t, y, ys, tokens, heads, time, eps);
    }
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  });
}

ojc_status qk_norm_rope_backward(ojc_backend* be, const bf16* x, int64_t xs, const float* w, const float* cos_t, const float* sin_t, const bf16* gy, int64_t gys,
                                 bf16* gx, int64_t gxs, float* gw, int64_t tokens, int heads, int dh, int time, float eps) {
  const char* op = "qk_norm_rope_backward";
  const int64_t rows = tokens * heads;
  if (rows == 0) return OJC_OK;
  return dispatch_tpr(op, dh, [&](auto tpr) {
    constexpr int TPR = decltype(tpr)::value;
    const int hl = 1;   // the backward measured faster with each thread walking all heads of its token (42 vs 46 us at 12 x 64); the forward the other way (23 vs 29 us)
    const int tokens_per_block = 128 / (TPR * hl);
    int64_t blocks = (tokens + tokens_per_block - 1) / tokens_per_block;
    if (blocks > (int64_t)REDUCE_SMS * 8) blocks = (int64_t)REDUCE_SMS * 8;
    void* part = nullptr;
    bool on_lane = false;
    cudaStream_t fs = nullptr;
    OJC_TRY(ojc_partials(be, (uint64_t)blocks * dh * 4, &part, &on_lane));
    if (hl == 4) qk_norm_rope_backward_kernel<TPR, 4><<<(unsigned)blocks, 128, 128 * 16 * 4, be->stream>>>(x, xs, w, cos_t, sin_t, gy, gys, gx, gxs, (float*)part, tokens, heads, time, eps);
    else qk_norm_rope_backward_kernel<TPR, 1><<<(unsigned)blocks, 128, 128 * 16 * 4, be->stream>>>(x, xs, w, cos_t, sin_t, gy, gys, gx, gxs, (float*)part, tokens, heads, time, eps);
    OJC_LAUNCHED(be, op);
    OJC_TRY(ojc_finish_stream(be, on_lane, &fs));
    fused_column_sum_kernel<<<(dh + 31) / 32, 256, 0, fs>>>((const float*)part, gw, (int)blocks, dh);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  });
}

ojc_status gate_apply_forward(ojc_backend* be, const bf16* z, int zld, const float* bias, const bf16* attn, bf16* out, float* scales, int64_t rows, int heads, int dh) {
  const char* op = "per_head_sigmoid_gate_forward";
  if (dh % 8 != 0) return ojc_fail(OJC_ERR_UNSUPPORTED_HEAD_DIM, op, "head_dim must be a multiple of 8");
  const int chunks = heads * (dh / 8);
  const int tx = chunks >= 256 ? 256 : ((chunks + 31) / 32) * 32, ty = 256 / tx > 0 ? (256 / tx < 4 ? 256 / tx : 4) : 1;
  const int64_t passes = (rows + ty - 1) / ty;
  gate_apply_forward_kernel<<<elementwise_grid(be, passes * tx * ty, tx * ty), dim3(tx, ty), 0, be->stream>>>(z, zld, attn, bias, out, scales, rows, heads, dh);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status gate_apply_backward(ojc_backend* be, const float* scales, const bf16* attn, const bf16* gout, bf16* gattn, bf16* gz, int zld, float* gbias, int64_t rows,
                               int heads, int dh, float* dr, int time) {
  const char* op = "per_head_sigmoid_gate_backward";
  const int per = dh / 8;
  if (dh % 8 != 0 || per > 32 || (per & (per - 1)) != 0) return ojc_fail(OJC_ERR_UNSUPPORTED_HEAD_DIM, op, "head_dim must be 8, 16, 32, 64, 128 or 256");
  const int warps = 8;
  int64_t blocks = (rows + warps - 1) / warps;
  if (blocks > (int64_t)REDUCE_SMS * 8) blocks = (int64_t)REDUCE_SMS * 8;
  void* part = nullptr;
  bool on_lane = false;
  cudaStream_t fs = nullptr;
  OJC_TRY(ojc_partials(be, (uint64_t)blocks * heads * 4, &part, &on_lane));
  gate_apply_backward_kernel<<<(unsigned)blocks, warps * 32, warps * heads * 4, be->stream>>>(scales, attn, gout, gattn, gz, zld, (float*)part, rows, heads, dh, dr, time > 0 ? time : 1);
  OJC_LAUNCHED(be, op);
  OJC_TRY(ojc_finish_stream(be, on_lane, &fs));
  fused_column_sum_kernel<<<(heads + 31) / 32, 256, 0, fs>>>((const float*)part, gbias, (int)blocks, heads);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status swiglu_rows_forward(ojc_backend* be, const bf16* au, int64_t ld, bf16* m, int64_t rows, int64_t f) {
  const char* op = "swiglu_forward";
  if (f % 8 != 0 || ld % 8 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "widths must be multiples of 8");
  swiglu_rows_forward_kernel<<<elementwise_grid(be, rows * (f / 8), 256), 256, 0, be->stream>>>(au, ld, m, rows, (int)(f / 8));
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}
ojc_status swiglu_rows_backward(ojc_backend* be, const bf16* au, const bf16* gm, bf16* gau, int64_t ld, int64_t rows, int64_t f) {
  const char* op = "swiglu_backward";
  if (f % 8 != 0 || ld % 8 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "widths must be multiples of 8");
  swiglu_rows_backward_kernel<<<elementwise_grid(be, rows * (f / 8), 256), 256, 0, be->stream>>>(au, gm, gau, ld, rows, (int)(f / 8));
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}
ojc_status vres_rows_forward(ojc_backend* be, const bf16* v, int64_t ldv, const bf16* v0, int64_t ld0, const float* lambda, bf16* y, int64_t rows, int64_t cols) {
  const char* op = "value_residual_blend_forward";
  if (cols % 8 != 0 || ldv % 8 != 0 || ld0 % 8 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "widths must be multiples of 8");
  vres_rows_forward_kernel<<<elementwise_grid(be, rows * (cols / 8), 256), 256, 0, be->stream>>>(v, ldv, v0, ld0, lambda, y, rows, (int)(cols / 8));
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}
ojc_status vres_rows_backward(ojc_backend* be, const bf16* v, int64_t ldv, const bf16* v0, int64_t ld0, const float* lambda, const bf16* gy, bf16* gv, int64_t ldg,
                              float* acc, bool first, float* glambda, int64_t rows, int64_t cols) {
  const char* op = "value_residual_blend_backward";
  if (cols % 8 != 0 || ldv % 8 != 0 || ld0 % 8 != 0 || ldg % 8 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "widths must be multiples of 8");
  const int blocks = REDUCE_SMS * 4;
  void* part = nullptr;
  OJC_TRY(ojc_scratch(be, (uint64_t)blocks * 8, &part));
  vres_rows_backward_kernel<<<blocks, 256, 0, be->stream>>>(v, ldv, v0, ld0, lambda, gy, gv, ldg, acc, first ? 1 : 0, (double*)part, rows, (int)(cols / 8));
  OJC_LAUNCHED(be, op);
  vres_rows_lambda_kernel<<<1, 32, 0, be->stream>>>((const double*)part, blocks, lambda, glambda);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}
ojc_status vres_root_backward(ojc_backend* be, const float* acc, const bf16* g, bf16* out, int64_t ldo, int64_t rows, int64_t cols) {
  const char* op = "value_residual_blend_backward";
  if (cols % 8 != 0 || ldo % 8 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "widths must be multiples of 8");
  vres_root_backward_kernel<<<elementwise_grid(be, rows * (cols / 8), 256), 256, 0, be->stream>>>(acc, g, out, ldo, rows, (int)(cols / 8));
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}


bool rms_backward_rows_supported(int64_t dim) { return dim == 512 || dim == 768 || dim == 1024 || dim == 2048; }
// part: [blocks, dim] scratch from the caller; returns the block count through *blocks_out for the column sum.
ojc_status rms_backward_rows(ojc_backend* be, const float* x, const float* w, const float* gy, float* gx, bf16* gx_b, float* part, int64_t rows, int64_t dim,
                             float eps, bool accumulate_gx, int blocks) {
  const char* op = "rms_norm_backward";
  const int warps = 4;
  const size_t smem = (size_t)warps * dim * 4;
#define OJC_RMS_ROWS(J) rms_backward_rows_kernel<J><<<blocks, warps * 32, smem, be->stream>>>(x, w, gy, gx, gx_b, part, rows, eps, accumulate_gx ? 1 : 0)
  if (dim == 512) OJC_RMS_ROWS(4);
  else if (dim == 768) OJC_RMS_ROWS(6);
  else if (dim == 1024) OJC_RMS_ROWS(8);
  else if (dim == 2048) OJC_RMS_ROWS(16);
  else return ojc_fail(OJC_ERR_UNSUPPORTED, op, "row width outside the vectorized forms");
#undef OJC_RMS_ROWS
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status rms_forward_rows(ojc_backend* be, const float* x, const float* w, bf16* y, float* copy, int64_t rows, int64_t dim, float eps) {
  const char* op = "rms_norm_forward";
  const int grid = elementwise_grid(be, rows * 32, 256);
#define OJC_RMS_FWD(J) rms_forward_rows_kernel<J><<<grid, 256, 0, be->stream>>>(x, w, y, copy, rows, eps, be->fault_dev)
  if (dim == 512) OJC_RMS_FWD(4);
  else if (dim == 768) OJC_RMS_FWD(6);
  else if (dim == 1024) OJC_RMS_FWD(8);
  else if (dim == 2048) OJC_RMS_FWD(16);
  else return ojc_fail(OJC_ERR_UNSUPPORTED, op, "row width outside the vectorized forms");
#undef OJC_RMS_FWD
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}
