// Optimizer-side ops: global gradient norm + clip, fused AdamW, Muon with five
// Newton-Schulz iterations. Reductions are two-stage with f64 finishes in a
// fixed order; the norm pass doubles as the non-finite scan, as the reference's
// does (ojas-cpu/src/optim.rs:86-95).
#include "common.cuh"
#include "dispatch.cuh"
#include "gemm.cuh"
#include "optim.cuh"

namespace {

constexpr int NORM_CHUNK = 8192;  // elements per block of the sum-of-squares pass

__device__ __forceinline__ double block_sum_f64(double v, double* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    v = threadIdx.x < (blockDim.x + 31) / 32 ? red[threadIdx.x] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  }
  return v;
}


__global__ void sumsq_partial_kernel(const float* __restrict__ x, int64_t n, double* __restrict__ part, uint32_t* fault, uint32_t op_id) {
  // squares and their sum in f64, as the reference's norm (ojas-cpu/src/optim.rs:96-126): an f32-summed norm is off in its last
  // bit often enough to change the clip coefficient, and with it the last bit of every clipped gradient
  __shared__ double red[32];
  const int64_t base = (int64_t)blockIdx.x * NORM_CHUNK;
  double acc = 0.0;
  for (int i = threadIdx.x; i < NORM_CHUNK; i += blockDim.x) {
    int64_t idx = base + i;
    if (idx < n) { const double v = (double)x[idx]; acc += v * v; }
  }
  const double t = block_sum_f64(acc, red);
  if (threadIdx.x == 0) {
    if (!isfinite(t)) raise_fault(fault, op_id);
    part[blockIdx.x] = t;
  }
}

// out[0] = norm (f32 of the f64 square root), out[1] = clip scale = min(1, max / (norm + 1e-6)) (ojas-core/src/backend.rs:277-303).
__global__ void norm_finish_kernel(const double* __restrict__ part, int64_t nparts, float max_norm, float* __restrict__ out) {
  __shared__ double red[256];
  double acc = 0.0;
  for (int64_t p = threadIdx.x; p < nparts; p += blockDim.x) acc += part[p];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) { if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
  if (threadIdx.x == 0) {
    float norm = (float)sqrt(red[0]);
    out[0] = norm;
    float coef = max_norm / (norm + 1e-6f);
    out[1] = max_norm >= 0.0f ? fminf(coef, 1.0f) : 1.0f;  // a negative max_norm asks for the norm only
  }
}

__global__ void scale_by_device_kernel(float* __restrict__ x, int64_t n, const float* __restrict__ scale) {
  const float s = scale[0];
  if (!(s < 1.0f)) return;  // multiply only when clipping (ojas-cpu/src/backend.rs:788-791)
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) x[i] *= s;
}

// The 7 f32 words of AdamWScalars::f32_words (ojas-core/src/backend.rs:462-476).
struct AdamWords { float decay, one_minus_b1, beta2, one_minus_b2, step_size, bc2_sqrt, eps; int decays, lerp_low; float lerp_high; };

// One element of torch's single-tensor AdamW in f32 (ojas-cpu/src/optim.rs:341-366): decay first, lerp form switch
// at weight 0.5, eps outside the square root. grad_scale (optional, device) folds the clip coefficient in.
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, bf16* __restrict__ mirror,
                             int64_t n, AdamWords w, const float* __restrict__ grad_scale, uint32_t* fault) {
  float gs = 1.0f;
  if (grad_scale) { gs = grad_scale[0]; if (gs < 0.0f) return; if (!(gs < 1.0f)) gs = 1.0f; }   // a negative scale calls the step off (STEP_CALLED_OFF)
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) {
    const float pi = p[i];
    float gi = g[i];
    if (gs != 1.0f) gi *= gs;
    const float mi = m[i], vi = v[i];
    const float m1 = w.lerp_low ? mi + w.one_minus_b1 * (gi - mi) : gi - (gi - mi) * w.lerp_high;
    const float v1 = w.beta2 * vi + w.one_minus_b2 * gi * gi;
    const float denom = sqrtf(v1) / w.bc2_sqrt + w.eps;
    const float delta = (-w.step_size) * m1 / denom;
    float q = pi;
    if (w.decays) q *= w.decay;
    q += delta;
    const float np = (!w.decays && delta == 0.0f) ? pi : q;
    if (!(isfinite(m1) && isfinite(v1) && isfinite(denom) && isfinite(delta) && isfinite(np))) { raise_fault(fault, OP_ADAMW); continue; }
    p[i] = np; m[i] = m1; v[i] = v1;
    if (mirror) mirror[i] = __float2bfloat16_rn(np);
  }
}

// Muon works on groups of same-shape matrices: blockIdx.y picks the matrix, the pointer table travels by value.
constexpr int MUON_MAX_BATCH = 48;
struct MuonBatch { const float* g[MUON_MAX_BATCH]; float* mom[MUON_MAX_BATCH]; float* p[MUON_MAX_BATCH]; bf16* mirror[MUON_MAX_BATCH]; };

// buf = mu * mom + g; u = nesterov ? fma(mu, buf, g) : buf; mom = buf (ojas-cpu/src/optim.rs:684-712).
// Also the block partial of sum u^2 (of the bf16-rounded u when ns5 runs in bf16). u: [batch][n], part: [batch][gridDim.x].
__global__ void muon_momentum_kernel(const MuonBatch mb, float* __restrict__ u_all, int64_t n, float mu, int nesterov, int round_u,
                                     const float* __restrict__ grad_scale, double* __restrict__ part, uint32_t* fault) {
  __shared__ double red[32];
  const float* __restrict__ g = mb.g[blockIdx.y];
  float* __restrict__ mom = mb.mom[blockIdx.y];
  float* __restrict__ u = u_all + (int64_t)blockIdx.y * n;
  float gs = 1.0f;
  bool off = false;     // a called-off step still forms u (the later kernels read it) but leaves the momentum buffer alone
  if (grad_scale) { gs = grad_scale[0]; off = gs < 0.0f; if (!(gs < 1.0f) || off) gs = 1.0f; }
  const int64_t base = (int64_t)blockIdx.x * NORM_CHUNK;
  // The Frobenius norm is summed in f64, as the reference does (optim.rs:893-900): the norm is rounded to bf16 under
  // Ns5Precision::Bf16, where an f32-summed value that lands on the other side of a rounding boundary would rescale the whole matrix.
  double acc = 0.0;
  for (int i = threadIdx.x; i < NORM_CHUNK; i += blockDim.x) {
    int64_t idx = base + i;
    if (idx >= n) break;
    float gi = g[idx];
    if (gs != 1.0f) gi *= gs;
    const float buf = __fadd_rn(__fmul_rn(mu, mom[idx]), gi);      // a multiply and an add, each rounded (optim.rs:684-700); only Nesterov's step is fused
    float ui = nesterov ? fmaf(mu, buf, gi) : buf;
    if (round_u) ui = round_bf16(ui);
    if (!off) mom[idx] = buf;
    u[idx] = ui;
    acc += (double)ui * (double)ui;
  }
  const double t = block_sum_f64(acc, red);
  if (threadIdx.x == 0) { if (!isfinite(t) && !off) raise_fault(fault, OP_MUON); part[(int64_t)blockIdx.y * gridDim.x + blockIdx.x] = t; }
}

// norm[matrix] = f32 of the f64 square root of its partial sums, added in the order norm_finish_kernel uses
__global__ void muon_norm_kernel(const double* __restrict__ part, int64_t nparts, float* __restrict__ norm) {
  __shared__ double red[256];
  const double* p = part + (int64_t)blockIdx.x * nparts;
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < nparts; i += blockDim.x) acc += p[i];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) { if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
  if (threadIdx.x == 0) norm[blockIdx.x] = (float)sqrt(red[0]);
}

// X = u / (norm + 1e-7), written in the wide orientation (transposed when rows > cols), as TX (f32 or bf16).
// In bf16 mode the norm, norm + eps and the quotient are each rounded (ojas-cpu/src/optim.rs:893-910).
template <class TX>
__global__ void muon_normalize_kernel(const float* __restrict__ u_all, const float* __restrict__ norm, TX* __restrict__ x_all, int rows, int cols, int tall, int bf16_mode) {
  pdl_trigger();
  const int64_t n = (int64_t)rows * cols;
  const float* __restrict__ u = u_all + (int64_t)blockIdx.y * n;
  TX* __restrict__ x = x_all + (int64_t)blockIdx.y * n;
  const float nrm = norm[blockIdx.y];
  const float denom = bf16_mode ? round_bf16(round_bf16(nrm) + 1e-7f) : nrm + 1e-7f;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) {
    int64_t r = i / cols, c = i % cols;
    float v = u[i] / denom;
    int64_t o = tall ? c * rows + r : i;
    stf(x, o, v);  // the bf16 store rounds to nearest even
  }
}

// Tall matrices (rows > cols) run Newton-Schulz on the transpose: X^T[c, r] = u[r, c] / denom, and the update reads X^T back.
// Both directions go through a 32 x 32 shared-memory tile so that reads and writes are row-contiguous on both sides.
// grid (cols / 32, rows / 32, matrices), block (32, 8).
template <class TX>
__global__ void muon_normalize_tall_kernel(const float* __restrict__ u_all, const float* __restrict__ norm, TX* __restrict__ x_all, int rows, int cols, int bf16_mode) {
  pdl_trigger();
  __shared__ float tile[32][33];
  const int64_t n = (int64_t)rows * cols;
  const float* __restrict__ u = u_all + (int64_t)blockIdx.z * n;
  TX* __restrict__ x = x_all + (int64_t)blockIdx.z * n;
  const float nrm = norm[blockIdx.z];
  const float denom = bf16_mode ? round_bf16(round_bf16(nrm) + 1e-7f) : nrm + 1e-7f;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = u[(int64_t)r * cols + c] / denom;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) stf(x, (int64_t)c * rows + r, tile[threadIdx.x][j]);
  }
}
template <class TX>
__global__ void muon_apply_tall_kernel(const MuonBatch mb, const TX* __restrict__ x_all, int rows, int cols, float alpha, float decay, int decays, uint32_t* fault,
                                       const float* __restrict__ gate) {
  __shared__ float tile[32][33];
  if (gate && gate[0] < 0.0f) return;
  const int64_t n = (int64_t)rows * cols;
  float* __restrict__ p = mb.p[blockIdx.z];
  bf16* __restrict__ mirror = mb.mirror[blockIdx.z];
  const TX* __restrict__ x = x_all + (int64_t)blockIdx.z * n;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = ldf(x, (int64_t)c * rows + r);
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r >= rows || c >= cols) continue;
    const int64_t i = (int64_t)r * cols + c;
    const float base = decays ? p[i] * decay : p[i];
    const float np = fmaf(alpha, tile[threadIdx.x][j], base);
    if (!isfinite(np)) { raise_fault(fault, OP_MUON); continue; }
    p[i] = np;
    if (mirror) mirror[i] = __float2bfloat16_rn(np);
  }
}

// Wide matrices in bf16 mode, four elements per thread (n % 4 == 0): the same arithmetic as the scalar kernels.
__global__ void muon_normalize_bf16x4_kernel(const float* __restrict__ u_all, const float* __restrict__ norm, bf16* __restrict__ x_all, int64_t n) {
  pdl_trigger();
  const float4* __restrict__ u = reinterpret_cast<const float4*>(u_all + (int64_t)blockIdx.y * n);
  uint2* __restrict__ x = reinterpret_cast<uint2*>(x_all + (int64_t)blockIdx.y * n);
  const float nrm = norm[blockIdx.y];
  const float denom = round_bf16(round_bf16(nrm) + 1e-7f);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n / 4; i += stride) {
    const float4 v = u[i];
    x[i] = make_uint2((uint32_t)f32_to_bf16_bits(v.x / denom) | ((uint32_t)f32_to_bf16_bits(v.y / denom) << 16),
                      (uint32_t)f32_to_bf16_bits(v.z / denom) | ((uint32_t)f32_to_bf16_bits(v.w / denom) << 16));
  }
}
__global__ void muon_apply_bf16x4_kernel(const MuonBatch mb, const bf16* __restrict__ x_all, int64_t n, float alpha, float decay, int decays, uint32_t* fault,
                                         const float* __restrict__ gate) {
  if (gate && gate[0] < 0.0f) return;
  float4* __restrict__ p = reinterpret_cast<float4*>(mb.p[blockIdx.y]);
  uint2* __restrict__ mirror = reinterpret_cast<uint2*>(mb.mirror[blockIdx.y]);
  const uint2* __restrict__ x = reinterpret_cast<const uint2*>(x_all + (int64_t)blockIdx.y * n);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n / 4; i += stride) {
    const uint2 xv = x[i];
    const float o[4] = {__uint_as_float(xv.x << 16), __uint_as_float(xv.x & 0xffff0000u), __uint_as_float(xv.y << 16), __uint_as_float(xv.y & 0xffff0000u)};
    float4 pv = p[i];
    float np[4] = {pv.x, pv.y, pv.z, pv.w};
    bool bad = false;
#pragma unroll
    for (int k = 0; k < 4; ++k) { np[k] = fmaf(alpha, o[k], decays ? np[k] * decay : np[k]); bad |= !isfinite(np[k]); }
    if (bad) { raise_fault(fault, OP_MUON); continue; }   // as the scalar kernel: a non-finite update is not stored
    p[i] = make_float4(np[0], np[1], np[2], np[3]);
    if (mirror) mirror[i] = make_uint2((uint32_t)f32_to_bf16_bits(np[0]) | ((uint32_t)f32_to_bf16_bits(np[1]) << 16),
                                       (uint32_t)f32_to_bf16_bits(np[2]) | ((uint32_t)f32_to_bf16_bits(np[3]) << 16));
  }
}

// eight bf16 values per 16-byte access for the bf16 forms below (same arithmetic and roundings as the scalar kernels)
__device__ __forceinline__ void unpack8(const uint4& t, float (&v)[8]) {
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) w[i] = (uint32_t)f32_to_bf16_bits(v[2 * i]) | ((uint32_t)f32_to_bf16_bits(v[2 * i + 1]) << 16);
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__global__ void ns_combine_a_bf16x8_kernel(const uint4* __restrict__ a, uint4* __restrict__ a2, int64_t n8, float bcoef, float ccoef) {
  pdl_trigger();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n8; i += stride) {
    float av[8], a2v[8], r[8];
    unpack8(a[i], av); unpack8(a2[i], a2v);
#pragma unroll
    for (int k = 0; k < 8; ++k) r[k] = round_bf16(round_bf16(bcoef * av[k]) + round_bf16(ccoef * a2v[k]));
    a2[i] = pack8(r);
  }
}
__global__ void ns_combine_x_bf16x8_kernel(const uint4* __restrict__ x, uint4* __restrict__ bx, int64_t n8, float acoef, uint32_t* fault) {
  pdl_trigger();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool bad = false;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n8; i += stride) {
    float xv[8], bv[8], r[8];
    unpack8(x[i], xv); unpack8(bx[i], bv);
#pragma unroll
    for (int k = 0; k < 8; ++k) { r[k] = round_bf16(round_bf16(acoef * xv[k]) + bv[k]); bad |= !isfinite(r[k]); }
    bx[i] = pack8(r);
  }
  if (bad) raise_fault(fault, OP_MUON);
}

// out = b * A + c * A2 (A2 overwritten), every scalar multiple and the sum rounded in bf16 mode (optim.rs:947-957).
template <class T>
__global__ void ns_combine_a_kernel(const T* __restrict__ a, T* __restrict__ a2, int64_t n, float bcoef, float ccoef, int bf16_mode) {
  pdl_trigger();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) {
    float av = ldf(a, i), a2v = ldf(a2, i);
    float r = bf16_mode ? round_bf16(round_bf16(bcoef * av) + round_bf16(ccoef * a2v)) : bcoef * av + ccoef * a2v;
    stf(a2, i, r);
  }
}

// bx = a * x + bx (optim.rs:966-974)
template <class T>
__global__ void ns_combine_x_kernel(const T* __restrict__ x, T* __restrict__ bx, int64_t n, float acoef, int bf16_mode, uint32_t* fault) {
  pdl_trigger();
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) {
    float xv = ldf(x, i), bv = ldf(bx, i);
    float r = bf16_mode ? round_bf16(round_bf16(acoef * xv) + bv) : acoef * xv + bv;
    if (!isfinite(r)) raise_fault(fault, OP_MUON);
    stf(bx, i, r);
  }
}

// p = fma(alpha, X, p * decay) with X read back through the transpose when the matrix was tall (optim.rs:718-736).
template <class TX>
__global__ void muon_apply_kernel(const MuonBatch mb, const TX* __restrict__ x_all, int rows, int cols, int tall, float alpha, float decay, int decays, uint32_t* fault,
                                  const float* __restrict__ gate) {
  if (gate && gate[0] < 0.0f) return;
  const int64_t n = (int64_t)rows * cols;
  float* __restrict__ p = mb.p[blockIdx.y];
  bf16* __restrict__ mirror = mb.mirror[blockIdx.y];
  const TX* __restrict__ x = x_all + (int64_t)blockIdx.y * n;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (const int64_t stride = (int64_t)gridDim.x * blockDim.x; i < n; i += stride) {
    int64_t r = i / cols, c = i % cols;
    float o = ldf(x, tall ? c * rows + r : i);
    float base = decays ? p[i] * decay : p[i];
    float np = fmaf(alpha, o, base);
    if (!isfinite(np)) { raise_fault(fault, OP_MUON); continue; }
    p[i] = np;
    if (mirror) mirror[i] = __float2bfloat16_rn(np);
  }
}

// The five Newton-Schulz iterations of one small matrix (r <= 32 rows after the wide orientation) inside one CTA: X lives
// in shared memory as f32 (holding bf16-rounded values in bf16 mode), A = X X^T, A2 = A A, B = b A + c A2, X <- a X + B X,
// with the same rounding points as the per-product path (every product and every combine rounds to bf16 in bf16 mode).
// blockIdx.x = matrix. Dot products are warp-strided over k and added by shuffles.
template <class TX>
__global__ void muon_small_ns5_kernel(TX* __restrict__ x_all, int r, int c, float acoef, float bcoef, float ccoef, int bf16_mode, uint32_t* fault) {
  extern __shared__ float sm[];
  float* X = sm;                       // [r][c]
  float* BX = X + (size_t)r * c;       // [r][c]
  float* A = BX + (size_t)r * c;       // [32][33]
  float* B = A + 32 * 33;              // [32][33]
  TX* x = x_all + (int64_t)blockIdx.x * r * c;
  const int tid = threadIdx.x;
  const int n = r * c;
  auto rnd = [&](float v) { return bf16_mode ? round_bf16(v) : v; };
  for (int i = tid; i < n; i += blockDim.x) X[i] = ldf(x, i);
  __syncthreads();
  for (int it = 0; it < 5; ++it) {
    // every product element is one chain over k ascending, a separately rounded multiply and add per step: the reference's
    // Exact product (ojas-cpu/src/gemm.rs:11-16), so a small matrix steps to the same bits in f32 mode as well as in bf16 mode
    for (int pair = tid; pair < r * r; pair += blockDim.x) {       // A = X X^T
      const int i = pair / r, j = pair % r;
      float acc = 0.0f;
      for (int k = 0; k < c; ++k) acc = __fadd_rn(acc, __fmul_rn(X[i * c + k], X[j * c + k]));
      A[i * 33 + j] = rnd(acc);
    }
    __syncthreads();
    for (int e = tid; e < r * r; e += blockDim.x) {                // B = b A + c (A A)
      const int i = e / r, j = e % r;
      float acc = 0.0f;
      for (int k = 0; k < r; ++k) acc = __fadd_rn(acc, __fmul_rn(A[i * 33 + k], A[k * 33 + j]));
      const float a2 = rnd(acc), av = A[i * 33 + j];
      B[i * 33 + j] = bf16_mode ? round_bf16(round_bf16(bcoef * av) + round_bf16(ccoef * a2)) : __fadd_rn(__fmul_rn(bcoef, av), __fmul_rn(ccoef, a2));
    }
    __syncthreads();
    for (int e = tid; e < n; e += blockDim.x) {                    // X <- a X + B X
      const int i = e / c, k = e % c;
      float acc = 0.0f;
      for (int j = 0; j < r; ++j) acc = __fadd_rn(acc, __fmul_rn(B[i * 33 + j], X[j * c + k]));
      const float bx = rnd(acc), xv = X[e];
      const float out = bf16_mode ? round_bf16(round_bf16(acoef * xv) + bx) : __fadd_rn(__fmul_rn(acoef, xv), bx);
      if (!isfinite(out)) raise_fault(fault, OP_MUON);
      BX[e] = out;
    }
    __syncthreads();
    float* t = X; X = BX; BX = t;
  }
  for (int i = tid; i < n; i += blockDim.x) stf(x, i, X[i]);
}

double pow_u64(double base, uint64_t e) {  // ojas-core/src/backend.rs:244-257
  double result = 1.0, b = base;
  while (e > 0) { if (e & 1) result *= b; e >>= 1; if (e > 0) b *= b; }
  return result;
}

}  // namespace

int64_t norm_partials(int64_t n) { return (n + NORM_CHUNK - 1) / NORM_CHUNK; }

ojc_status grad_norm_device(ojc_backend* be, const float* const* ptrs, const int64_t* lens, int64_t count, float max_norm, float* norm_and_scale_dev) {
  const char* op = "clip_grad_norm";
  int64_t total_parts = 0;
  for (int64_t i = 0; i < count; ++i) total_parts += norm_partials(lens[i]);
  void* ws = nullptr;
  OJC_TRY(ojc_scratch(be, (uint64_t)total_parts * 8 + 8, &ws));
  double* part = (double*)ws;
  int64_t off = 0;
  for (int64_t i = 0; i < count; ++i) {
    int64_t parts = norm_partials(lens[i]);
    if (parts == 0) continue;
    sumsq_partial_kernel<<<(unsigned)parts, 256, 0, be->stream>>>(ptrs[i], lens[i], part + off, be->fault_dev, OP_CLIP);
    OJC_LAUNCHED(be, op);
    off += parts;
  }
  norm_finish_kernel<<<1, 256, 0, be->stream>>>(part, total_parts, max_norm, norm_and_scale_dev);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status scale_by_device(ojc_backend* be, float* x, int64_t n, const float* scale_dev) {
  if (n == 0) return OJC_OK;
  scale_by_device_kernel<<<elementwise_grid(be, n, 256), 256, 0, be->stream>>>(x, n, scale_dev);
  OJC_LAUNCHED(be, "clip_grad_norm");
  return OJC_OK;
}

ojc_status adamw_device(ojc_backend* be, float* p, const float* g, float* m, float* v, bf16* mirror, int64_t n, uint64_t step_before,
                        const ojc_adamw_config& cfg, const float* grad_scale_dev) {
  const char* op = "adamw_step";
  // check_adamw, ojas-core/src/backend.rs:312-356
  const double sc[5] = {cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay};
  for (double s : sc) if (!std::isfinite(s)) return ojc_fail(OJC_ERR_NON_FINITE, op, "a configuration scalar is not finite");
  if (!(cfg.beta1 >= 0.0 && cfg.beta1 < 1.0 && cfg.beta2 >= 0.0 && cfg.beta2 < 1.0)) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "adamw beta must be in [0, 1)");
  if (cfg.eps <= 0.0) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "adamw eps must be > 0");
  if (cfg.lr < 0.0 || cfg.weight_decay < 0.0) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "lr or weight_decay is negative");
  if (step_before == UINT64_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "step counter overflows");
  const uint64_t step = step_before + 1;
  const double bc1 = 1.0 - pow_u64(cfg.beta1, step), bc2 = 1.0 - pow_u64(cfg.beta2, step);
  if (!(std::isfinite(bc1) && std::isfinite(bc2) && bc1 > 0.0 && bc2 > 0.0)) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "adamw bias correction is not a positive finite value");
  AdamWords w;
  const double one_minus_b1 = 1.0 - cfg.beta1;
  w.decay = (float)(1.0 - cfg.lr * cfg.weight_decay);
  w.one_minus_b1 = (float)one_minus_b1;
  w.beta2 = (float)cfg.beta2;
  w.one_minus_b2 = (float)(1.0 - cfg.beta2);
  w.step_size = (float)(cfg.lr / bc1);
  w.bc2_sqrt = (float)std::sqrt(bc2);
  w.eps = (float)cfg.eps;
  w.decays = cfg.weight_decay != 0.0;
  w.lerp_low = w.one_minus_b1 < 0.5f;
  w.lerp_high = 1.0f - w.one_minus_b1;
  const float words[7] = {w.decay, w.one_minus_b1, w.beta2, w.one_minus_b2, w.step_size, w.bc2_sqrt, w.eps};
  for (float x : words) if (!std::isfinite(x)) return ojc_fail(OJC_ERR_NON_FINITE, op, "a scalar word is not finite in f32");
  if (n == 0) return OJC_OK;
  adamw_kernel<<<elementwise_grid(be, n, 256), 256, 0, be->stream>>>(p, g, m, v, mirror, n, w, grad_scale_dev, be->fault_dev);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

static uint64_t muon_group_scratch_bytes(int64_t rows, int64_t cols, bool bf16_mode, int64_t batch) {
  const int64_t r = rows < cols ? rows : cols, n = rows * cols;
  const uint64_t es = bf16_mode ? 2 : 4;
  auto al = [](uint64_t b) { return (b + 255) & ~uint64_t(255); };
  return al(batch * n * 4) /*u*/ + 2 * al(batch * n * es) /*x, bx*/ + 2 * al((uint64_t)batch * r * r * es) /*A, A2*/ + al(batch * norm_partials(n) * 8) + al(batch * 4);
}
uint64_t muon_scratch_bytes(int64_t rows, int64_t cols, bool bf16_mode) { return muon_group_scratch_bytes(rows, cols, bf16_mode, 1); }

// One Muon NS5 step for `batch` matrices of one shape (ojas-cpu/src/optim.rs:684-985 per matrix). The element-wise phases
// run as one launch over the group; the three products of each Newton-Schulz iteration run as batched tensor-core GEMMs
// when the operands are bf16 and eligible, as one GEMM per matrix otherwise.
ojc_status muon_group_device(ojc_backend* be, float* const* p, const float* const* g, float* const* mom, bf16* const* mirror, int64_t batch, int64_t rows,
                             int64_t cols, const ojc_muon_config& cfg, const float* grad_scale_dev) {
  const char* op = "muon_ns5_step";
  if (!std::isfinite(cfg.lr) || !std::isfinite(cfg.momentum) || !std::isfinite(cfg.weight_decay)) return ojc_fail(OJC_ERR_NON_FINITE, op, "a configuration scalar is not finite");
  if (cfg.lr < 0.0 || cfg.momentum < 0.0 || cfg.weight_decay < 0.0) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "lr, momentum or weight_decay is negative");
  if (rows <= 0 || cols <= 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  if (batch < 1 || batch > MUON_MAX_BATCH) return ojc_fail(OJC_ERR_SHAPE, op, "group size out of range");
  const bool bf = cfg.ns5_bf16 != 0, tall = rows > cols;
  const int64_t r = tall ? cols : rows, c = tall ? rows : cols, n = rows * cols;
  const int32_t dt = bf ? OJC_BF16 : OJC_F32;
  const uint64_t es = bf ? 2 : 4;
  auto al = [](uint64_t b) { return (b + 255) & ~uint64_t(255); };
  MuonBatch mb{};
  for (int64_t i = 0; i < batch; ++i) { mb.g[i] = g[i]; mb.mom[i] = mom[i]; mb.p[i] = p[i]; mb.mirror[i] = mirror ? mirror[i] : nullptr; }
  void* ws = nullptr;
  OJC_TRY(ojc_alloc(be, muon_group_scratch_bytes(rows, cols, bf, batch), &ws));
  char* cur = (char*)ws;
  float* u = (float*)cur; cur += al(batch * n * 4);
  void* x = cur; cur += al(batch * n * es);
  void* bx = cur; cur += al(batch * n * es);
  void* am = cur; cur += al((uint64_t)batch * r * r * es);
  void* a2 = cur; cur += al((uint64_t)batch * r * r * es);
  double* part = (double*)cur; cur += al(batch * norm_partials(n) * 8);
  float* norm = (float*)cur;
  ojc_status st = OJC_OK;
  // C_i = A_i . B_i for every matrix of the group
  // `comb`: the combine that follows this product; *fused says whether the product's epilogue did it (tensor-core path only)
  auto product = [&](const GemmOperand& ga, const GemmOperand& gb, void* cptr, int64_t m_, int64_t n_, int64_t k_, int64_t a_bs, int64_t b_bs, int64_t c_bs,
                     const NsCombine* comb = nullptr, bool* fused = nullptr) -> ojc_status {
    if (fused) *fused = false;
    // One matrix takes the same kernel, tiling and unsplit reduction as a group of them: a matrix's update must not depend on how
    // many others of its shape are stepped with it (the groups shrink when the Muon phase is split across data-parallel ranks).
    if (bf && n_ >= 64 && a_bs % 8 == 0 && b_bs % 8 == 0 && c_bs % 8 == 0 && gemm_tc_eligible(ga, gb, cptr, dt, n_, m_, n_, k_)) {
      const bool can = comb && comb->src_ld % 8 == 0 && comb->src_bs % 8 == 0 && ((uintptr_t)comb->src & 15) == 0;
      if (fused) *fused = can;
      return gemm_tc_batched(be, op, ga, gb, cptr, dt, n_, m_, n_, k_, batch, a_bs, b_bs, c_bs, 1.0f, false, nullptr, can ? comb : nullptr, false);
    }
    for (int64_t i = 0; i < batch; ++i) {
      GemmOperand ai{(const char*)ga.ptr + i * a_bs * es, ga.dtype, ga.rs, ga.cs}, bi{(const char*)gb.ptr + i * b_bs * es, gb.dtype, gb.rs, gb.cs};
      OJC_TRY(gemm_auto(be, op, ai, bi, (char*)cptr + i * c_bs * es, dt, n_, m_, n_, k_, 1.0f, false, nullptr));
    }
    return OJC_OK;
  };
  auto run = [&]() -> ojc_status {
    const int64_t parts = norm_partials(n);
    const unsigned nb = (unsigned)batch;
    muon_momentum_kernel<<<dim3((unsigned)parts, nb), 256, 0, be->stream>>>(mb, u, n, (float)cfg.momentum, cfg.nesterov, bf ? 1 : 0, grad_scale_dev, part, be->fault_dev);
    OJC_LAUNCHED(be, op);
    muon_norm_kernel<<<nb, 256, 0, be->stream>>>(part, parts, norm);
    OJC_LAUNCHED(be, op);
    const int grid = elementwise_grid(be, n, 256), grid_all = elementwise_grid(be, n * batch, 256), grid_a = elementwise_grid(be, r * r * batch, 256);
    bool mirrors_aligned = ((uintptr_t)u & 15) == 0 && ((uintptr_t)x & 7) == 0;
    for (int64_t i = 0; i < batch; ++i) mirrors_aligned = mirrors_aligned && ((uintptr_t)mb.p[i] & 15) == 0 && ((uintptr_t)mb.mirror[i] & 7) == 0;
    const dim3 tgrid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), nb), tblock(32, 8);
    const bool tiled = tall && nb <= 65535 && (rows + 31) / 32 <= 65535;
    if (tiled && bf) muon_normalize_tall_kernel<bf16><<<tgrid, tblock, 0, be->stream>>>(u, norm, (bf16*)x, (int)rows, (int)cols, 1);
    else if (tiled) muon_normalize_tall_kernel<float><<<tgrid, tblock, 0, be->stream>>>(u, norm, (float*)x, (int)rows, (int)cols, 0);
    else if (bf && !tall && n % 4 == 0 && mirrors_aligned) muon_normalize_bf16x4_kernel<<<dim3(elementwise_grid(be, n / 4, 256), nb), 256, 0, be->stream>>>(u, norm, (bf16*)x, n);
    else if (bf) muon_normalize_kernel<bf16><<<dim3(grid, nb), 256, 0, be->stream>>>(u, norm, (bf16*)x, (int)rows, (int)cols, tall, 1);
    else muon_normalize_kernel<float><<<dim3(grid, nb), 256, 0, be->stream>>>(u, norm, (float*)x, (int)rows, (int)cols, tall, 0);
    OJC_LAUNCHED(be, op);
    const float a = (float)3.4445, b = (float)-4.7750, cc = (float)2.0315;  // MUON_NS5_{A,B,C}, ojas-core/src/backend.rs:144-146
    const size_t small_smem = ((size_t)2 * r * c + 2 * 32 * 33) * 4;
    const bool small = r <= 32 && small_smem <= 200 * 1024;     // e.g. the [heads, d] gate weights: one CTA per matrix, alone or in a group
    if (small) {
      static PerDeviceFlag attr_of;
      bool& attr = attr_of[be->device];
      if (!attr) {
        OJC_CUDA(be, cudaFuncSetAttribute(muon_small_ns5_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), op);
        OJC_CUDA(be, cudaFuncSetAttribute(muon_small_ns5_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), op);
        attr = true;
      }
      if (bf) muon_small_ns5_kernel<bf16><<<nb, 512, small_smem, be->stream>>>((bf16*)x, (int)r, (int)c, a, b, cc, 1, be->fault_dev);
      else muon_small_ns5_kernel<float><<<nb, 512, small_smem, be->stream>>>((float*)x, (int)r, (int)c, a, b, cc, 0, be->fault_dev);
      OJC_LAUNCHED(be, op);
    }
    for (int it = 0; it < 5 && !small; ++it) {
      GemmOperand xk{x, dt, c, 1}, xt{x, dt, 1, c}, xn{x, dt, c, 1};
      OJC_TRY(product(xk, xt, am, r, r, c, n, n, r * r));                                                  // A = X X^T
      GemmOperand ak{am, dt, r, 1}, an{am, dt, r, 1};
      bool fused_a = false, fused_x = false;
      const NsCombine comb_a{am, r, r * r, b, cc};                                                          // B = b A + c (A A)
      OJC_TRY(product(ak, an, a2, r, r, r, r * r, r * r, r * r, bf ? &comb_a : nullptr, &fused_a));           // A2 = A A (-> B in the epilogue)
      if (!fused_a) {
        const bool v8a = bf && (r * r * batch) % 8 == 0 && (((uintptr_t)am | (uintptr_t)a2) & 15) == 0;
        if (v8a) ns_combine_a_bf16x8_kernel<<<elementwise_grid(be, r * r * batch / 8, 256), 256, 0, be->stream>>>((const uint4*)am, (uint4*)a2, r * r * batch / 8, b, cc);
        else if (bf) ns_combine_a_kernel<bf16><<<grid_a, 256, 0, be->stream>>>((const bf16*)am, (bf16*)a2, r * r * batch, b, cc, 1);
        else ns_combine_a_kernel<float><<<grid_a, 256, 0, be->stream>>>((const float*)am, (float*)a2, r * r * batch, b, cc, 0);
        OJC_LAUNCHED(be, op);
      }
      GemmOperand bk{a2, dt, r, 1};
      const NsCombine comb_x{x, c, n, a, 1.0f};                                                             // X <- a X + B X
      OJC_TRY(product(bk, xn, bx, r, c, r, r * r, n, n, bf ? &comb_x : nullptr, &fused_x));                   // BX = B X (-> the new X in the epilogue)
      if (!fused_x) {
        const bool v8x = bf && (n * batch) % 8 == 0 && (((uintptr_t)x | (uintptr_t)bx) & 15) == 0;
        if (v8x) ns_combine_x_bf16x8_kernel<<<elementwise_grid(be, n * batch / 8, 256), 256, 0, be->stream>>>((const uint4*)x, (uint4*)bx, n * batch / 8, a, be->fault_dev);
        else if (bf) ns_combine_x_kernel<bf16><<<grid_all, 256, 0, be->stream>>>((const bf16*)x, (bf16*)bx, n * batch, a, 1, be->fault_dev);
        else ns_combine_x_kernel<float><<<grid_all, 256, 0, be->stream>>>((const float*)x, (float*)bx, n * batch, a, 0, be->fault_dev);
        OJC_LAUNCHED(be, op);
      }
      std::swap(x, bx);
    }
    const double scale = std::sqrt(std::max(1.0, (double)rows / (double)cols));
    const float alpha = (float)(-cfg.lr * scale), decay = (float)(1.0 - cfg.lr * cfg.weight_decay);
    if (tiled && bf) muon_apply_tall_kernel<bf16><<<tgrid, tblock, 0, be->stream>>>(mb, (const bf16*)x, (int)rows, (int)cols, alpha, decay, cfg.weight_decay != 0.0, be->fault_dev, grad_scale_dev);
    else if (tiled) muon_apply_tall_kernel<float><<<tgrid, tblock, 0, be->stream>>>(mb, (const float*)x, (int)rows, (int)cols, alpha, decay, cfg.weight_decay != 0.0, be->fault_dev, grad_scale_dev);
    else if (bf && !tall && n % 4 == 0 && mirrors_aligned) muon_apply_bf16x4_kernel<<<dim3(elementwise_grid(be, n / 4, 256), nb), 256, 0, be->stream>>>(mb, (const bf16*)x, n, alpha, decay, cfg.weight_decay != 0.0, be->fault_dev, grad_scale_dev);
    else if (bf) muon_apply_kernel<bf16><<<dim3(grid, nb), 256, 0, be->stream>>>(mb, (const bf16*)x, (int)rows, (int)cols, tall, alpha, decay, cfg.weight_decay != 0.0, be->fault_dev, grad_scale_dev);
    else muon_apply_kernel<float><<<dim3(grid, nb), 256, 0, be->stream>>>(mb, (const float*)x, (int)rows, (int)cols, tall, alpha, decay, cfg.weight_decay != 0.0, be->fault_dev, grad_scale_dev);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  };
  st = run();
  ojc_free(be, ws);
  return st;
}

ojc_status muon_device(ojc_backend* be, float* p, const float* g, float* mom, bf16* mirror, int64_t rows, int64_t cols, const ojc_muon_config& cfg,
                       const float* grad_scale_dev) {
  return muon_group_device(be, &p, &g, &mom, mirror ? &mirror : nullptr, 1, rows, cols, cfg, grad_scale_dev);
}

extern "C" {

ojc_status ojc_clip_grad_norm(ojc_backend* be, ojc_tensor* const* grads, int64_t count, float max_norm, float* norm_out) {
  const char* op = "clip_grad_norm";
  OJC_ALIVE(be, op);
  if (count < 0 || (count > 0 && !grads)) return ojc_fail(OJC_ERR_SHAPE, op, "bad gradient list");
  if (std::isnan(max_norm) || max_norm == -INFINITY) return ojc_fail(OJC_ERR_NON_FINITE, op, "max_norm is not a number");
  if (max_norm < 0.0f) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "max_norm is negative");
  std::vector<const float*> ptrs(count);
  std::vector<int64_t> lens(count);
  for (int64_t i = 0; i < count; ++i) {
    OJC_TRY(check_tensor(op, "grad", grads[i]));
    if (grads[i]->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "gradients must be F32");
    ptrs[i] = (const float*)grads[i]->data; lens[i] = numel(grads[i]);
  }
  void* ns = nullptr;
  OJC_TRY(ojc_alloc(be, 8, &ns));
  ojc_status st = grad_norm_device(be, ptrs.data(), lens.data(), count, std::isinf(max_norm) ? 3.0e38f : max_norm, (float*)ns);
  float host[2] = {0, 1};
  if (st == OJC_OK) st = ojc_download(be, host, ns, 8);  // the sync point: also reports a deferred fault (the norm pass is the NaN scan)
  if (st == OJC_OK && !std::isfinite(host[0])) st = ojc_fail(OJC_ERR_NON_FINITE, op, "the gradient norm is not finite");
  if (st == OJC_OK && host[1] < 1.0f)
    for (int64_t i = 0; i < count && st == OJC_OK; ++i) st = scale_by_device(be, (float*)grads[i]->data, lens[i], (float*)ns + 1);
  ojc_free(be, ns);
  if (norm_out) *norm_out = host[0];
  return st;
}

ojc_status ojc_adamw_step(ojc_backend* be, ojc_tensor* param, const ojc_tensor* grad, ojc_tensor* m, ojc_tensor* v, uint64_t step_before,
                          const ojc_adamw_config* cfg, ojc_tensor* mirror) {
  const char* op = "adamw_step";
  OJC_ALIVE(be, op);
  if (!cfg) return ojc_fail(OJC_ERR_BACKEND, op, "null config");
  OJC_TRY(check_tensor(op, "param", param)); OJC_TRY(check_tensor(op, "grad", grad)); OJC_TRY(check_tensor(op, "m", m)); OJC_TRY(check_tensor(op, "v", v));
  if (!same_shape(param, grad) || !same_shape(param, m) || !same_shape(param, v)) return ojc_fail(OJC_ERR_SHAPE, op, "param, grad, m, v must share a shape");
  if (param->dtype != OJC_F32 || grad->dtype != OJC_F32 || m->dtype != OJC_F32 || v->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "param, grad, m, v must be F32");
  if (mirror) { OJC_TRY(check_tensor(op, "bf16_mirror", mirror)); if (mirror->dtype != OJC_BF16 || numel(mirror) != numel(param)) return ojc_fail(OJC_ERR_SHAPE, op, "mirror must be BF16 of the parameter's size"); }
  if (numel(param) == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  return adamw_device(be, (float*)param->data, (const float*)grad->data, (float*)m->data, (float*)v->data, mirror ? (bf16*)mirror->data : nullptr,
                      numel(param), step_before, *cfg, nullptr);
}

ojc_status ojc_muon_ns5_step(ojc_backend* be, ojc_tensor* param, const ojc_tensor* grad, ojc_tensor* momentum, const ojc_muon_config* cfg, ojc_tensor* mirror) {
  const char* op = "muon_ns5_step";
  OJC_ALIVE(be, op);
  if (!cfg) return ojc_fail(OJC_ERR_BACKEND, op, "null config");
  OJC_TRY(check_tensor(op, "param", param)); OJC_TRY(check_tensor(op, "grad", grad)); OJC_TRY(check_tensor(op, "momentum", momentum));
  if (param->rank != 2 || !same_shape(param, grad) || !same_shape(param, momentum)) return ojc_fail(OJC_ERR_SHAPE, op, "param, grad, momentum must be one [rows, cols] shape");
  if (param->dtype != OJC_F32 || grad->dtype != OJC_F32 || momentum->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "param, grad, momentum must be F32");
  if (mirror) { OJC_TRY(check_tensor(op, "bf16_mirror", mirror)); if (mirror->dtype != OJC_BF16 || numel(mirror) != numel(param)) return ojc_fail(OJC_ERR_SHAPE, op, "mirror must be BF16 of the parameter's size"); }
  return muon_device(be, (float*)param->data, (const float*)grad->data, (float*)momentum->data, mirror ? (bf16*)mirror->data : nullptr, param->shape[0],
                     param->shape[1], *cfg, nullptr);
}

ojc_status ojc_optimizer_scratch_bytes(ojc_backend* be, int32_t kind, int64_t rows, int64_t cols, uint64_t* bytes) {
  if (!bytes) return ojc_fail(OJC_ERR_BACKEND, "optimizer_scratch_bytes", "null out pointer");
  if (kind == 0) { *bytes = 0; return OJC_OK; }
  if (kind == 1) { *bytes = std::max(muon_scratch_bytes(rows, cols, false), muon_scratch_bytes(rows, cols, true)); return OJC_OK; }
  return ojc_fail(OJC_ERR_UNSUPPORTED, "optimizer_scratch_bytes", "unknown optimizer kind");
}

}  // extern "C"
