// Mean cross-entropy over logits, and the fused tied-head form
// linear_cross_entropy_mean that never holds [N, V] logits: rows are processed
// in tiles (logits tile -> row statistics -> d(logits) -> dX, dW GEMMs).
//
// Per row (ojas-cpu/src/pointwise.rs:2329-2390, fused_ce.rs:290-452):
//   loss_n = max + ln(sum exp(z - max)) - z[target];  G = (softmax - onehot) / n_valid
// A row whose target holds the maximum and whose sum rounds to 1 uses the
// target-excluded form: loss = log1p(s), G_target = -(s / (1 + s)) / n_valid with
// s = sum over the other classes (the softmax-collapse rule, pointwise.rs:2300-2307).
// Rows whose target equals ignore_index contribute nothing and get a zero gradient.
#include "ce.cuh"
#include "common.cuh"
#include "dispatch.cuh"
#include "gemm.cuh"
#include "linear.cuh"
#include "tc_common.cuh"

namespace {

// valid[0] = number of non-ignored targets; a target outside the vocabulary raises the range fault.
__global__ void ce_count_kernel(const uint32_t* __restrict__ targets, int64_t rows, int has_ignore, uint32_t ignore, int64_t vocab, uint32_t* __restrict__ valid,
                                uint32_t* fault) {
  __shared__ uint32_t red[32];
  uint32_t cnt = 0;
  for (int64_t i = threadIdx.x; i < rows; i += blockDim.x) {
    uint32_t t = targets[i];
    if (has_ignore && t == ignore) continue;
    if (t >= vocab) { raise_fault(fault, OP_ID_RANGE); continue; }
    ++cnt;
  }
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t total = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += red[w];
    valid[0] = total;
    if (total == 0) raise_fault(fault, OP_CE);  // an all-ignored batch has no mean (fused_ce.rs:148-150)
  }
}

// One block per row. terms[row] = the row's loss term (0 for ignored rows). grad (optional) = G row.
template <class TL, class TG>
__global__ void ce_rows_kernel(const TL* __restrict__ logits, int64_t ld, const uint32_t* __restrict__ targets, int64_t vocab, int has_ignore, uint32_t ignore,
                               const uint32_t* __restrict__ valid, float* __restrict__ terms, TG* __restrict__ grad, int64_t ldg, float seed, uint32_t* fault) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const TL* z = logits + row * ld;
  const uint32_t target = targets[row];
  const bool ignored = has_ignore && target == ignore;
  if (ignored || target >= vocab) {
    if (threadIdx.x == 0) terms[row] = 0.0f;
    if (grad) for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) stf(grad, row * ldg + c, 0.0f);
    return;
  }
  // one pass for both statistics: each thread keeps a running (max, sum) over its columns, then the block combines them
  float tm = -INFINITY, ts = 0.0f;
  for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) {
    const float v = ldf(z, c);
    if (v > tm) { ts = ts * expf(tm - v) + 1.0f; tm = v; }
    else ts += expf(v - tm);
  }
  const float mx = block_max(tm, red);
  float sum = block_sum(tm == -INFINITY ? 0.0f : ts * expf(tm - mx), red);
  const float picked = ldf(z, target);
  if (!(isfinite(mx) && isfinite(sum) && sum > 0.0f)) { if (threadIdx.x == 0) { raise_fault(fault, OP_CE); terms[row] = 0.0f; } }
  float other = 0.0f;
  bool collapsed = false;
  if (picked == mx && sum == 1.0f) {
    float o = 0.0f;
    for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) if (c != target) o += expf(ldf(z, c) - mx);
    other = block_sum(o, red);
    collapsed = other > 0.0f;
  }
  if (threadIdx.x == 0) terms[row] = collapsed ? log1pf(other) : (mx + logf(sum) - picked);
  if (grad) {
    const float denom = (float)valid[0];
    const float inv = collapsed ? 1.0f / (1.0f + other) : 1.0f / sum;
    for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) {
      float g = (expf(ldf(z, c) - mx) * inv) / denom;
      if (c == target) g = collapsed ? -(other * inv) / denom : g - 1.0f / denom;
      stf(grad, row * ldg + c, g * seed);
    }
  }
}

// The bf16-tier form of ce_rows_kernel for F32 logits and a BF16 gradient: 512 threads per row and two rows per SM (so the
// rows in flight stay inside L2 between the statistics pass and the gradient pass), 128-bit loads, ex2.approx on
// log2-scaled differences, one multiply per gradient element. Same row rules as above.
__device__ __forceinline__ float ex2_fast(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) { uint32_t r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }

__global__ void __launch_bounds__(512, 2)
ce_rows_fast_kernel(const float* __restrict__ logits, int64_t ld, const uint32_t* __restrict__ targets, int64_t vocab, int has_ignore, uint32_t ignore,
                    const uint32_t* __restrict__ valid, float* __restrict__ terms, bf16* __restrict__ grad, int64_t ldg, float seed, uint32_t* fault) {
  __shared__ float red[32];
  constexpr float L2E = 1.4426950408889634f;
  const int64_t row = blockIdx.x;
  const float* z = logits + row * ld;
  bf16* g = grad ? grad + row * ldg : nullptr;
  const uint32_t target = targets[row];
  const int64_t v4 = vocab >> 2;            // whole float4 groups; the tail (vocab % 4) is handled by scalar code
  if ((has_ignore && target == ignore) || target >= vocab) {
    if (threadIdx.x == 0) terms[row] = 0.0f;
    if (g) {
      for (int64_t i = threadIdx.x; i < v4; i += blockDim.x) *reinterpret_cast<uint2*>(g + 4 * i) = make_uint2(0u, 0u);
      for (int64_t c = 4 * v4 + threadIdx.x; c < vocab; c += blockDim.x) g[c] = __float2bfloat16_rn(0.0f);
    }
    return;
  }
  float tm = -INFINITY, ts = 0.0f;          // running maximum (log2 domain) and sum of 2^(v - tm)
#pragma unroll 4
  for (int64_t i = threadIdx.x; i < v4; i += blockDim.x) {
    const float4 t = *reinterpret_cast<const float4*>(z + 4 * i);
    const float a = t.x * L2E, b = t.y * L2E, c = t.z * L2E, d = t.w * L2E;
    const float m4 = fmaxf(fmaxf(a, b), fmaxf(c, d));
    if (m4 > tm) { ts *= ex2_fast(tm - m4); tm = m4; }
    ts += ex2_fast(a - tm) + ex2_fast(b - tm) + ex2_fast(c - tm) + ex2_fast(d - tm);
  }
  for (int64_t c = 4 * v4 + threadIdx.x; c < vocab; c += blockDim.x) {
    const float a = z[c] * L2E;
    if (a > tm) { ts *= ex2_fast(tm - a); tm = a; }
    ts += ex2_fast(a - tm);
  }
  const float mx2 = block_max(tm, red);
  const float sum = block_sum(tm == -INFINITY ? 0.0f : ts * ex2_fast(tm - mx2), red);
  const float picked = z[target];
  const float mx = mx2 * (1.0f / L2E);
  if (!(isfinite(mx2) && isfinite(sum) && sum > 0.0f)) { if (threadIdx.x == 0) { raise_fault(fault, OP_CE); terms[row] = 0.0f; } }
  float other = 0.0f;
  bool collapsed = false;
  if (picked * L2E == mx2 && sum == 1.0f) {
    float o = 0.0f;
    for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) if (c != target) o += ex2_fast(z[c] * L2E - mx2);
    other = block_sum(o, red);
    collapsed = other > 0.0f;
  }
  if (threadIdx.x == 0) terms[row] = collapsed ? log1pf(other) : (mx + logf(sum) - picked);
  if (!g) return;
  const float denom = (float)valid[0];
  const float inv = collapsed ? 1.0f / (1.0f + other) : 1.0f / sum;
  const float k = inv / denom * seed;
#pragma unroll 4
  for (int64_t i = threadIdx.x; i < v4; i += blockDim.x) {
    const float4 t = *reinterpret_cast<const float4*>(z + 4 * i);
    *reinterpret_cast<uint2*>(g + 4 * i) = make_uint2(pack_bf16x2(ex2_fast(fmaf(t.x, L2E, -mx2)) * k, ex2_fast(fmaf(t.y, L2E, -mx2)) * k),
                                                      pack_bf16x2(ex2_fast(fmaf(t.z, L2E, -mx2)) * k, ex2_fast(fmaf(t.w, L2E, -mx2)) * k));
  }
  for (int64_t c = 4 * v4 + threadIdx.x; c < vocab; c += blockDim.x) g[c] = __float2bfloat16_rn(ex2_fast(fmaf(z[c], L2E, -mx2)) * k);
  __syncthreads();
  if (threadIdx.x == 0) {
    const float gt = collapsed ? -(other * inv) / denom : (ex2_fast(fmaf(picked, L2E, -mx2)) * inv) / denom - 1.0f / denom;
    g[target] = __float2bfloat16_rn(gt * seed);
  }
}

// The bf16 step's form: BF16 logits (the head GEMM's output, rounded once from its f32 accumulator, as a matmul output is under
// torch's autocast) turned into the BF16 gradient IN PLACE: a thread reads the same 8-value groups in both passes and overwrites only
// those, so no second tile exists. Statistics and the loss term are f32. 6 bytes per logit cross HBM for the head (GEMM write 2,
// read 2, write 2) instead of 10 with an f32 tile and a separate gradient tile. Three passes over a row (the later ones hit L2):
// maximum; one ex2 per logit, summed in f32 and written back as bf16 exponentials; exponentials scaled into the gradient. The
// gradient therefore carries two bf16 roundings (the exponential's and its own). Same row rules as above.
__device__ __forceinline__ void unpack_bf16x8(const uint4& t, float (&v)[8]) {
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
constexpr size_t CE_ROW_SMEM_MAX = 112 * 1024;   // two such rows and the reduction scratch fit in an SM
int g_ce_rows_variant = 0;                       // ojc_ce_rows_variant: 0 the library's choice, 1 always the form that keeps the row in L2, 2 a CTA per row with the row in shared memory

__global__ void __launch_bounds__(512, 2)
ce_rows_inplace_bf16_kernel(bf16* __restrict__ logits, int64_t ld, const uint32_t* __restrict__ targets, int64_t vocab, int has_ignore, uint32_t ignore,
                            const uint32_t* __restrict__ valid, float* __restrict__ terms, int want_grad, float seed, uint32_t* fault) {
  pdl_trigger();
  __shared__ float red[32];
  constexpr float L2E = 1.4426950408889634f;
  const int64_t row = blockIdx.x;
  bf16* z = logits + row * ld;
  const uint32_t target = targets[row];
  const int64_t v8 = vocab >> 3;            // whole 16-byte groups; the tail (vocab % 8) is handled by scalar code
  if ((has_ignore && target == ignore) || target >= vocab) {
    if (threadIdx.x == 0) terms[row] = 0.0f;
    if (want_grad) {
      for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) *reinterpret_cast<uint4*>(z + 8 * i) = make_uint4(0u, 0u, 0u, 0u);
      for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) z[c] = __float2bfloat16_rn(0.0f);
    }
    return;
  }
  const float picked = __bfloat162float(z[target]);   // read before any thread overwrites the row
  // pass 1: the row maximum (no exponentials)
  float tm = -INFINITY;
#pragma unroll 2
  for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) {
    float v[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(z + 8 * i), v);
#pragma unroll
    for (int e = 0; e < 8; ++e) tm = fmaxf(tm, v[e]);
  }
  for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) tm = fmaxf(tm, __bfloat162float(z[c]));
  const float mx = block_max(tm, red);
  const float mx2 = mx * L2E;
  // pass 2: one ex2 per logit. The sum is taken over the f32 exponentials; when a gradient is wanted each group is written back
  // as bf16 exponentials over the logits it came from (a thread reads and writes the same groups in every pass)
  float ts = 0.0f;
#pragma unroll 2
  for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) {
    float v[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(z + 8 * i), v);
#pragma unroll
    for (int e = 0; e < 8; ++e) { v[e] = ex2_fast(fmaf(v[e], L2E, -mx2)); ts += v[e]; }
    if (want_grad) *reinterpret_cast<uint4*>(z + 8 * i) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  }
  for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) {
    const float e = ex2_fast(fmaf(__bfloat162float(z[c]), L2E, -mx2));
    ts += e;
    if (want_grad) z[c] = __float2bfloat16_rn(e);
  }
  const float sum = block_sum(ts, red);
  if (!(isfinite(mx2) && isfinite(sum) && sum > 0.0f)) { if (threadIdx.x == 0) { raise_fault(fault, OP_CE); terms[row] = 0.0f; } }
  // the target-excluded form for a collapsed row (the target holds the maximum and the sum rounds to 1): the others' exponentials
  float other = 0.0f;
  bool collapsed = false;
  if (picked == mx && sum == 1.0f) {
    float o = 0.0f;
    if (want_grad) { for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) if (c != target) o += __bfloat162float(z[c]); }        // the row now holds exponentials
    else { for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) if (c != target) o += ex2_fast(fmaf(__bfloat162float(z[c]), L2E, -mx2)); }
    other = block_sum(o, red);
    collapsed = other > 0.0f;
  }
  if (threadIdx.x == 0) terms[row] = collapsed ? log1pf(other) : (mx + logf(sum) - picked);
  if (!want_grad) return;
  const float denom = (float)valid[0];
  const float inv = collapsed ? 1.0f / (1.0f + other) : 1.0f / sum;
  const float k = inv / denom * seed;
  // pass 3: exponentials -> gradient, one multiply each
#pragma unroll 2
  for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) {
    float v[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(z + 8 * i), v);
    *reinterpret_cast<uint4*>(z + 8 * i) = make_uint4(pack_bf16x2(v[0] * k, v[1] * k), pack_bf16x2(v[2] * k, v[3] * k), pack_bf16x2(v[4] * k, v[5] * k), pack_bf16x2(v[6] * k, v[7] * k));
  }
  for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) z[c] = __float2bfloat16_rn(__bfloat162float(z[c]) * k);
  __syncthreads();
  if (threadIdx.x == 0) {
    const float gt = collapsed ? -(other * inv) / denom : (ex2_fast(fmaf(picked, L2E, -mx2)) * inv) / denom - 1.0f / denom;
    z[target] = __float2bfloat16_rn(gt * seed);
  }
}

// The same kernel with the row held in shared memory: a row of the 124M head (50304 bf16 = 98.25 KB) fits twice in an SM, so the row
// crosses the SM's memory port once in each direction (the form above reads it three times and writes it twice through L2, which is
// what bounded it: 1.16 GB in and 1.65 GB out per 8192-row tile against 0.82 GB each way here). The maximum is taken while the row
// is copied in, the exponentials replace the logits in shared memory, and the gradient goes straight out. The same arithmetic on the
// same elements in the same per-thread order as the form above, so the same bits.
__global__ void __launch_bounds__(512, 2)
ce_rows_smem_bf16_kernel(bf16* __restrict__ logits, int64_t ld, const uint32_t* __restrict__ targets, int64_t vocab, int has_ignore, uint32_t ignore,
                         const uint32_t* __restrict__ valid, float* __restrict__ terms, int want_grad, float seed, uint32_t* fault) {
  pdl_trigger();
  extern __shared__ __align__(16) uint8_t row_raw[];
  __shared__ float red[32];
  bf16* srow = reinterpret_cast<bf16*>(row_raw);
  constexpr float L2E = 1.4426950408889634f;
  const int64_t row = blockIdx.x;
  bf16* z = logits + row * ld;
  const uint32_t target = targets[row];
  const int64_t v8 = vocab >> 3;            // whole 16-byte groups; the tail (vocab % 8) is handled by scalar code
  if ((has_ignore && target == ignore) || target >= vocab) {
    if (threadIdx.x == 0) terms[row] = 0.0f;
    if (want_grad) {
      for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) *reinterpret_cast<uint4*>(z + 8 * i) = make_uint4(0u, 0u, 0u, 0u);
      for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) z[c] = __float2bfloat16_rn(0.0f);
    }
    return;
  }
  const float picked = __bfloat162float(z[target]);
  // pass 1: copy the row in, taking the maximum on the way
  float tm = -INFINITY;
#pragma unroll 4
  for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) {
    const uint4 t = *reinterpret_cast<const uint4*>(z + 8 * i);
    *reinterpret_cast<uint4*>(srow + 8 * i) = t;
    float v[8];
    unpack_bf16x8(t, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) tm = fmaxf(tm, v[e]);
  }
  for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) { srow[c] = z[c]; tm = fmaxf(tm, __bfloat162float(srow[c])); }
  const float mx = block_max(tm, red);      // (its barriers also make the copied row visible to every thread)
  const float mx2 = mx * L2E;
  // pass 2: one ex2 per logit, summed in f32; the bf16 exponentials replace the logits in shared memory
  float ts = 0.0f;
#pragma unroll 2
  for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) {
    float v[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(srow + 8 * i), v);
#pragma unroll
    for (int e = 0; e < 8; ++e) { v[e] = ex2_fast(fmaf(v[e], L2E, -mx2)); ts += v[e]; }
    *reinterpret_cast<uint4*>(srow + 8 * i) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  }
  for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) {
    const float e = ex2_fast(fmaf(__bfloat162float(srow[c]), L2E, -mx2));
    ts += e;
    srow[c] = __float2bfloat16_rn(e);
  }
  const float sum = block_sum(ts, red);
  if (!(isfinite(mx2) && isfinite(sum) && sum > 0.0f)) { if (threadIdx.x == 0) { raise_fault(fault, OP_CE); terms[row] = 0.0f; } }
  float other = 0.0f;
  bool collapsed = false;
  if (picked == mx && sum == 1.0f) {        // the target-excluded form for a collapsed row: the others' exponentials (the row holds them now)
    float o = 0.0f;
    for (int64_t c = threadIdx.x; c < vocab; c += blockDim.x) if (c != target) o += __bfloat162float(srow[c]);
    other = block_sum(o, red);
    collapsed = other > 0.0f;
  }
  if (threadIdx.x == 0) terms[row] = collapsed ? log1pf(other) : (mx + logf(sum) - picked);
  if (!want_grad) return;
  const float denom = (float)valid[0];
  const float inv = collapsed ? 1.0f / (1.0f + other) : 1.0f / sum;
  const float k = inv / denom * seed;
  // pass 3: exponentials -> gradient, one multiply each, out to the logits' place
#pragma unroll 4
  for (int64_t i = threadIdx.x; i < v8; i += blockDim.x) {
    float v[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(srow + 8 * i), v);
    *reinterpret_cast<uint4*>(z + 8 * i) = make_uint4(pack_bf16x2(v[0] * k, v[1] * k), pack_bf16x2(v[2] * k, v[3] * k), pack_bf16x2(v[4] * k, v[5] * k), pack_bf16x2(v[6] * k, v[7] * k));
  }
  for (int64_t c = 8 * v8 + threadIdx.x; c < vocab; c += blockDim.x) z[c] = __float2bfloat16_rn(__bfloat162float(srow[c]) * k);
  __syncthreads();
  if (threadIdx.x == 0) {
    const float gt = collapsed ? -(other * inv) / denom : (ex2_fast(fmaf(picked, L2E, -mx2)) * inv) / denom - 1.0f / denom;
    z[target] = __float2bfloat16_rn(gt * seed);
  }
}

// The streaming form, for whole tiles of such rows: one persistent CTA per SM with two row buffers. A seventeenth warp moves the rows:
// cp.async.bulk brings row k + 2 into a buffer as soon as the bulk store of row k has read it, so the loads and stores of neighbouring
// rows are in flight while the sixteen compute warps work on the row between them; the compute warps never touch global memory for
// the row itself (the gradient is formed in place in shared memory, target column included, and leaves as one bulk store). The same
// arithmetic on the same elements in the same per-thread order as the two forms above, so the same bits. Needs vocab % 8 == 0.
__device__ __forceinline__ void ce_bar_compute() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ float ce_block_sum16(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  ce_bar_compute();
  if (lane == 0) red[warp] = v;
  ce_bar_compute();
  return warp_sum(lane < 16 ? red[lane] : 0.0f);
}
__device__ __forceinline__ float ce_block_max16(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  ce_bar_compute();
  if (lane == 0) red[warp] = v;
  ce_bar_compute();
  return warp_max(lane < 16 ? red[lane] : -INFINITY);
}
constexpr int CE_STREAM_THREADS = 544;
__global__ void __launch_bounds__(CE_STREAM_THREADS, 1)
ce_rows_stream_bf16_kernel(bf16* __restrict__ logits, int64_t ld, const uint32_t* __restrict__ targets, int64_t rows, int64_t vocab, int has_ignore, uint32_t ignore,
                           const uint32_t* __restrict__ valid, float* __restrict__ terms, int want_grad, float seed, uint32_t* fault) {
  pdl_trigger();
  extern __shared__ __align__(128) uint8_t row_raw[];
  __shared__ float red[32];
  __shared__ __align__(8) uint64_t bars[4];          // full[2] (bytes of a row have landed), done[2] (the compute warps are through with it)
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  constexpr float L2E = 1.4426950408889634f;
  const uint32_t row_bytes = (uint32_t)vocab * 2u, stride = (row_bytes + 127u) & ~127u;
  const uint32_t buf0 = tc::smem_u32(row_raw), bar0 = tc::smem_u32(bars);
  if (threadIdx.x == 0) {
    tc::mbar_init(bar0, 1); tc::mbar_init(bar0 + 8, 1); tc::mbar_init(bar0 + 16, 512); tc::mbar_init(bar0 + 24, 512);
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int64_t v8 = vocab >> 3;
  if (threadIdx.x >= 512) {
    // ------------------------------------------------------------ the rows' mover
    if (threadIdx.x == 512) {
      auto load = [&](int64_t row, uint32_t b) {
        tc::mbar_expect_tx(bar0 + 8 * b, row_bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(buf0 + b * stride), "l"(logits + row * ld), "r"(row_bytes),
                     "r"(bar0 + 8 * b) : "memory");
      };
      const int64_t first = blockIdx.x, step = gridDim.x;
      if (first < rows) load(first, 0);
      if (first + step < rows) load(first + step, 1);
      uint32_t k = 0;
      for (int64_t row = first; row < rows; row += step, ++k) {
        const uint32_t b = k & 1;
        if (!tc::mbar_wait(bar0 + 16 + 8 * b, (k >> 1) & 1, fault, abort_flag)) break;
        if (want_grad) {
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(logits + row * ld), "r"(buf0 + b * stride), "r"(row_bytes) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");       // the buffer may be refilled
        }
        if (row + 2 * step < rows) load(row + 2 * step, b);
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    return;
  }
  // ------------------------------------------------------------ the compute warps
  const float denom = (float)valid[0];
  uint32_t k = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, ++k) {
    const uint32_t b = k & 1;
    bf16* srow = reinterpret_cast<bf16*>(row_raw + b * stride);
    const uint32_t target = targets[row];
    if (!tc::mbar_wait(bar0 + 8 * b, (k >> 1) & 1, fault, abort_flag)) break;
    if ((has_ignore && target == ignore) || target >= vocab) {
      if (threadIdx.x == 0) terms[row] = 0.0f;
      if (want_grad) for (int64_t i = threadIdx.x; i < v8; i += 512) *reinterpret_cast<uint4*>(srow + 8 * i) = make_uint4(0u, 0u, 0u, 0u);
    } else {
      const float picked = __bfloat162float(srow[target]);
      float tm = -INFINITY;
#pragma unroll 2
      for (int64_t i = threadIdx.x; i < v8; i += 512) {
        float v[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(srow + 8 * i), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) tm = fmaxf(tm, v[e]);
      }
      const float mx = ce_block_max16(tm, red);
      const float mx2 = mx * L2E;
      float ts = 0.0f;
#pragma unroll 2
      for (int64_t i = threadIdx.x; i < v8; i += 512) {
        float v[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(srow + 8 * i), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) { v[e] = ex2_fast(fmaf(v[e], L2E, -mx2)); ts += v[e]; }
        *reinterpret_cast<uint4*>(srow + 8 * i) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
      }
      const float sum = ce_block_sum16(ts, red);
      if (!(isfinite(mx2) && isfinite(sum) && sum > 0.0f)) { if (threadIdx.x == 0) { raise_fault(fault, OP_CE); terms[row] = 0.0f; } }
      float other = 0.0f;
      bool collapsed = false;
      if (picked == mx && sum == 1.0f) {
        float o = 0.0f;
        for (int64_t c = threadIdx.x; c < vocab; c += 512) if (c != target) o += __bfloat162float(srow[c]);
        other = ce_block_sum16(o, red);
        collapsed = other > 0.0f;
      }
      if (threadIdx.x == 0) terms[row] = collapsed ? log1pf(other) : (mx + logf(sum) - picked);
      if (want_grad) {
        const float inv = collapsed ? 1.0f / (1.0f + other) : 1.0f / sum;
        const float kk = inv / denom * seed;
#pragma unroll 2
        for (int64_t i = threadIdx.x; i < v8; i += 512) {
          float v[8];
          unpack_bf16x8(*reinterpret_cast<const uint4*>(srow + 8 * i), v);
          *reinterpret_cast<uint4*>(srow + 8 * i) =
              make_uint4(pack_bf16x2(v[0] * kk, v[1] * kk), pack_bf16x2(v[2] * kk, v[3] * kk), pack_bf16x2(v[4] * kk, v[5] * kk), pack_bf16x2(v[6] * kk, v[7] * kk));
        }
        ce_bar_compute();
        if (threadIdx.x == 0) {
          const float gt = collapsed ? -(other * inv) / denom : (ex2_fast(fmaf(picked, L2E, -mx2)) * inv) / denom - 1.0f / denom;
          srow[target] = __float2bfloat16_rn(gt * seed);
        }
      }
    }
    tc::fence_async_smem();                   // the row's new contents, before the bulk store reads them
    tc::mbar_arrive(bar0 + 16 + 8 * b);
  }
}

// loss = (sum of the row terms, added in a fixed tree order) / n_valid
__global__ void ce_loss_finish_kernel(const float* __restrict__ terms, int64_t rows, const uint32_t* __restrict__ valid, float* __restrict__ loss, uint32_t* fault) {
  __shared__ double red[256];
  double acc = 0.0;
  for (int64_t i = threadIdx.x; i < rows; i += blockDim.x) acc += (double)terms[i];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) { if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
  if (threadIdx.x == 0) {
    float l = (float)(red[0] / (double)valid[0]);
    if (!isfinite(l)) raise_fault(fault, OP_CE);
    loss[0] = l;
  }
}

}  // namespace

ojc_status ce_count(ojc_backend* be, const uint32_t* targets, int64_t rows, int has_ignore, uint32_t ignore, int64_t vocab, uint32_t* valid_dev) {
  ce_count_kernel<<<1, 1024, 0, be->stream>>>(targets, rows, has_ignore, ignore, vocab, valid_dev, be->fault_dev);
  OJC_LAUNCHED(be, "cross_entropy_mean");
  return OJC_OK;
}

ojc_status ce_rows(ojc_backend* be, const void* logits, int32_t l_dt, int64_t ld, const uint32_t* targets, int64_t rows, int64_t vocab, int has_ignore,
                   uint32_t ignore, const uint32_t* valid_dev, float* terms, void* grad, int32_t g_dt, int64_t ldg, float seed) {
  const char* op = "cross_entropy_mean";
  if (rows == 0) return OJC_OK;
  if (l_dt == OJC_F32 && grad && g_dt == OJC_BF16 && ld % 4 == 0 && ldg % 4 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(grad) & 7) == 0) {
    ce_rows_fast_kernel<<<(unsigned)rows, 512, 0, be->stream>>>((const float*)logits, ld, targets, vocab, has_ignore, ignore, valid_dev, terms, (bf16*)grad, ldg, seed,
                                                                be->fault_dev);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }
  return dispatch_float(op, l_dt, [&](auto tl) { return dispatch_float(op, grad ? g_dt : OJC_F32, [&](auto tg) {
    using TL = decltype(tl); using TG = decltype(tg);
    ce_rows_kernel<TL, TG><<<(unsigned)rows, 256, 0, be->stream>>>((const TL*)logits, ld, targets, vocab, has_ignore, ignore, valid_dev, terms, (TG*)grad, ldg, seed, be->fault_dev);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }); });
}

ojc_status ce_loss_finish(ojc_backend* be, const float* terms, int64_t rows, const uint32_t* valid_dev, float* loss_dev) {
  ce_loss_finish_kernel<<<1, 256, 0, be->stream>>>(terms, rows, valid_dev, loss_dev, be->fault_dev);
  OJC_LAUNCHED(be, "cross_entropy_mean");
  return OJC_OK;
}

// The fused tied-head loss. x [rows, dim] and w [vocab, dim] share a dtype class (both F32: f32 tier with F32 logits
// and F32 G; both BF16: tensor-core GEMMs, BF16 logits turned into BF16 G in place). gx (same dtype as x, or F32) and gw (F32) are optional;
// gw_accumulate adds into gw (the tied embedding's gradient buffer). `seed` scales G, i.e. both gradients.
ojc_status linear_ce_impl(ojc_backend* be, const void* x, int32_t x_dt, const void* w, int32_t w_dt, const uint32_t* targets, int64_t rows, int64_t dim,
                          int64_t vocab, int has_ignore, uint32_t ignore, int64_t chunk_rows, float* loss_dev, void* gx, int32_t gx_dt, float* gw,
                          bool gw_accumulate, float seed) {
  const char* op = "linear_cross_entropy_mean";
  const bool bf = x_dt == OJC_BF16 && w_dt == OJC_BF16;
  const int32_t g_dt = bf ? OJC_BF16 : OJC_F32;
  if (chunk_rows <= 0) chunk_rows = bf ? 8192 : 1024;   // bf16 tier: 8192-row tiles measured 1% of the 124M step faster than 4096 (half the accumulating dW passes), 16384 no better
  if (chunk_rows > rows) chunk_rows = rows;
  const bool want = gx || gw;
  const int64_t ldl = (vocab + 7) & ~int64_t(7);  // keep tile rows 16-byte aligned for the tensor-core kernels
  // bf16 tier: one BF16 tile holds the logits and then, in place, their gradient; f32 tier: an F32 logits tile and an F32 gradient tile
  void *logits = nullptr, *gbuf = nullptr, *small = nullptr;
  OJC_TRY(ojc_alloc(be, (uint64_t)chunk_rows * ldl * (bf ? 2 : 4), &logits));
  ojc_status st = OJC_OK;
  if (want && !bf) st = ojc_alloc(be, (uint64_t)chunk_rows * ldl * 4, &gbuf);
  if (st == OJC_OK) st = ojc_alloc(be, (uint64_t)rows * 4 + 256, &small);
  auto run = [&]() -> ojc_status {
    uint32_t* valid = (uint32_t*)small;
    float* terms = (float*)((char*)small + 256);
    OJC_TRY(ce_count(be, targets, rows, has_ignore, ignore, vocab, valid));
    for (int64_t r0 = 0; r0 < rows; r0 += chunk_rows) {
      const int64_t r = std::min(chunk_rows, rows - r0);
      const char* xc = (const char*)x + r0 * dim * dtype_size(x_dt);
      GemmOperand a{xc, x_dt, dim, 1}, b{w, w_dt, 1, dim};
      OJC_TRY(gemm_auto(be, op, a, b, logits, bf ? OJC_BF16 : OJC_F32, ldl, r, vocab, dim, 1.0f, false, nullptr));
      void* g = gbuf;
      if (bf) {
        // a row that fits twice in an SM's shared memory is worked on there; wider ones stay in L2
        const size_t row_bytes = (size_t)((vocab * 2 + 15) / 16 * 16);
        if (row_bytes <= CE_ROW_SMEM_MAX && g_ce_rows_variant == 0 && vocab % 8 == 0 && r >= 2 * be->sm_count) {
          static PerDeviceFlag attr2_of;
          bool& attr2 = attr2_of[be->device];
          const size_t stride = (row_bytes + 127) / 128 * 128;
          if (!attr2) { OJC_CUDA(be, cudaFuncSetAttribute(ce_rows_stream_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * CE_ROW_SMEM_MAX)), op); attr2 = true; }
          ce_rows_stream_bf16_kernel<<<(unsigned)be->sm_count, CE_STREAM_THREADS, 2 * stride, be->stream>>>((bf16*)logits, ldl, targets + r0, r, vocab, has_ignore, ignore, valid,
                                                                                                     terms + r0, want ? 1 : 0, seed, be->fault_dev);
        } else if (row_bytes <= CE_ROW_SMEM_MAX && g_ce_rows_variant != 1) {
          static PerDeviceFlag attr_of;
          bool& attr = attr_of[be->device];
          if (!attr) { OJC_CUDA(be, cudaFuncSetAttribute(ce_rows_smem_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CE_ROW_SMEM_MAX), op); attr = true; }
          ce_rows_smem_bf16_kernel<<<(unsigned)r, 512, row_bytes, be->stream>>>((bf16*)logits, ldl, targets + r0, vocab, has_ignore, ignore, valid, terms + r0, want ? 1 : 0,
                                                                               seed, be->fault_dev);
        } else {
          ce_rows_inplace_bf16_kernel<<<(unsigned)r, 512, 0, be->stream>>>((bf16*)logits, ldl, targets + r0, vocab, has_ignore, ignore, valid, terms + r0, want ? 1 : 0, seed,
                                                                          be->fault_dev);
        }
        OJC_LAUNCHED(be, op);
        g = logits;
      } else {
        OJC_TRY(ce_rows(be, logits, OJC_F32, ldl, targets + r0, r, vocab, has_ignore, ignore, valid, terms + r0, want ? gbuf : nullptr, g_dt, ldl, seed));
      }
      if (gx) {  // dX_c = G . W
        GemmOperand ga{g, g_dt, ldl, 1}, wb{w, w_dt, dim, 1};
        OJC_TRY(gemm_auto(be, op, ga, wb, (char*)gx + r0 * dim * dtype_size(gx_dt), gx_dt, dim, r, dim, vocab, 1.0f, false, nullptr));
      }
      if (gw) {  // dW += G^T . x_c (rows ascending across tiles)
        GemmOperand gt{g, g_dt, 1, ldl}, xb{xc, x_dt, dim, 1};
        OJC_TRY(gemm_auto(be, op, gt, xb, gw, OJC_F32, dim, vocab, dim, r, 1.0f, gw_accumulate || r0 > 0, nullptr));
      }
    }
    return ce_loss_finish(be, terms, rows, valid, loss_dev);
  };
  if (st == OJC_OK) st = run();
  if (logits) ojc_free(be, logits);
  if (gbuf) ojc_free(be, gbuf);
  if (small) ojc_free(be, small);
  return st;
}

extern "C" {

ojc_status ojc_ce_rows_variant(int32_t variant) { g_ce_rows_variant = variant == 1 || variant == 2 ? variant : 0; return OJC_OK; }

static ojc_status ce_args(const char* op, const ojc_tensor* logits, const ojc_tensor* targets, int64_t* rows, int64_t* vocab) {
  OJC_TRY(check_tensor(op, "logits", logits)); OJC_TRY(check_tensor(op, "targets", targets));
  if (logits->rank != 2 || numel(targets) != logits->shape[0]) return ojc_fail(OJC_ERR_SHAPE, op, "logits [rows, vocab], targets [rows]");
  if (targets->dtype != OJC_U32 || !is_float(logits)) return ojc_fail(OJC_ERR_DTYPE, op, "logits float, targets U32");
  *rows = logits->shape[0]; *vocab = logits->shape[1];
  if (*rows == 0 || *vocab == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  return OJC_OK;
}

ojc_status ojc_cross_entropy_mean_forward(ojc_backend* be, const ojc_tensor* logits, const ojc_tensor* targets, int32_t has_ignore, uint32_t ignore, ojc_tensor* loss) {
  const char* op = "cross_entropy_mean_forward";
  OJC_ALIVE(be, op);
  int64_t rows, vocab;
  OJC_TRY(ce_args(op, logits, targets, &rows, &vocab));
  OJC_TRY(check_tensor(op, "loss", loss));
  if (numel(loss) != 1 || loss->dtype != OJC_F32) return ojc_fail(OJC_ERR_SHAPE, op, "loss must be one F32 value");
  void* small = nullptr;
  OJC_TRY(ojc_alloc(be, (uint64_t)rows * 4 + 256, &small));
  uint32_t* valid = (uint32_t*)small; float* terms = (float*)((char*)small + 256);
  ojc_status st = ce_count(be, (const uint32_t*)targets->data, rows, has_ignore, ignore, vocab, valid);
  if (st == OJC_OK) st = ce_rows(be, logits->data, logits->dtype, vocab, (const uint32_t*)targets->data, rows, vocab, has_ignore, ignore, valid, terms, nullptr, OJC_F32, 0, 1.0f);
  if (st == OJC_OK) st = ce_loss_finish(be, terms, rows, valid, (float*)loss->data);
  ojc_free(be, small);
  return st;
}

ojc_status ojc_cross_entropy_mean_backward(ojc_backend* be, const ojc_tensor* logits, const ojc_tensor* targets, int32_t has_ignore, uint32_t ignore, ojc_tensor* grad) {
  const char* op = "cross_entropy_mean_backward";
  OJC_ALIVE(be, op);
  int64_t rows, vocab;
  OJC_TRY(ce_args(op, logits, targets, &rows, &vocab));
  OJC_TRY(check_tensor(op, "grad_logits", grad));
  if (!same_shape(grad, logits) || !is_float(grad)) return ojc_fail(OJC_ERR_SHAPE, op, "grad_logits must match logits");
  void* small = nullptr;
  OJC_TRY(ojc_alloc(be, (uint64_t)rows * 4 + 256, &small));
  uint32_t* valid = (uint32_t*)small; float* terms = (float*)((char*)small + 256);
  ojc_status st = ce_count(be, (const uint32_t*)targets->data, rows, has_ignore, ignore, vocab, valid);
  if (st == OJC_OK) st = ce_rows(be, logits->data, logits->dtype, vocab, (const uint32_t*)targets->data, rows, vocab, has_ignore, ignore, valid, terms, grad->data, grad->dtype, vocab, 1.0f);
  ojc_free(be, small);
  return st;
}

ojc_status ojc_linear_cross_entropy_mean(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* w, const ojc_tensor* targets, int32_t has_ignore, uint32_t ignore,
                                         int64_t chunk_rows, int64_t chunk_cols, ojc_tensor* loss, ojc_tensor* gx, ojc_tensor* gw) {
  const char* op = "linear_cross_entropy_mean";
  OJC_ALIVE(be, op);
  (void)chunk_cols;  // the vocabulary axis is never tiled here
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "weight", w)); OJC_TRY(check_tensor(op, "targets", targets)); OJC_TRY(check_tensor(op, "loss", loss));
  if (x->rank != 2 || w->rank != 2 || x->shape[1] != w->shape[1] || numel(targets) != x->shape[0]) return ojc_fail(OJC_ERR_SHAPE, op, "x [rows, d], weight [vocab, d], targets [rows]");
  if (targets->dtype != OJC_U32 || !is_float(x) || !is_float(w)) return ojc_fail(OJC_ERR_DTYPE, op, "x and weight float, targets U32");
  if (numel(loss) != 1 || loss->dtype != OJC_F32) return ojc_fail(OJC_ERR_SHAPE, op, "loss must be one F32 value");
  if (numel(x) == 0 || numel(w) == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  if (chunk_rows < 0) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "chunk rows is negative");
  if (gx) { OJC_TRY(check_tensor(op, "grad_input", gx)); if (!same_shape(gx, x) || !is_float(gx)) return ojc_fail(OJC_ERR_SHAPE, op, "grad_input must match x"); }
  if (gw) { OJC_TRY(check_tensor(op, "grad_weight", gw)); if (!same_shape(gw, w) || gw->dtype != OJC_F32) return ojc_fail(OJC_ERR_SHAPE, op, "grad_weight must be F32 like weight"); }
  return linear_ce_impl(be, x->data, x->dtype, w->data, w->dtype, (const uint32_t*)targets->data, x->shape[0], x->shape[1], w->shape[0], has_ignore, ignore,
                        chunk_rows, (float*)loss->data, gx ? gx->data : nullptr, gx ? gx->dtype : OJC_F32, gw ? (float*)gw->data : nullptr, false, 1.0f);
}

}  // extern "C"
