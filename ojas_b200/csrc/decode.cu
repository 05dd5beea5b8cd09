// Decode-time ops of the same backend (ojas-core/src/backend.rs:1553-1612, 2521-2565): KV-cache ring writes, attention of
// new queries against the cache, and the top-k leaders of logit rows. All three are latency-bound at decode sizes (one to
// a few query positions per sequence) and memory-bound in the cache length; none reshapes its work into a GEMM.
#include "common.cuh"

namespace {

// ======================================================================== kv_cache_write
// src [B, Tn, Hkv, D] -> cache [B, Tcap, Hkv, D]: position at + t goes to slot (at + t) % Tcap. 16-byte moves when a
// (Hkv * D)-float step is a multiple of four floats, scalar otherwise.
template <int VEC>
__global__ void kv_cache_write_kernel(float* __restrict__ cache, const float* __restrict__ src, int64_t batch, int64_t tn, int64_t cap, int64_t step, int64_t at) {
  const int64_t per = step / VEC, total = batch * tn * per;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = i % per, t = (i / per) % tn, b = i / (per * tn);
    const int64_t slot = (at + t) % cap;
    const float* s = src + (b * tn + t) * step + e * VEC;
    float* d = cache + (b * cap + slot) * step + e * VEC;
    if (VEC == 4) *reinterpret_cast<float4*>(d) = *reinterpret_cast<const float4*>(s);
    else *d = *s;
  }
}

// ======================================================================== cached_attention_forward
// One block per (batch, query, head). Phase 1: every thread scores whole keys (dot over D ascending, as the per-row kernel
// of causal_sdpa_forward does) into shared memory and checks the slots it reads for NaN / infinity; phase 2: row maximum
// and sum in a fixed tree; phase 3: thread d mixes value column d over the keys, oldest first. Keys are visited in position
// order lo .. p; position j sits in slot j % Tcap.
__global__ void cached_attention_kernel(const float* __restrict__ q, const float* __restrict__ kc, const float* __restrict__ vc, float* __restrict__ out,
                                        int tq, int heads, int kv_heads, int dh, int64_t cap, int64_t kv_len, int64_t window, float scale, uint32_t* fault) {
  extern __shared__ float sm[];                 // [dh] query, [nkeys] scores, [32] reduction
  const int h = blockIdx.x % heads, i = (blockIdx.x / heads) % tq;
  const int64_t b = blockIdx.x / ((int64_t)heads * tq);
  const int hk = h / (heads / kv_heads);
  const int64_t p = kv_len - tq + i, lo = window > 0 ? max((int64_t)0, p + 1 - window) : 0, nkeys = p + 1 - lo;
  float* qs = sm;
  float* sc = sm + dh;
  float* red = sc + nkeys;
  const float* qrow = q + ((b * tq + i) * heads + h) * dh;
  for (int d = threadIdx.x; d < dh; d += blockDim.x) qs[d] = qrow[d];
  __syncthreads();
  const int64_t step = (int64_t)kv_heads * dh;
  bool bad = false;
  float mx = -INFINITY;
  for (int64_t j = threadIdx.x; j < nkeys; j += blockDim.x) {
    const float* krow = kc + (b * cap + (lo + j) % cap) * step + (int64_t)hk * dh;
    float acc = 0.0f;
    for (int d = 0; d < dh; ++d) { const float kv = krow[d]; bad |= !isfinite(kv); acc += qs[d] * kv; }
    acc *= scale;
    sc[j] = acc;
    mx = fmaxf(mx, acc);
  }
  for (int d = threadIdx.x; d < dh; d += blockDim.x) bad |= !isfinite(qs[d]);
  // block maximum
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < nwarps; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  // probabilities (unnormalised) and their sum: per-thread partials in key order, then a fixed tree
  float sum = 0.0f;
  for (int64_t j = threadIdx.x; j < nkeys; j += blockDim.x) { const float e = expf(sc[j] - mx); sc[j] = e; sum += e; }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = 0.0f;
  for (int w = 0; w < nwarps; ++w) sum += red[w];
  const float inv = 1.0f / sum;
  // value mix: column d of the head, keys oldest first
  for (int d = threadIdx.x; d < dh; d += blockDim.x) {
    float acc = 0.0f;
    for (int64_t j = 0; j < nkeys; ++j) {
      const float vv = vc[(b * cap + (lo + j) % cap) * step + (int64_t)hk * dh + d];
      bad |= !isfinite(vv);
      acc += (sc[j] * inv) * vv;
    }
    out[((b * tq + i) * heads + h) * dh + d] = acc;
  }
  if (bad) raise_fault(fault, OP_CACHED_ATTN);
}

// ======================================================================== topk_rows
// rank_logits (ojas-core/src/backend.rs:186-195): value descending with +0.0 and -0.0 one value and -inf after every
// finite value, then column ascending. The key below is smaller for a better value; (key << 32 | column) ascending is
// the rank order, distinct for distinct columns.
__device__ __forceinline__ uint32_t rank_key(float v) {
  if (v == 0.0f) v = 0.0f;                                       // -0.0 ranks as +0.0
  const uint32_t u = __float_as_uint(v);
  const uint32_t asc = (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // ascending in value for every non-NaN float
  return ~asc;
}

constexpr int TOPK_THREADS = 256, TOPK_MAX = 1024;

// One block per row. Four 8-bit radix passes over the row find the key of the k-th leader and how many columns beat it;
// the columns that beat it, plus the lowest-numbered of those that tie with it, are gathered (ties in column order through
// a block scan), sorted by (key, column) in shared memory, and written with the row's own value bits.
__global__ void __launch_bounds__(TOPK_THREADS)
topk_rows_kernel(const float* __restrict__ x, float* __restrict__ values, uint32_t* __restrict__ ids, int64_t cols, int k, uint32_t* fault) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need, s_scan[TOPK_THREADS / 32 + 1], s_less, s_ties;
  __shared__ unsigned long long cand[TOPK_MAX];
  const float* row = x + (int64_t)blockIdx.x * cols;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  bool bad = false;
  // radix select: after the pass over digit `pass`, s_prefix holds the leading digits of the k-th key and s_need how many
  // columns with exactly that prefix are still to be taken
  if (tid == 0) { s_prefix = 0; s_need = (uint32_t)k; }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = pass == 0 ? 0u : 0xffffffffu << (shift + 8);
    for (int64_t c = tid; c < cols; c += TOPK_THREADS) {
      const float v = row[c];
      if (pass == 0) bad |= (v != v) || v == INFINITY;
      const uint32_t key = rank_key(v);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t need = s_need, d = 0;
      while (hist[d] < need) { need -= hist[d]; ++d; }           // the counts sum to at least `need`
      s_prefix = prefix | (d << shift);
      s_need = need;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix, quota = s_need;                  // take `quota` of the columns whose key equals kth
  if (tid == 0) { s_less = 0; s_ties = 0; }
  __syncthreads();
  // gather: columns in order, so that tied columns are taken lowest first
  for (int64_t c0 = 0; c0 < cols; c0 += TOPK_THREADS) {
    const int64_t c = c0 + tid;
    uint32_t key = 0xffffffffu;
    bool live = c < cols;
    if (live) key = rank_key(row[c]);
    const bool less = live && key < kth, tie = live && key == kth;
    const uint32_t bl = __ballot_sync(0xffffffffu, less), bt = __ballot_sync(0xffffffffu, tie);
    if (lane == 0) s_scan[warp] = (uint32_t)__popc(bl) | ((uint32_t)__popc(bt) << 16);
    __syncthreads();
    uint32_t before_l = 0, before_t = 0, all_l = 0, all_t = 0;
    for (int w = 0; w < TOPK_THREADS / 32; ++w) {
      const uint32_t v = s_scan[w];
      if (w < warp) { before_l += v & 0xffffu; before_t += v >> 16; }
      all_l += v & 0xffffu; all_t += v >> 16;
    }
    const uint32_t lower = (1u << lane) - 1u;
    const uint32_t base_l = s_less, base_t = s_ties;
    if (less) cand[base_l + before_l + __popc(bl & lower)] = ((unsigned long long)key << 32) | (uint32_t)c;
    if (tie) {
      const uint32_t pos = base_t + before_t + __popc(bt & lower);
      if (pos < quota) cand[(uint32_t)k - quota + pos] = ((unsigned long long)key << 32) | (uint32_t)c;
    }
    __syncthreads();
    if (tid == 0) { s_less = base_l + all_l; s_ties = base_t + all_t; }
    __syncthreads();
  }
  // bitonic sort of the k candidates (padded with the largest key) by (key, column)
  int n = 1;
  while (n < k) n <<= 1;
  for (int i = k + tid; i < n; i += TOPK_THREADS) cand[i] = ~0ull;
  __syncthreads();
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < n / 2; i += TOPK_THREADS) {
        const int lo = 2 * i - (i & (stride - 1)), hi = lo + stride;
        const bool up = (lo & size) == 0;
        const unsigned long long a = cand[lo], b2 = cand[hi];
        if ((a > b2) == up) { cand[lo] = b2; cand[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = tid; i < k; i += TOPK_THREADS) {
    const uint32_t c = (uint32_t)cand[i];
    ids[(int64_t)blockIdx.x * k + i] = c;
    values[(int64_t)blockIdx.x * k + i] = row[c];
  }
  if (bad) raise_fault(fault, OP_TOPK);
}

}  // namespace

extern "C" {

ojc_status ojc_kv_cache_write(ojc_backend* be, ojc_tensor* cache, const ojc_tensor* src, uint64_t at) {
  const char* op = "kv_cache_write";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "cache", cache)); OJC_TRY(check_tensor(op, "src", src));
  if (cache->dtype != OJC_F32 || src->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "cache and src are F32");
  if (cache->rank != 4 || src->rank != 4) return ojc_fail(OJC_ERR_SHAPE, op, "cache [B, Tcap, Hkv, D], src [B, Tn, Hkv, D]");
  const int64_t batch = cache->shape[0], cap = cache->shape[1], hkv = cache->shape[2], dh = cache->shape[3], tn = src->shape[1];
  if (src->shape[0] != batch || src->shape[2] != hkv || src->shape[3] != dh) return ojc_fail(OJC_ERR_SHAPE, op, "src and cache differ in batch, KV heads or head dim");
  if (batch == 0 || cap == 0 || hkv == 0 || dh == 0 || tn == 0) return ojc_fail(OJC_ERR_SHAPE, op, "every dimension must be non-zero");
  if (at > UINT64_MAX - (uint64_t)tn || at + (uint64_t)tn > (uint64_t)INT64_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "at + Tn overflows");
  if (tn > cap) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "the new positions exceed the cache capacity");
  const int64_t step = hkv * dh;
  const bool vec = step % 4 == 0 && ((uintptr_t)cache->data % 16 == 0) && ((uintptr_t)src->data % 16 == 0);
  const int64_t total = batch * tn * (vec ? step / 4 : step);
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, (int64_t)be->sm_count * 16);
  if (vec) kv_cache_write_kernel<4><<<grid, 256, 0, be->stream>>>((float*)cache->data, (const float*)src->data, batch, tn, cap, step, (int64_t)at);
  else kv_cache_write_kernel<1><<<grid, 256, 0, be->stream>>>((float*)cache->data, (const float*)src->data, batch, tn, cap, step, (int64_t)at);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status ojc_cached_attention_forward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k_cache, const ojc_tensor* v_cache, uint64_t kv_len, int64_t window,
                                        ojc_tensor* out) {
  const char* op = "cached_attention_forward";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "q", q)); OJC_TRY(check_tensor(op, "k_cache", k_cache)); OJC_TRY(check_tensor(op, "v_cache", v_cache)); OJC_TRY(check_tensor(op, "out", out));
  if (q->dtype != OJC_F32 || k_cache->dtype != OJC_F32 || v_cache->dtype != OJC_F32 || out->dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "operands are F32");
  if (q->rank != 4 || k_cache->rank != 4 || !same_shape(k_cache, v_cache) || !same_shape(q, out))
    return ojc_fail(OJC_ERR_SHAPE, op, "q, out [B, Tq, H, D]; k_cache = v_cache [B, Tcap, Hkv, D]");
  const int64_t batch = q->shape[0], tq = q->shape[1], heads = q->shape[2], dh = q->shape[3], cap = k_cache->shape[1], hkv = k_cache->shape[2];
  if (k_cache->shape[0] != batch || k_cache->shape[3] != dh) return ojc_fail(OJC_ERR_SHAPE, op, "the caches differ from q in batch or head dim");
  if (batch == 0 || tq == 0 || heads == 0 || dh == 0 || cap == 0 || hkv == 0) return ojc_fail(OJC_ERR_SHAPE, op, "every dimension must be non-zero");
  if (heads % hkv != 0) return ojc_fail(OJC_ERR_SHAPE, op, "heads must be a multiple of KV heads");
  if (window == 0) return ojc_fail(OJC_ERR_SHAPE, op, "attention window must be at least 1");
  if (kv_len < (uint64_t)tq) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "kv_len is below the new positions");
  if (kv_len > (uint64_t)INT32_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "kv_len exceeds what this kernel indexes");
  // a window that covers every position is no window; the positions read must still be in the ring (shapes.rs:2803-2816)
  const int64_t len = (int64_t)kv_len, w = (window > 0 && window < len) ? window : -1;
  const int64_t span = w > 0 ? std::min(len, tq + w - 1) : len;
  if (span > cap) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "the positions read exceed the cache capacity");
  const int64_t widest = w > 0 ? std::min(len, w) : len;
  const size_t smem = (size_t)(dh + widest + 32) * 4;
  if (smem > 200 * 1024) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "more than ~51,000 visible positions per query are not supported by this kernel");
  static PerDeviceInt attr_of(0);
  int& attr = attr_of[be->device];
  if (smem > 48 * 1024 && smem > (size_t)attr) {
    OJC_CUDA(be, cudaFuncSetAttribute(cached_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), op);
    attr = 200 * 1024;
  }
  const float scale = 1.0f / sqrtf((float)dh);
  cached_attention_kernel<<<(unsigned)(batch * tq * heads), 128, smem, be->stream>>>((const float*)q->data, (const float*)k_cache->data, (const float*)v_cache->data,
                                                                                   (float*)out->data, (int)tq, (int)heads, (int)hkv, (int)dh, cap, len, w, scale, be->fault_dev);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status ojc_topk_rows(ojc_backend* be, const ojc_tensor* x, int64_t k, ojc_tensor* values, ojc_tensor* ids) {
  const char* op = "topk_rows";
  OJC_ALIVE(be, op);
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "values", values)); OJC_TRY(check_tensor(op, "ids", ids));
  if (x->dtype != OJC_F32 || values->dtype != OJC_F32 || ids->dtype != OJC_U32) return ojc_fail(OJC_ERR_DTYPE, op, "x, values F32; ids U32");
  if (x->rank != 2 || values->rank != 2 || ids->rank != 2) return ojc_fail(OJC_ERR_SHAPE, op, "x [rows, cols]; values, ids [rows, k]");
  const int64_t rows = x->shape[0], cols = x->shape[1];
  if (rows == 0 || cols == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  if (k < 1 || k > cols) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "k must be in 1..=cols");
  if (cols > (int64_t)UINT32_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "cols does not fit u32");
  if (values->shape[0] != rows || values->shape[1] != k || ids->shape[0] != rows || ids->shape[1] != k) return ojc_fail(OJC_ERR_SHAPE, op, "values, ids are [rows, k]");
  if (k > TOPK_MAX) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "k above 1024 is not supported on the device");
  topk_rows_kernel<<<(unsigned)rows, TOPK_THREADS, 0, be->stream>>>((const float*)x->data, (float*)values->data, (uint32_t*)ids->data, cols, (int)k, be->fault_dev);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

}  // extern "C"
