// Causal scaled-dot-product attention, forward (+ row log-sum-exp) and backward.
//
// Blockwise with an online softmax: no T x T matrix is ever stored. Key j is
// visible to query t iff t - W < j <= t; query head h reads KV head h / (H / Hkv)
// (ojas-cpu/src/attn.rs:626-700). q/k/v/out are read through their strides, so a
// [B,T,H,dh] buffer viewed as [B,H,T,dh] needs no permute copy.
//
// This file holds the f32-math tier (any head_dim up to 256, F32 or BF16
// storage): one warp per query row (forward, dQ) or key row (dK/dV), lanes
// across keys / queries, no atomics. The bf16 tensor-core tier is sdpa_tc.cu.
#include "common.cuh"
#include "dispatch.cuh"
#include "sdpa.cuh"

namespace {

constexpr int MAXI = 8;  // head_dim <= 256: each lane owns columns lane + 32 i

template <class T>
__global__ void sdpa_forward_kernel(SdpaView<const T> q, SdpaView<const T> k, SdpaView<const T> v, SdpaView<T> out, float* __restrict__ lse,
                                    int heads, int kv_heads, int time, int dim, int window, float scale, uint32_t* fault) {
  extern __shared__ float sm[];  // [warps][dim] query rows
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t = blockIdx.x * nwarps + warp;
  const int plane = blockIdx.y, b = plane / heads, h = plane % heads;
  const int rep = heads / kv_heads, hk = h / rep;
  if (t >= time) return;
  float* qs = sm + warp * dim;
  const T* qp = q.row(b, h, t);
  for (int d = lane; d < dim; d += 32) qs[d] = ldf(qp, d);
  __syncwarp();
  const int j_first = window < 0 ? 0 : max(0, t + 1 - window);
  float m = -INFINITY, l = 0.0f, o[MAXI];
#pragma unroll
  for (int i = 0; i < MAXI; ++i) o[i] = 0.0f;
  for (int j0 = j_first; j0 <= t; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= t;
    float s = -INFINITY;
    if (valid) {
      const T* kp = k.row(b, hk, j);
      float acc = 0.0f;
      for (int d = 0; d < dim; ++d) acc = fmaf(qs[d], ldf(kp, d), acc);
      s = acc * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.0f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAXI; ++i) o[i] *= corr;
    const int cnt = min(32, t - j0 + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T* vp = v.row(b, hk, j0 + jj);
#pragma unroll
      for (int i = 0; i < MAXI; ++i) { const int d = lane + 32 * i; if (d < dim) o[i] = fmaf(pj, ldf(vp, d), o[i]); }
    }
    m = m_new;
  }
  if (!(isfinite(l) && l > 0.0f && isfinite(m))) { if (lane == 0) raise_fault(fault, OP_SDPA); }
  T* op = out.row(b, h, t);
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < MAXI; ++i) { const int d = lane + 32 * i; if (d < dim) stf(op, d, o[i] * inv); }
  if (lane == 0) lse[((int64_t)b * heads + h) * time + t] = m + logf(l);
}

// dQ and the row statistic Dr = dO . O  (ojas-cpu/src/attn.rs:540-595).
template <class T>
__global__ void sdpa_backward_dq_kernel(SdpaView<const T> q, SdpaView<const T> k, SdpaView<const T> v, SdpaView<const T> out, SdpaView<const T> gout,
                                        const float* __restrict__ lse, SdpaView<T> gq, float* __restrict__ dr_out, int heads, int kv_heads, int time,
                                        int dim, int window, float scale) {
  extern __shared__ float sm[];  // [warps][2 * dim]: q row, dO row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t = blockIdx.x * nwarps + warp;
  const int plane = blockIdx.y, b = plane / heads, h = plane % heads;
  const int rep = heads / kv_heads, hk = h / rep;
  if (t >= time) return;
  float* qs = sm + warp * 2 * dim;
  float* gs = qs + dim;
  const T* qp = q.row(b, h, t);
  const T* gp = gout.row(b, h, t);
  const T* op = out.row(b, h, t);
  float dr = 0.0f;
  for (int d = lane; d < dim; d += 32) { qs[d] = ldf(qp, d); float g = ldf(gp, d); gs[d] = g; dr = fmaf(g, ldf(op, d), dr); }
  dr = warp_sum(dr);
  __syncwarp();
  const int64_t stat = ((int64_t)b * heads + h) * time + t;
  if (lane == 0) dr_out[stat] = dr;
  const float row_lse = lse[stat];
  const int j_first = window < 0 ? 0 : max(0, t + 1 - window);
  float acc[MAXI];
#pragma unroll
  for (int i = 0; i < MAXI; ++i) acc[i] = 0.0f;
  for (int j0 = j_first; j0 <= t; j0 += 32) {
    const int j = j0 + lane;
    float ds = 0.0f;
    if (j <= t) {
      const T* kp = k.row(b, hk, j);
      const T* vp = v.row(b, hk, j);
      float s = 0.0f, dp = 0.0f;
      for (int d = 0; d < dim; ++d) { s = fmaf(qs[d], ldf(kp, d), s); dp = fmaf(gs[d], ldf(vp, d), dp); }
      const float p = expf(s * scale - row_lse);
      ds = scale * (p * (dp - dr));
    }
    const int cnt = min(32, t - j0 + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float c = __shfl_sync(0xffffffffu, ds, jj);
      const T* kp = k.row(b, hk, j0 + jj);
#pragma unroll
      for (int i = 0; i < MAXI; ++i) { const int d = lane + 32 * i; if (d < dim) acc[i] = fmaf(c, ldf(kp, d), acc[i]); }
    }
  }
  T* dst = gq.row(b, h, t);
#pragma unroll
  for (int i = 0; i < MAXI; ++i) { const int d = lane + 32 * i; if (d < dim) stf(dst, d, acc[i]); }
}

// dK and dV: one warp owns key row j of one KV head and walks the queries that see it, query heads of the group
// in increasing order, so no two warps write the same gradient element.
template <class T>
__global__ void sdpa_backward_dkv_kernel(SdpaView<const T> q, SdpaView<const T> k, SdpaView<const T> v, SdpaView<const T> gout,
                                         const float* __restrict__ lse, const float* __restrict__ dr, SdpaView<T> gk, SdpaView<T> gv, int heads,
                                         int kv_heads, int time, int dim, int window, float scale) {
  extern __shared__ float sm[];  // [warps][2 * dim]: k row, v row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int j = blockIdx.x * nwarps + warp;
  const int plane = blockIdx.y, b = plane / kv_heads, hk = plane % kv_heads;
  const int rep = heads / kv_heads;
  if (j >= time) return;
  float* ks = sm + warp * 2 * dim;
  float* vs = ks + dim;
  const T* kp = k.row(b, hk, j);
  const T* vp = v.row(b, hk, j);
  for (int d = lane; d < dim; d += 32) { ks[d] = ldf(kp, d); vs[d] = ldf(vp, d); }
  __syncwarp();
  const int t_last = window < 0 ? time - 1 : min(time - 1, j + window - 1);
  float dk[MAXI], dv[MAXI];
#pragma unroll
  for (int i = 0; i < MAXI; ++i) { dk[i] = 0.0f; dv[i] = 0.0f; }
  for (int r = 0; r < rep; ++r) {
    const int h = hk * rep + r;
    const int64_t stat0 = ((int64_t)b * heads + h) * time;
    for (int t0 = j; t0 <= t_last; t0 += 32) {
      const int t = t0 + lane;
      float p = 0.0f, ds = 0.0f;
      if (t <= t_last) {
        const T* qp = q.row(b, h, t);
        const T* gp = gout.row(b, h, t);
        float s = 0.0f, dp = 0.0f;
        for (int d = 0; d < dim; ++d) { s = fmaf(ldf(qp, d), ks[d], s); dp = fmaf(ldf(gp, d), vs[d], dp); }
        p = expf(s * scale - lse[stat0 + t]);
        ds = scale * (p * (dp - dr[stat0 + t]));
      }
      const int cnt = min(32, t_last - t0 + 1);
      for (int tt = 0; tt < cnt; ++tt) {
        const float pp = __shfl_sync(0xffffffffu, p, tt), cc = __shfl_sync(0xffffffffu, ds, tt);
        const T* qp = q.row(b, h, t0 + tt);
        const T* gp = gout.row(b, h, t0 + tt);
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
          const int d = lane + 32 * i;
          if (d < dim) { dv[i] = fmaf(pp, ldf(gp, d), dv[i]); dk[i] = fmaf(cc, ldf(qp, d), dk[i]); }
        }
      }
    }
  }
  T* dkp = gk.row(b, hk, j);
  T* dvp = gv.row(b, hk, j);
#pragma unroll
  for (int i = 0; i < MAXI; ++i) { const int d = lane + 32 * i; if (d < dim) { stf(dkp, d, dk[i]); stf(dvp, d, dv[i]); } }
}

template <class T, class P> SdpaView<P> view_of(const ojc_tensor* t) { return SdpaView<P>{(P*)t->data, t->stride[0], t->stride[1], t->stride[2]}; }

}  // namespace

ojc_status sdpa_check(const char* op, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, SdpaDims* d) {
  OJC_TRY(check_tensor(op, "q", q, false)); OJC_TRY(check_tensor(op, "k", k, false)); OJC_TRY(check_tensor(op, "v", v, false));
  if (q->rank != 4 || k->rank != 4 || !same_shape(k, v) || q->shape[0] != k->shape[0] || q->shape[2] != k->shape[2] || q->shape[3] != k->shape[3])
    return ojc_fail(OJC_ERR_SHAPE, op, "q [B,H,T,dh]; k, v [B,Hkv,T,dh]");
  d->batch = (int)q->shape[0]; d->heads = (int)q->shape[1]; d->kv_heads = (int)k->shape[1]; d->time = (int)q->shape[2]; d->dim = (int)q->shape[3];
  if (d->batch == 0 || d->heads == 0 || d->time == 0 || d->dim == 0) return ojc_fail(OJC_ERR_SHAPE, op, "empty tensor");
  if (d->kv_heads == 0 || d->heads % d->kv_heads != 0) return ojc_fail(OJC_ERR_SHAPE, op, "n_head must be a multiple of n_kv_head");
  if (d->dim > 32 * MAXI) return ojc_fail(OJC_ERR_UNSUPPORTED_HEAD_DIM, op, "head_dim above 256");
  if (q->stride[3] != 1 || k->stride[3] != 1 || v->stride[3] != 1) return ojc_fail(OJC_ERR_SHAPE, op, "the head_dim axis must be contiguous");
  if (q->dtype != k->dtype || q->dtype != v->dtype || !is_float(q)) return ojc_fail(OJC_ERR_DTYPE, op, "q, k, v must share a float dtype");
  d->scale = 1.0f / sqrtf((float)d->dim);  // sdpa_scale, ojas-core/src/backend.rs:159
  return OJC_OK;
}

ojc_status sdpa_forward_f32tier(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, int64_t window, ojc_tensor* out,
                                float* lse, const SdpaDims& d) {
  const char* op = "causal_sdpa_forward";
  const int warps = 4;
  dim3 grid((d.time + warps - 1) / warps, d.batch * d.heads);
  return dispatch_float(op, q->dtype, [&](auto tq) {
    using T = decltype(tq);
    sdpa_forward_kernel<T><<<grid, warps * 32, warps * d.dim * 4, be->stream>>>(
        view_of<T, const T>(q), view_of<T, const T>(k), view_of<T, const T>(v), view_of<T, T>(out), lse, d.heads, d.kv_heads, d.time, d.dim,
        window < 0 ? -1 : (int)std::min<int64_t>(window, INT32_MAX), d.scale, be->fault_dev);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  });
}

ojc_status sdpa_backward_f32tier(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const float* lse,
                                 const ojc_tensor* gout, int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const SdpaDims& d, float* dr) {
  const char* op = "causal_sdpa_backward";
  const int warps = 4;
  const int w = window < 0 ? -1 : (int)std::min<int64_t>(window, INT32_MAX);
  return dispatch_float(op, q->dtype, [&](auto tq) {
    using T = decltype(tq);
    dim3 grid_q((d.time + warps - 1) / warps, d.batch * d.heads);
    sdpa_backward_dq_kernel<T><<<grid_q, warps * 32, warps * 2 * d.dim * 4, be->stream>>>(
        view_of<T, const T>(q), view_of<T, const T>(k), view_of<T, const T>(v), view_of<T, const T>(out), view_of<T, const T>(gout), lse,
        view_of<T, T>(gq), dr, d.heads, d.kv_heads, d.time, d.dim, w, d.scale);
    OJC_LAUNCHED(be, op);
    dim3 grid_k((d.time + warps - 1) / warps, d.batch * d.kv_heads);
    sdpa_backward_dkv_kernel<T><<<grid_k, warps * 32, warps * 2 * d.dim * 4, be->stream>>>(
        view_of<T, const T>(q), view_of<T, const T>(k), view_of<T, const T>(v), view_of<T, const T>(gout), lse, dr, view_of<T, T>(gk),
        view_of<T, T>(gv), d.heads, d.kv_heads, d.time, d.dim, w, d.scale);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  });
}

// 16-byte row loads: aligned base and strides
static bool strides_ok_for_rows(const ojc_tensor* t) {
  return (reinterpret_cast<uintptr_t>(t->data) & 15) == 0 && t->stride[3] == 1 && t->stride[0] % 8 == 0 && t->stride[1] % 8 == 0 && t->stride[2] % 8 == 0;
}

static ojc_status like(const char* op, const char* what, const ojc_tensor* t, const ojc_tensor* ref) {
  OJC_TRY(check_tensor(op, what, t, false));
  if (!same_shape(t, ref) || t->dtype != ref->dtype || t->stride[3] != 1) return ojc_fail(OJC_ERR_SHAPE, op, std::string(what) + " must match its operand (contiguous head_dim)");
  return OJC_OK;
}

extern "C" {

ojc_status ojc_causal_sdpa_forward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, int64_t window, ojc_tensor* out, ojc_tensor* lse) {
  const char* op = "causal_sdpa_forward";
  OJC_ALIVE(be, op);
  SdpaDims d;
  OJC_TRY(sdpa_check(op, q, k, v, &d));
  if (window == 0) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "window must be at least 1");
  OJC_TRY(like(op, "out", out, q));
  OJC_TRY(check_tensor(op, "lse", lse));
  if (lse->dtype != OJC_F32 || numel(lse) != (int64_t)d.batch * d.heads * d.time) return ojc_fail(OJC_ERR_SHAPE, op, "lse must be F32 [B,H,T]");
  if (sdpa_tcgen05_eligible(be, q, k, v, out, window, d)) return sdpa_forward_tcgen05(be, q, k, v, out, (float*)lse->data, d);
  if (sdpa_tc_eligible(q, k, v, out, d)) return sdpa_forward_tc(be, q, k, v, window, out, (float*)lse->data, d);
  return sdpa_forward_f32tier(be, q, k, v, window, out, (float*)lse->data, d);
}

ojc_status ojc_causal_sdpa_backward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const ojc_tensor* lse,
                                    const ojc_tensor* gout, int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv) {
  const char* op = "causal_sdpa_backward";
  OJC_ALIVE(be, op);
  SdpaDims d;
  OJC_TRY(sdpa_check(op, q, k, v, &d));
  if (window == 0) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "window must be at least 1");
  OJC_TRY(like(op, "out", out, q)); OJC_TRY(like(op, "grad_out", gout, q)); OJC_TRY(like(op, "grad_q", gq, q));
  OJC_TRY(like(op, "grad_k", gk, k)); OJC_TRY(like(op, "grad_v", gv, v));
  OJC_TRY(check_tensor(op, "lse", lse));
  if (lse->dtype != OJC_F32 || numel(lse) != (int64_t)d.batch * d.heads * d.time) return ojc_fail(OJC_ERR_SHAPE, op, "lse must be F32 [B,H,T]");
  void* dr = nullptr;
  OJC_TRY(ojc_scratch(be, (uint64_t)d.batch * d.heads * d.time * 8, &dr));   // Dr, and room for the tcgen05 path's scaled lse
  if (sdpa_tcgen05_bwd_eligible(be, q, k, v, gout, gq, gk, gv, window, d) && out->dtype == OJC_BF16 && strides_ok_for_rows(out) && strides_ok_for_rows(gout))
    return sdpa_backward_tcgen05(be, q, k, v, out, (const float*)lse->data, gout, gq, gk, gv, d, (float*)dr);
  if (sdpa_tc_eligible(q, k, v, out, d)) return sdpa_backward_tc(be, q, k, v, out, (const float*)lse->data, gout, window, gq, gk, gv, d, (float*)dr);
  return sdpa_backward_f32tier(be, q, k, v, out, (const float*)lse->data, gout, window, gq, gk, gv, d, (float*)dr);
}

}  // extern "C"

bool sdpa_backward_takes_dr(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const ojc_tensor* gout,
                            const ojc_tensor* gq, const ojc_tensor* gk, const ojc_tensor* gv, int64_t window) {
  SdpaDims d;
  if (sdpa_check("causal_sdpa_backward", q, k, v, &d) != OJC_OK) return false;
  return sdpa_tcgen05_bwd_eligible(be, q, k, v, gout, gq, gk, gv, window, d) && out->dtype == OJC_BF16 && strides_ok_for_rows(out) && strides_ok_for_rows(gout);
}

ojc_status sdpa_backward_with_dr(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const ojc_tensor* lse,
                                 const ojc_tensor* gout, int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const float* dr, bool* taken) {
  *taken = false;
  if (!sdpa_backward_takes_dr(be, q, k, v, out, gout, gq, gk, gv, window)) return OJC_OK;
  SdpaDims d;
  OJC_TRY(sdpa_check("causal_sdpa_backward", q, k, v, &d));
  if (lse->dtype != OJC_F32 || numel(lse) != (int64_t)d.batch * d.heads * d.time) return ojc_fail(OJC_ERR_SHAPE, "causal_sdpa_backward", "lse must be F32 [B,H,T]");
  *taken = true;
  return sdpa_backward_tcgen05(be, q, k, v, out, (const float*)lse->data, gout, gq, gk, gv, d, nullptr, dr);
}

extern "C" {

// The backward that never trusts a saved (possibly bf16-rounded) output: it reruns the forward for O and lse in
// workspace first, so Dr = dO . O cancels the row sum exactly (ojas-core/src/autocast.rs:1200-1254).
ojc_status ojc_causal_sdpa_backward_recompute(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* gout,
                                              int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv) {
  const char* op = "causal_sdpa_backward_recompute";
  OJC_ALIVE(be, op);
  SdpaDims d;
  OJC_TRY(sdpa_check(op, q, k, v, &d));
  const int64_t n = (int64_t)d.batch * d.heads * d.time;
  void *o_mem = nullptr, *lse_mem = nullptr;
  OJC_TRY(ojc_alloc(be, (uint64_t)n * d.dim * dtype_size(q->dtype), &o_mem));
  ojc_status st = ojc_alloc(be, (uint64_t)n * 4, &lse_mem);
  if (st != OJC_OK) { ojc_free(be, o_mem); return st; }
  ojc_tensor o = *q, l;
  o.data = o_mem;
  o.stride[3] = 1; o.stride[2] = d.dim; o.stride[1] = (int64_t)d.time * d.dim; o.stride[0] = (int64_t)d.heads * d.time * d.dim;
  l.data = lse_mem; l.dtype = OJC_F32; l.rank = 3;
  l.shape[0] = d.batch; l.shape[1] = d.heads; l.shape[2] = d.time;
  l.stride[2] = 1; l.stride[1] = d.time; l.stride[0] = (int64_t)d.heads * d.time;
  st = ojc_causal_sdpa_forward(be, q, k, v, window, &o, &l);
  if (st == OJC_OK) st = ojc_causal_sdpa_backward(be, q, k, v, &o, &l, gout, window, gq, gk, gv);
  ojc_free(be, o_mem); ojc_free(be, lse_mem);
  return st;
}

}  // extern "C"
