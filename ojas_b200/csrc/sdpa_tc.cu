// bf16 tensor-core tier of causal attention: FlashAttention-style forward (O and row log-sum-exp) and a two-kernel
// backward that recomputes P from lse (dK/dV per key tile, dQ per query tile), so no gradient element has two
// writers and nothing is accumulated with atomics. f32 softmax statistics and accumulators, exp2 with the scale
// folded in, causal / sliding-window tile skipping, GQA by kv head = h / (H / Hkv).
//
// Tiles are 64 queries x 64 keys per CTA of four warps (16 rows per warp), operands staged in padded shared memory
// and fed to warp-level bf16 MMAs (m16n8k16). head_dim 64 or 128.
#include "common.cuh"
#include "sdpa.cuh"

namespace {

constexpr int BM = 64, BN = 64, NTHREADS = 128;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

// Copy `rows_valid` rows of D bf16 (16-byte chunks) into a padded tile; rows past the end are zero.
template <int D>
__device__ __forceinline__ void load_tile(bf16 (*dst)[D + 8], const SdpaView<const bf16>& src, int b, int h, int t0, int time) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < 64 * CH; i += NTHREADS) {
    const int r = i / CH, c = i % CH;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (t0 + r < time) val = *reinterpret_cast<const uint4*>(src.row(b, h, t0 + r) + c * 8);
    *reinterpret_cast<uint4*>(&dst[r][c * 8]) = val;
  }
}

// A fragments (16 rows x D) of this warp's rows from a padded tile.
template <int D>
__device__ __forceinline__ void load_a_frags(uint32_t (&f)[D / 16][4], bf16 (*tile)[D + 8], int row0, int lane) {
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) ldsm_x4(smem_addr(&tile[row0 + (lane & 15)][ks * 16 + (lane >> 4) * 8]), f[ks][0], f[ks][1], f[ks][2], f[ks][3]);
}

// acc[8][4] (16 x 64) += A(16 x D) . tile(64 x D)^T : B fragments straight from row-major rows (k = column).
template <int D>
__device__ __forceinline__ void mma_a_tileT(float (&acc)[8][4], const uint32_t (&a)[D / 16][4], bf16 (*tile)[D + 8], int lane) {
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
    for (int jp = 0; jp < 4; ++jp) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(smem_addr(&tile[jp * 16 + (lane >> 4) * 8 + (lane & 7)][ks * 16 + ((lane >> 3) & 1) * 8]), b0, b1, b2, b3);
      mma16816(acc[2 * jp], a[ks], b0, b1);
      mma16816(acc[2 * jp + 1], a[ks], b2, b3);
    }
}

// acc[D/8][4] (16 x D) += P(16 x 64, as A fragments) . tile(64 x D): B fragments through transposing loads (k = row).
template <int D>
__device__ __forceinline__ void mma_p_tile(float (&acc)[D / 8][4], const uint32_t (&p)[4][4], bf16 (*tile)[D + 8], int lane) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(smem_addr(&tile[j * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)][dp * 16 + (lane >> 4) * 8]), b0, b1, b2, b3);
      mma16816(acc[2 * dp], p[j], b0, b1);
      mma16816(acc[2 * dp + 1], p[j], b2, b3);
    }
}

__device__ __forceinline__ bool visible(int key, int query, int window, int time) {
  return key <= query && key < time && query < time && (window < 0 || key > query - window);
}

// ------------------------------------------------------------------------------------------------ forward
template <int D>
__global__ void __launch_bounds__(NTHREADS) sdpa_fwd_tc_kernel(SdpaView<const bf16> q, SdpaView<const bf16> k, SdpaView<const bf16> v, SdpaView<bf16> out,
                                                               float* __restrict__ lse, int heads, int kv_heads, int time, int window, float scale) {
  extern __shared__ __align__(16) uint8_t smem[];
  bf16(*Qs)[D + 8] = reinterpret_cast<bf16(*)[D + 8]>(smem);
  bf16(*Ks)[D + 8] = Qs + BM;
  bf16(*Vs)[D + 8] = Ks + BN;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qt = gridDim.x - 1 - blockIdx.x;  // long (late) query tiles first
  const int q0 = qt * BM;
  const int plane = blockIdx.y, b = plane / heads, h = plane % heads, hk = h / (heads / kv_heads);
  const float sl2 = scale * LOG2E;
  load_tile<D>(Qs, q, b, h, q0, time);
  __syncthreads();
  uint32_t qf[D / 16][4];
  load_a_frags<D>(qf, Qs, warp * 16, lane);
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.0f, 0.0f}, acc_o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { acc_o[i][0] = acc_o[i][1] = acc_o[i][2] = acc_o[i][3] = 0.0f; }
  const int n_end = min(time, q0 + BM);
  const int n_start = window < 0 ? 0 : (max(0, q0 - window + 1) / BN) * BN;
  const int row_a = q0 + warp * 16 + (lane >> 2), row_b = row_a + 8;
  for (int n0 = n_start; n0 < n_end; n0 += BN) {
    __syncthreads();
    load_tile<D>(Ks, k, b, hk, n0, time);
    load_tile<D>(Vs, v, b, hk, n0, time);
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
    mma_a_tileT<D>(s, qf, Ks, lane);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = n0 + nt * 8 + (lane & 3) * 2 + (e & 1), row = (e < 2) ? row_a : row_b;
        const float val = visible(key, row, window, time) ? s[nt][e] * sl2 : -INFINITY;
        s[nt][e] = val;
        mx[e >> 1] = fmaxf(mx[e >> 1], val);
      }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_i[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.0f : m_new;
      corr[r] = exp2f(m_i[r] - m_use[r]);
      m_i[r] = m_new;
      l_i[r] *= corr[r];
    }
    uint32_t pf[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]), p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
      l_i[0] += p0 + p1; l_i[1] += p2 + p3;
      pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { acc_o[i][0] *= corr[0]; acc_o[i][1] *= corr[0]; acc_o[i][2] *= corr[1]; acc_o[i][3] *= corr[1]; }
    mma_p_tile<D>(acc_o, pf, Vs, lane);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
  }
  const float inv_a = 1.0f / l_i[0], inv_b = 1.0f / l_i[1];
  if (row_a < time) {
    bf16* o = out.row(b, h, row_a);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(o + i * 8 + (lane & 3) * 2) = pack_bf16(acc_o[i][0] * inv_a, acc_o[i][1] * inv_a);
    if ((lane & 3) == 0) lse[((int64_t)b * heads + h) * time + row_a] = (m_i[0] + log2f(l_i[0])) * LN2;
  }
  if (row_b < time) {
    bf16* o = out.row(b, h, row_b);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(o + i * 8 + (lane & 3) * 2) = pack_bf16(acc_o[i][2] * inv_b, acc_o[i][3] * inv_b);
    if ((lane & 3) == 0) lse[((int64_t)b * heads + h) * time + row_b] = (m_i[1] + log2f(l_i[1])) * LN2;
  }
}

// Dr[b,h,t] = sum_d dO . O  (one warp per row)
__global__ void sdpa_dr_kernel(SdpaView<const bf16> out, SdpaView<const bf16> gout, float* __restrict__ dr, int heads, int time, int dim) {
  const int lane = threadIdx.x & 31;
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t total = (int64_t)gridDim.y * time;
  (void)total;
  const int plane = blockIdx.y, b = plane / heads, h = plane % heads;
  if (row >= time) return;
  const bf16* o = out.row(b, h, (int)row);
  const bf16* g = gout.row(b, h, (int)row);
  float acc = 0.0f;
  for (int d = lane; d < dim; d += 32) acc = fmaf(__bfloat162float(o[d]), __bfloat162float(g[d]), acc);
  acc = warp_sum(acc);
  if (lane == 0) dr[((int64_t)b * heads + h) * time + row] = acc;
}

// ------------------------------------------------------------------------------------------------ dK, dV
template <int D>
__global__ void __launch_bounds__(NTHREADS) sdpa_bwd_dkv_tc_kernel(SdpaView<const bf16> q, SdpaView<const bf16> k, SdpaView<const bf16> v, SdpaView<const bf16> gout,
                                                                   const float* __restrict__ lse, const float* __restrict__ dr, SdpaView<bf16> gk, SdpaView<bf16> gv,
                                                                   int heads, int kv_heads, int time, int window, float scale) {
  extern __shared__ __align__(16) uint8_t smem[];
  bf16(*Qs)[D + 8] = reinterpret_cast<bf16(*)[D + 8]>(smem);
  bf16(*Gs)[D + 8] = Qs + BM;
  float* lse_s = reinterpret_cast<float*>(Gs + BM);
  float* dr_s = lse_s + BM;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int k0 = blockIdx.x * BN;
  const int plane = blockIdx.y, b = plane / kv_heads, hk = plane % kv_heads, rep = heads / kv_heads;
  const float sl2 = scale * LOG2E;
  // this warp's 16 key rows of K and V as A fragments (staged through the Q / dO tiles)
  load_tile<D>(Qs, k, b, hk, k0, time);
  load_tile<D>(Gs, v, b, hk, k0, time);
  __syncthreads();
  uint32_t kf[D / 16][4], vf[D / 16][4];
  load_a_frags<D>(kf, Qs, warp * 16, lane);
  load_a_frags<D>(vf, Gs, warp * 16, lane);
  float acc_dk[D / 8][4], acc_dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { acc_dk[i][0] = acc_dk[i][1] = acc_dk[i][2] = acc_dk[i][3] = 0.0f; acc_dv[i][0] = acc_dv[i][1] = acc_dv[i][2] = acc_dv[i][3] = 0.0f; }
  const int key_a = k0 + warp * 16 + (lane >> 2), key_b = key_a + 8;
  const int q_end = window < 0 ? time : min(time, k0 + BN - 1 + window);
  for (int r = 0; r < rep; ++r) {
    const int h = hk * rep + r;
    const int64_t stat0 = ((int64_t)b * heads + h) * time;
    for (int q0 = k0; q0 < q_end; q0 += BM) {
      __syncthreads();
      load_tile<D>(Qs, q, b, h, q0, time);
      load_tile<D>(Gs, gout, b, h, q0, time);
      if (threadIdx.x < BM) {
        const int t = q0 + threadIdx.x;
        lse_s[threadIdx.x] = t < time ? lse[stat0 + t] * LOG2E : INFINITY;
        dr_s[threadIdx.x] = t < time ? dr[stat0 + t] : 0.0f;
      }
      __syncthreads();
      float s[8][4], dp[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.0f; }
      mma_a_tileT<D>(s, kf, Qs, lane);    // S^T  = K_w . Q^T
      mma_a_tileT<D>(dp, vf, Gs, lane);   // dP^T = V_w . dO^T
      uint32_t pf[4][4], dsf[4][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float pv[4], dv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qc = nt * 8 + (lane & 3) * 2 + (e & 1), query = q0 + qc, key = (e < 2) ? key_a : key_b;
          const float p = visible(key, query, window, time) ? exp2f(s[nt][e] * sl2 - lse_s[qc]) : 0.0f;
          pv[e] = p;
          dv[e] = p * (dp[nt][e] - dr_s[qc]) * scale;
        }
        pf[nt >> 1][(nt & 1) * 2] = pack_bf16(pv[0], pv[1]);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
        dsf[nt >> 1][(nt & 1) * 2] = pack_bf16(dv[0], dv[1]);
        dsf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(dv[2], dv[3]);
      }
      mma_p_tile<D>(acc_dv, pf, Gs, lane);   // dV_w += P^T . dO
      mma_p_tile<D>(acc_dk, dsf, Qs, lane);  // dK_w += dS^T . Q
    }
  }
  if (key_a < time) {
    bf16* dk = gk.row(b, hk, key_a);
    bf16* dv = gv.row(b, hk, key_a);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      *reinterpret_cast<uint32_t*>(dk + i * 8 + (lane & 3) * 2) = pack_bf16(acc_dk[i][0], acc_dk[i][1]);
      *reinterpret_cast<uint32_t*>(dv + i * 8 + (lane & 3) * 2) = pack_bf16(acc_dv[i][0], acc_dv[i][1]);
    }
  }
  if (key_b < time) {
    bf16* dk = gk.row(b, hk, key_b);
    bf16* dv = gv.row(b, hk, key_b);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      *reinterpret_cast<uint32_t*>(dk + i * 8 + (lane & 3) * 2) = pack_bf16(acc_dk[i][2], acc_dk[i][3]);
      *reinterpret_cast<uint32_t*>(dv + i * 8 + (lane & 3) * 2) = pack_bf16(acc_dv[i][2], acc_dv[i][3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ dQ
template <int D>
__global__ void __launch_bounds__(NTHREADS) sdpa_bwd_dq_tc_kernel(SdpaView<const bf16> q, SdpaView<const bf16> k, SdpaView<const bf16> v, SdpaView<const bf16> gout,
                                                                  const float* __restrict__ lse, const float* __restrict__ dr, SdpaView<bf16> gq, int heads,
                                                                  int kv_heads, int time, int window, float scale) {
  extern __shared__ __align__(16) uint8_t smem[];
  bf16(*Ks)[D + 8] = reinterpret_cast<bf16(*)[D + 8]>(smem);
  bf16(*Vs)[D + 8] = Ks + BN;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * BM;
  const int plane = blockIdx.y, b = plane / heads, h = plane % heads, hk = h / (heads / kv_heads);
  const float sl2 = scale * LOG2E;
  load_tile<D>(Ks, q, b, h, q0, time);
  load_tile<D>(Vs, gout, b, h, q0, time);
  __syncthreads();
  uint32_t qf[D / 16][4], gf[D / 16][4];
  load_a_frags<D>(qf, Ks, warp * 16, lane);
  load_a_frags<D>(gf, Vs, warp * 16, lane);
  const int row_a = q0 + warp * 16 + (lane >> 2), row_b = row_a + 8;
  const int64_t stat0 = ((int64_t)b * heads + h) * time;
  const float lse_a = row_a < time ? lse[stat0 + row_a] * LOG2E : INFINITY, lse_b = row_b < time ? lse[stat0 + row_b] * LOG2E : INFINITY;
  const float dr_a = row_a < time ? dr[stat0 + row_a] : 0.0f, dr_b = row_b < time ? dr[stat0 + row_b] : 0.0f;
  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }
  const int n_end = min(time, q0 + BM);
  const int n_start = window < 0 ? 0 : (max(0, q0 - window + 1) / BN) * BN;
  for (int n0 = n_start; n0 < n_end; n0 += BN) {
    __syncthreads();
    load_tile<D>(Ks, k, b, hk, n0, time);
    load_tile<D>(Vs, v, b, hk, n0, time);
    __syncthreads();
    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.0f; }
    mma_a_tileT<D>(s, qf, Ks, lane);   // S  = Q_w . K^T
    mma_a_tileT<D>(dp, gf, Vs, lane);  // dP = dO_w . V^T
    uint32_t dsf[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      float dv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = n0 + nt * 8 + (lane & 3) * 2 + (e & 1), row = (e < 2) ? row_a : row_b;
        const float p = visible(key, row, window, time) ? exp2f(s[nt][e] * sl2 - ((e < 2) ? lse_a : lse_b)) : 0.0f;
        dv[e] = p * (dp[nt][e] - ((e < 2) ? dr_a : dr_b)) * scale;
      }
      dsf[nt >> 1][(nt & 1) * 2] = pack_bf16(dv[0], dv[1]);
      dsf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(dv[2], dv[3]);
    }
    mma_p_tile<D>(acc, dsf, Ks, lane);  // dQ_w += dS . K
  }
  if (row_a < time) {
    bf16* o = gq.row(b, h, row_a);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(o + i * 8 + (lane & 3) * 2) = pack_bf16(acc[i][0], acc[i][1]);
  }
  if (row_b < time) {
    bf16* o = gq.row(b, h, row_b);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(o + i * 8 + (lane & 3) * 2) = pack_bf16(acc[i][2], acc[i][3]);
  }
}

template <class P> SdpaView<P> view_of(const ojc_tensor* t) { return SdpaView<P>{(P*)t->data, t->stride[0], t->stride[1], t->stride[2]}; }
bool aligned_rows(const ojc_tensor* t) {
  return (reinterpret_cast<uintptr_t>(t->data) & 15) == 0 && t->stride[0] % 8 == 0 && t->stride[1] % 8 == 0 && t->stride[2] % 8 == 0 && t->stride[3] == 1;
}

}  // namespace

bool sdpa_tc_eligible(const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const SdpaDims& d) {
  if (q->dtype != OJC_BF16 || (d.dim != 64 && d.dim != 128)) return false;
  return aligned_rows(q) && aligned_rows(k) && aligned_rows(v) && aligned_rows(out);
}

ojc_status sdpa_forward_tc(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, int64_t window, ojc_tensor* out, float* lse,
                           const SdpaDims& d) {
  const char* op = "causal_sdpa_forward";
  const int w = window < 0 ? -1 : (int)std::min<int64_t>(window, INT32_MAX);
  dim3 grid((d.time + BM - 1) / BM, d.batch * d.heads);
  const size_t smem = (size_t)(BM + 2 * BN) * (d.dim + 8) * 2;
  static PerDeviceFlag attr64_of, attr128_of;
  bool &attr64 = attr64_of[be->device], &attr128 = attr128_of[be->device];
  if (d.dim == 64) {
    if (!attr64) { OJC_CUDA(be, cudaFuncSetAttribute(sdpa_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), op); attr64 = true; }
    sdpa_fwd_tc_kernel<64><<<grid, NTHREADS, smem, be->stream>>>(view_of<const bf16>(q), view_of<const bf16>(k), view_of<const bf16>(v), view_of<bf16>(out), lse,
                                                                 d.heads, d.kv_heads, d.time, w, d.scale);
  } else {
    if (!attr128) { OJC_CUDA(be, cudaFuncSetAttribute(sdpa_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), op); attr128 = true; }
    sdpa_fwd_tc_kernel<128><<<grid, NTHREADS, smem, be->stream>>>(view_of<const bf16>(q), view_of<const bf16>(k), view_of<const bf16>(v), view_of<bf16>(out), lse,
                                                                  d.heads, d.kv_heads, d.time, w, d.scale);
  }
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status sdpa_dr(ojc_backend* be, const ojc_tensor* out, const ojc_tensor* gout, float* dr, const SdpaDims& d) {
  dim3 grid((d.time * 32 + 255) / 256, d.batch * d.heads);
  sdpa_dr_kernel<<<grid, 256, 0, be->stream>>>(view_of<const bf16>(out), view_of<const bf16>(gout), dr, d.heads, d.time, d.dim);
  OJC_LAUNCHED(be, "causal_sdpa_backward");
  return OJC_OK;
}

ojc_status sdpa_backward_tc(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const float* lse,
                            const ojc_tensor* gout, int64_t window, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const SdpaDims& d, float* dr) {
  const char* op = "causal_sdpa_backward";
  if (!aligned_rows(gout) || !aligned_rows(gq) || !aligned_rows(gk) || !aligned_rows(gv))
    return sdpa_backward_f32tier(be, q, k, v, out, lse, gout, window, gq, gk, gv, d, dr);
  const int w = window < 0 ? -1 : (int)std::min<int64_t>(window, INT32_MAX);
  {
    dim3 grid((d.time * 32 + 255) / 256, d.batch * d.heads);
    sdpa_dr_kernel<<<grid, 256, 0, be->stream>>>(view_of<const bf16>(out), view_of<const bf16>(gout), dr, d.heads, d.time, d.dim);
    OJC_LAUNCHED(be, op);
  }
  dim3 grid_k((d.time + BN - 1) / BN, d.batch * d.kv_heads), grid_q((d.time + BM - 1) / BM, d.batch * d.heads);
  const size_t smem_k = (size_t)2 * BM * (d.dim + 8) * 2 + 2 * BM * 4, smem_q = (size_t)2 * BN * (d.dim + 8) * 2;
  static PerDeviceFlag attr_of;
  bool& attr = attr_of[be->device];
  if (!attr) {
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dkv_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)2 * BM * 136 * 2 + 2 * BM * 4)), op);
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dq_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)2 * BN * 136 * 2)), op);
    attr = true;
  }
  if (d.dim == 64) {
    sdpa_bwd_dkv_tc_kernel<64><<<grid_k, NTHREADS, smem_k, be->stream>>>(view_of<const bf16>(q), view_of<const bf16>(k), view_of<const bf16>(v), view_of<const bf16>(gout),
                                                                        lse, dr, view_of<bf16>(gk), view_of<bf16>(gv), d.heads, d.kv_heads, d.time, w, d.scale);
    OJC_LAUNCHED(be, op);
    sdpa_bwd_dq_tc_kernel<64><<<grid_q, NTHREADS, smem_q, be->stream>>>(view_of<const bf16>(q), view_of<const bf16>(k), view_of<const bf16>(v), view_of<const bf16>(gout),
                                                                       lse, dr, view_of<bf16>(gq), d.heads, d.kv_heads, d.time, w, d.scale);
  } else {
    sdpa_bwd_dkv_tc_kernel<128><<<grid_k, NTHREADS, smem_k, be->stream>>>(view_of<const bf16>(q), view_of<const bf16>(k), view_of<const bf16>(v), view_of<const bf16>(gout),
                                                                         lse, dr, view_of<bf16>(gk), view_of<bf16>(gv), d.heads, d.kv_heads, d.time, w, d.scale);
    OJC_LAUNCHED(be, op);
    sdpa_bwd_dq_tc_kernel<128><<<grid_q, NTHREADS, smem_q, be->stream>>>(view_of<const bf16>(q), view_of<const bf16>(k), view_of<const bf16>(v), view_of<const bf16>(gout),
                                                                        lse, dr, view_of<bf16>(gq), d.heads, d.kv_heads, d.time, w, d.scale);
  }
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}
