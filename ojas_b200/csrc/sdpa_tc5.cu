// Causal attention forward on the Blackwell tensor cores (tcgen05 + TMEM), head_dim 64, bf16 operands.
//
// One CTA owns 128 query rows of one (batch, head) and walks the visible key blocks of 128:
//   warp 4   TMA producer: Q once, then K (two stages) and V tiles, 128-byte swizzle, no multicast
//   warp 5   allocates 256 TMEM columns and issues the MMAs: S = Q K^T (M128 N128 K64, both K-major) into columns
//            [0,128), then PV = P V (M128 N64 K128, P K-major from shared memory, V MN-major) into columns [128,192)
//   warps 0-3  one thread per query row (= TMEM lane): read S, online softmax in the log2 domain, write P as bf16 into
//            the swizzled shared-memory A-operand layout, then add PV into the f32 output row kept in registers
//            (rescaled whenever the running maximum moves), finally normalise, store O and lse.
// Two CTAs fit on an SM (96 KB of shared memory, 256 TMEM columns each), so one CTA's softmax overlaps the other's MMAs.
// Every mbarrier wait is bounded; on expiry the CTA raises the fault word, drains and frees its TMEM.
#include "sdpa.cuh"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BN = 128, D = 64;
constexpr int TILE_BYTES = 128 * D * 2;                       // 16 KB: 128 rows of 128 bytes
constexpr int OFF_Q = 0, OFF_K = TILE_BYTES, OFF_V = 3 * TILE_BYTES, OFF_P = 4 * TILE_BYTES, OFF_BAR = 6 * TILE_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 128 + 1024;
constexpr int NTHREADS = 192, BWD_THREADS = 320;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
enum { B_QFULL = 0, B_KFULL0, B_KFULL1, B_KEMPTY0, B_KEMPTY1, B_VFULL, B_VEMPTY, B_SFULL, B_PREADY, B_PVFULL, B_COUNT };

struct FwdArgs {
  SdpaView<bf16> out;
  float* lse;
  int heads, kv_heads, time;
  int h_first;      // tensor-map dimension order: 1 = (dh, H, T, B), 0 = (dh, T, H, B)
  float scale;
  uint32_t* fault;
};

__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int h_first, int h, int t0, int b) {
  if (h_first) tma_load_4d(dst, map, bar, 0, h, t0, b);
  else tma_load_4d(dst, map, bar, 0, t0, h, b);
}

__global__ void __launch_bounds__(NTHREADS, 2)
sdpa_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const FwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  auto bar = [&](int i) { return base + OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + OFF_BAR + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;   // long (late) query tiles first
  const int q0 = qt * BM;
  const int plane = blockIdx.y, b = plane / args.heads, h = plane % args.heads, hk = h / (args.heads / args.kv_heads);
  const int n_end = min(args.time, q0 + BM);
  const int nblocks = (n_end + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int i = 0; i < B_COUNT; ++i) mbar_init(bar(i), i == B_PREADY ? 128 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar(B_QFULL), TILE_BYTES);
      load_tile(base + OFF_Q, &tm_q, bar(B_QFULL), args.h_first, h, q0, b);
      for (int j = 0; j < nblocks && !*abort_flag; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(B_KEMPTY0 + s), ((j >> 1) & 1) ^ 1, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(B_KFULL0 + s), TILE_BYTES);
        load_tile(base + OFF_K + s * TILE_BYTES, &tm_k, bar(B_KFULL0 + s), args.h_first, hk, j * BN, b);
        if (!mbar_wait(bar(B_VEMPTY), (j & 1) ^ 1, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(B_VFULL), TILE_BYTES);
        load_tile(base + OFF_V, &tm_v, bar(B_VFULL), args.h_first, hk, j * BN, b);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, 0, 0), idesc_pv = make_idesc(BM, D, 0, 1);
      bool ok = mbar_wait(bar(B_QFULL), 0, args.fault, abort_flag);
      for (int j = 0; j < nblocks && ok && !*abort_flag; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(B_KFULL0 + s), (j >> 1) & 1, args.fault, abort_flag)) break;
        fence_after();
        // S = Q K^T: both operands K-major rows of 128 bytes, 8-row groups 1024 bytes apart, one step = 32 bytes.
        // The S columns are free: every softmax thread arrived on B_PREADY for block j - 1 after its last S read.
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma(tmem_base, make_desc(base + OFF_Q + kk * 32, 0, 1024), make_desc(base + OFF_K + s * TILE_BYTES + kk * 32, 0, 1024), idesc_s, kk > 0);
        umma_commit(bar(B_KEMPTY0 + s));
        umma_commit(bar(B_SFULL));
        if (!mbar_wait(bar(B_PREADY), j & 1, args.fault, abort_flag)) break;
        if (!mbar_wait(bar(B_VFULL), j & 1, args.fault, abort_flag)) break;
        fence_after();
        // PV = P V: P is two K-major halves of 64 keys (16 KB apart); V is MN-major (one 64-wide block), 16 keys = 2048 bytes.
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          umma(tmem_base + 128, make_desc(base + OFF_P + (kk >> 2) * TILE_BYTES + (kk & 3) * 32, 0, 1024), make_desc(base + OFF_V + kk * 2048, 1024, 1024),
               idesc_pv, kk > 0);
        umma_commit(bar(B_VEMPTY));
        umma_commit(bar(B_PVFULL));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output rows (warps 0..3)
    const int tid = threadIdx.x;                  // query row within the tile = TMEM lane
    const int row = q0 + tid;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    float m = -INFINITY, l = 0.0f, o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.0f;
    uint8_t* p_row = base_ptr + OFF_P + tid * 128;
    bool ok = true;
    for (int j = 0; j < nblocks && ok && !*abort_flag; ++j) {
      if (!mbar_wait(bar(B_SFULL), j & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      const int key0 = j * BN;
      const bool diag = key0 + BN > q0;           // only blocks touching the diagonal or the sequence end need masking
      const bool tail = key0 + BN > args.time;
      const bool masked = diag || tail;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + c * 32, r);
        tmem_wait_ld();
        if (!masked) {
#pragma unroll
          for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int key = key0 + c * 32 + e;
            if (key <= row && key < args.time) mx = fmaxf(mx, __uint_as_float(r[e]));
          }
        }
      }
      mx *= sl2;                                   // the scale is positive: max(s) * scale = max(s * scale)
      const float m_new = fmaxf(m, mx);
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float corr = fast_exp2(m - m_use);
      float rowsum = 0.0f;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float p[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            p[e] = fast_exp2(fmaf(__uint_as_float(r[g * 8 + e]), sl2, -m_use));
            if (masked) { const int key = key0 + c * 32 + g * 8 + e; if (!(key <= row && key < args.time)) p[e] = 0.0f; }
            rowsum += p[e];
          }
          const int ci = c * 4 + g;               // 16-byte chunk of this row's 128 keys; the swizzle XORs it with row % 8
          *reinterpret_cast<uint4*>(p_row + (ci >> 3) * TILE_BYTES + (((ci & 7) ^ (tid & 7)) << 4)) =
              make_uint4(pack2_bf16(p[0], p[1]), pack2_bf16(p[2], p[3]), pack2_bf16(p[4], p[5]), pack2_bf16(p[6], p[7]));
        }
      }
      l = l * corr + rowsum;
      m = m_new;
      fence_before();
      fence_async_smem();
      mbar_arrive(bar(B_PREADY));
#pragma unroll
      for (int i = 0; i < D; ++i) o[i] *= corr;   // overlaps the PV MMAs
      if (!mbar_wait(bar(B_PVFULL), j & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + 128 + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] += __uint_as_float(r[e]);
      }
      fence_before();
    }
    if (ok && row < args.time) {
      const float inv = 1.0f / l;
      bf16* dst = args.out.row(b, h, row);
#pragma unroll
      for (int i = 0; i < D; i += 8) {
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack2_bf16(o[i] * inv, o[i + 1] * inv), pack2_bf16(o[i + 2] * inv, o[i + 3] * inv),
                                                        pack2_bf16(o[i + 4] * inv, o[i + 5] * inv), pack2_bf16(o[i + 6] * inv, o[i + 7] * inv));
      }
      args.lse[((int64_t)b * args.heads + h) * args.time + row] = (m + log2f(l)) * LN2;
      if (!(l > 0.0f) || !isfinite(l) || !isfinite(m)) raise_fault(args.fault, OP_SDPA);
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 5) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

// ================================================================================================ backward
// Two kernels, each recomputing P from lse (no atomics, one writer per gradient element):
//   dK/dV: a CTA owns 128 keys and walks the query blocks that see them; S^T = K Q^T and dP^T = V dO^T land in TMEM,
//          the 128 threads (one per key) form P^T and dS^T and write them as swizzled bf16 A operands, and
//          dV += P^T dO, dK += dS^T Q accumulate in TMEM across the whole walk (query heads of a GQA group included).
//   dQ:    a CTA owns 128 queries and walks the key blocks: S = Q K^T, dP = dO V^T, dS -> shared memory, dQ += dS K in TMEM.
struct BwdArgs {
  SdpaView<bf16> g0, g1;          // dK, dV  or  dQ (g1 unused)
  const float* lse;
  const float* dr;
  int heads, kv_heads, time, h_first;
  float scale;
  uint32_t* fault;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void store_chunk(uint8_t* row_ptr, int ci, int tid, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(row_ptr + (ci >> 3) * TILE_BYTES + (((ci & 7) ^ (tid & 7)) << 4)) =
      make_uint4(pack2_bf16(v[0], v[1]), pack2_bf16(v[2], v[3]), pack2_bf16(v[4], v[5]), pack2_bf16(v[6], v[7]));
}
template <int COLS>
__device__ __forceinline__ void store_row_bf16(bf16* dst, uint32_t taddr) {
#pragma unroll
  for (int c = 0; c < COLS / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_wait_ld();
    if (dst) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        *reinterpret_cast<uint4*>(dst + c * 32 + i) =
            make_uint4(pack2_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), pack2_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                       pack2_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])), pack2_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
      }
    }
  }
}

// ---- dK, dV
constexpr int KV_OFF_K = 0, KV_OFF_V = TILE_BYTES, KV_OFF_Q = 2 * TILE_BYTES, KV_OFF_G = 4 * TILE_BYTES, KV_OFF_P = 6 * TILE_BYTES, KV_OFF_DS = 8 * TILE_BYTES,
              KV_OFF_STAT = 10 * TILE_BYTES, KV_OFF_BAR = KV_OFF_STAT + 2 * 2 * 128 * 4;
constexpr int KV_SMEM_BYTES = KV_OFF_BAR + 128 + 1024;
enum { KB_KVFULL = 0, KB_QDFULL0, KB_QDFULL1, KB_QDEMPTY0, KB_QDEMPTY1, KB_SFULL, KB_PREADY, KB_DONE, KB_COUNT };

__global__ void __launch_bounds__(BWD_THREADS, 1)
sdpa_bwd_dkv_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                            const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  auto bar = [&](int i) { return base + KV_OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + KV_OFF_BAR + 8 * KB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat = reinterpret_cast<float*>(base_ptr + KV_OFF_STAT);   // [2 buffers][lse 128 | dr 128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * BN;
  const int plane = blockIdx.y, b = plane / args.kv_heads, hk = plane % args.kv_heads, rep = args.heads / args.kv_heads;
  const int q_blocks = (args.time - k0 + BM - 1) / BM;      // query blocks k0, k0 + 128, ... (k0 is a multiple of 128)
  const int iters = rep * q_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < KB_COUNT; ++i) mbar_init(bar(i), i == KB_PREADY ? 256 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(bar(KB_KVFULL), 2 * TILE_BYTES);
      load_tile(base + KV_OFF_K, &tm_k, bar(KB_KVFULL), args.h_first, hk, k0, b);
      load_tile(base + KV_OFF_V, &tm_v, bar(KB_KVFULL), args.h_first, hk, k0, b);
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        const int s = it & 1, h = hk * rep + it / q_blocks, q0 = k0 + (it % q_blocks) * BM;
        if (!mbar_wait(bar(KB_QDEMPTY0 + s), ((it >> 1) & 1) ^ 1, args.fault, abort_flag)) break;
        // the block's row statistics ride on the same barrier (time is a multiple of 4, so the copies are whole 16-byte units)
        const uint32_t stat_bytes = (uint32_t)min(BM, args.time - q0) * 4u;
        const int64_t idx = ((int64_t)b * args.heads + h) * args.time + q0;
        mbar_expect_tx(bar(KB_QDFULL0 + s), 2 * TILE_BYTES + 2 * stat_bytes);
        load_tile(base + KV_OFF_Q + s * TILE_BYTES, &tm_q, bar(KB_QDFULL0 + s), args.h_first, h, q0, b);
        load_tile(base + KV_OFF_G + s * TILE_BYTES, &tm_g, bar(KB_QDFULL0 + s), args.h_first, h, q0, b);
        bulk_load(base + KV_OFF_STAT + s * 1024, args.lse + idx, stat_bytes, bar(KB_QDFULL0 + s));
        bulk_load(base + KV_OFF_STAT + s * 1024 + 512, args.dr + idx, stat_bytes, bar(KB_QDFULL0 + s));
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BN, BM, 0, 0), idesc_o = make_idesc(BN, D, 0, 1);
      bool ok = mbar_wait(bar(KB_KVFULL), 0, args.fault, abort_flag);
      for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
        const int s = it & 1;
        if (!mbar_wait(bar(KB_QDFULL0 + s), (it >> 1) & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        const uint32_t qs = base + KV_OFF_Q + s * TILE_BYTES, gs = base + KV_OFF_G + s * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)   // S^T = K Q^T
          umma(tmem_base, make_desc(base + KV_OFF_K + kk * 32, 0, 1024), make_desc(qs + kk * 32, 0, 1024), idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)   // dP^T = V dO^T
          umma(tmem_base + 128, make_desc(base + KV_OFF_V + kk * 32, 0, 1024), make_desc(gs + kk * 32, 0, 1024), idesc_s, kk > 0);
        umma_commit(bar(KB_SFULL));
        if (!mbar_wait(bar(KB_PREADY), it & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk)  // dV += P^T dO   (dO as the MN-major B operand)
          umma(tmem_base + 256, make_desc(base + KV_OFF_P + (kk >> 2) * TILE_BYTES + (kk & 3) * 32, 0, 1024), make_desc(gs + kk * 2048, 1024, 1024), idesc_o,
               (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk)  // dK += dS^T Q
          umma(tmem_base + 320, make_desc(base + KV_OFF_DS + (kk >> 2) * TILE_BYTES + (kk & 3) * 32, 0, 1024), make_desc(qs + kk * 2048, 1024, 1024), idesc_o,
               (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(KB_QDEMPTY0 + s));
      }
      if (ok) umma_commit(bar(KB_DONE));
    }
  } else {
    // two warpgroups share the 128 TMEM lanes (a warp reaches lanes 32 * (warp % 4) ..): group 0 takes query columns [0,64), group 1 [64,128)
    const int tid = threadIdx.x & 127, half = warp >> 2, key = k0 + tid;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    uint8_t* p_row = base_ptr + KV_OFF_P + tid * 128;
    uint8_t* ds_row = base_ptr + KV_OFF_DS + tid * 128;
    bool ok = true;
    for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
      const int q0 = k0 + (it % q_blocks) * BM;
      const float* st = stat + (it & 1) * 256;   // lse[128] | dr[128] of this query block, landed with the Q / dO tiles
      if (!mbar_wait(bar(KB_SFULL), it & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      const bool masked = q0 == k0 || q0 + BM > args.time || k0 + BN > args.time;   // diagonal block or a ragged end
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(lane_base + c * 32, rs);
        tmem_ld32(lane_base + 128 + c * 32, rp);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float pv[8], dv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int qc = c * 32 + g * 8 + e;
            float p = fast_exp2(fmaf(__uint_as_float(rs[g * 8 + e]), sl2, -st[qc] * LOG2E));
            if (masked && !(key < args.time && q0 + qc < args.time && key <= q0 + qc)) p = 0.0f;
            pv[e] = p;
            dv[e] = p * (__uint_as_float(rp[g * 8 + e]) - st[128 + qc]) * args.scale;
          }
          store_chunk(p_row, c * 4 + g, tid, pv);
          store_chunk(ds_row, c * 4 + g, tid, dv);
        }
      }
      fence_before();
      fence_async_smem();
      mbar_arrive(bar(KB_PREADY));
    }
    if (ok && mbar_wait(bar(KB_DONE), 0, args.fault, abort_flag)) {
      fence_after();
      if (half == 0) store_row_bf16<D>(key < args.time ? args.g1.row(b, hk, key) : nullptr, lane_base + 256);   // dV
      else store_row_bf16<D>(key < args.time ? args.g0.row(b, hk, key) : nullptr, lane_base + 320);             // dK
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- dQ
constexpr int DQ_OFF_Q = 0, DQ_OFF_G = TILE_BYTES, DQ_OFF_K = 2 * TILE_BYTES, DQ_OFF_V = 4 * TILE_BYTES, DQ_OFF_DS = 6 * TILE_BYTES, DQ_OFF_BAR = 8 * TILE_BYTES;
constexpr int DQ_SMEM_BYTES = DQ_OFF_BAR + 128 + 1024;
enum { QB_QDFULL = 0, QB_KVFULL0, QB_KVFULL1, QB_KVEMPTY0, QB_KVEMPTY1, QB_SFULL, QB_PREADY, QB_DONE, QB_COUNT };

__global__ void __launch_bounds__(BWD_THREADS, 1)
sdpa_bwd_dq_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                           const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  auto bar = [&](int i) { return base + DQ_OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + DQ_OFF_BAR + 8 * QB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * BM;
  const int plane = blockIdx.y, b = plane / args.heads, h = plane % args.heads, hk = h / (args.heads / args.kv_heads);
  const int n_end = min(args.time, q0 + BM);
  const int nblocks = (n_end + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int i = 0; i < QB_COUNT; ++i) mbar_init(bar(i), i == QB_PREADY ? 256 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(bar(QB_QDFULL), 2 * TILE_BYTES);
      load_tile(base + DQ_OFF_Q, &tm_q, bar(QB_QDFULL), args.h_first, h, q0, b);
      load_tile(base + DQ_OFF_G, &tm_g, bar(QB_QDFULL), args.h_first, h, q0, b);
      for (int j = 0; j < nblocks && !*abort_flag; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(QB_KVEMPTY0 + s), ((j >> 1) & 1) ^ 1, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(QB_KVFULL0 + s), 2 * TILE_BYTES);
        load_tile(base + DQ_OFF_K + s * TILE_BYTES, &tm_k, bar(QB_KVFULL0 + s), args.h_first, hk, j * BN, b);
        load_tile(base + DQ_OFF_V + s * TILE_BYTES, &tm_v, bar(QB_KVFULL0 + s), args.h_first, hk, j * BN, b);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, 0, 0), idesc_o = make_idesc(BM, D, 0, 1);
      bool ok = mbar_wait(bar(QB_QDFULL), 0, args.fault, abort_flag);
      for (int j = 0; j < nblocks && ok && !*abort_flag; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(QB_KVFULL0 + s), (j >> 1) & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        const uint32_t ks = base + DQ_OFF_K + s * TILE_BYTES, vs = base + DQ_OFF_V + s * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)   // S = Q K^T
          umma(tmem_base, make_desc(base + DQ_OFF_Q + kk * 32, 0, 1024), make_desc(ks + kk * 32, 0, 1024), idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)   // dP = dO V^T
          umma(tmem_base + 128, make_desc(base + DQ_OFF_G + kk * 32, 0, 1024), make_desc(vs + kk * 32, 0, 1024), idesc_s, kk > 0);
        umma_commit(bar(QB_SFULL));
        if (!mbar_wait(bar(QB_PREADY), j & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)  // dQ += dS K   (K as the MN-major B operand)
          umma(tmem_base + 256, make_desc(base + DQ_OFF_DS + (kk >> 2) * TILE_BYTES + (kk & 3) * 32, 0, 1024), make_desc(ks + kk * 2048, 1024, 1024), idesc_o,
               (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(QB_KVEMPTY0 + s));
      }
      if (ok) umma_commit(bar(QB_DONE));
    }
  } else {
    const int tid = threadIdx.x & 127, half = warp >> 2, row = q0 + tid;   // warpgroup `half` takes key columns [64 * half, 64 * half + 64)
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    const int64_t idx = ((int64_t)b * args.heads + h) * args.time + row;
    const float lse_row = row < args.time ? args.lse[idx] * LOG2E : INFINITY, dr_row = row < args.time ? args.dr[idx] : 0.0f;
    uint8_t* ds_row = base_ptr + DQ_OFF_DS + tid * 128;
    bool ok = true;
    for (int j = 0; j < nblocks && ok && !*abort_flag; ++j) {
      if (!mbar_wait(bar(QB_SFULL), j & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      const int key0 = j * BN;
      const bool diag = key0 + BN > q0, tail = key0 + BN > args.time;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(lane_base + c * 32, rs);
        tmem_ld32(lane_base + 128 + c * 32, rp);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float dv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int key = key0 + c * 32 + g * 8 + e;
            float p = fast_exp2(fmaf(__uint_as_float(rs[g * 8 + e]), sl2, -lse_row));
            if ((diag || tail) && !(key <= row && key < args.time)) p = 0.0f;
            dv[e] = p * (__uint_as_float(rp[g * 8 + e]) - dr_row) * args.scale;
          }
          store_chunk(ds_row, c * 4 + g, tid, dv);
        }
      }
      fence_before();
      fence_async_smem();
      mbar_arrive(bar(QB_PREADY));
    }
    if (ok && mbar_wait(bar(QB_DONE), 0, args.fault, abort_flag)) {
      fence_after();
      store_row_bf16<32>(row < args.time ? args.g0.row(b, h, row) + half * 32 : nullptr, lane_base + 256 + half * 32);
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A [B, H, T, dh] view (any batch / head / time strides, dh contiguous) as a 4-D tensor map whose tiles are 128 time steps of one head.
ojc_status make_map(ojc_backend* be, const char* op, CUtensorMap* map, const ojc_tensor* t, bool h_first) {
  const uint64_t B = t->shape[0], H = t->shape[1], T = t->shape[2], dh = t->shape[3];
  cuuint64_t gdim[4], gstride[3];
  cuuint32_t box[4], estride[4] = {1, 1, 1, 1};
  gdim[0] = dh; box[0] = (cuuint32_t)dh;
  if (h_first) { gdim[1] = H; gstride[0] = t->stride[1] * 2; box[1] = 1; gdim[2] = T; gstride[1] = t->stride[2] * 2; box[2] = 128; }
  else { gdim[1] = T; gstride[0] = t->stride[2] * 2; box[1] = 128; gdim[2] = H; gstride[1] = t->stride[1] * 2; box[2] = 1; }
  gdim[3] = B; gstride[2] = t->stride[0] * 2; box[3] = 1;
  CUresult r = ((EncodeTiledFn)be->tmap_encode)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t->data, gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ojc_fail(OJC_ERR_BACKEND, op, "cuTensorMapEncodeTiled refused an attention operand (code " + std::to_string((int)r) + ")");
  return OJC_OK;
}

bool strides_ok(const ojc_tensor* t) {
  return (reinterpret_cast<uintptr_t>(t->data) & 15) == 0 && t->stride[3] == 1 && t->stride[0] % 8 == 0 && t->stride[1] % 8 == 0 && t->stride[2] % 8 == 0 &&
         t->stride[0] > 0 && t->stride[1] > 0 && t->stride[2] > 0;
}

}  // namespace

bool sdpa_tcgen05_eligible(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, int64_t window, const SdpaDims& d) {
  if (!be->tmap_encode || q->dtype != OJC_BF16 || d.dim != D || window >= 0) return false;
  if (!strides_ok(q) || !strides_ok(k) || !strides_ok(v) || !strides_ok(out)) return false;
  // one dimension order for all three maps: heads inside time, or time inside heads
  const bool hf = q->stride[1] < q->stride[2];
  return (k->stride[1] < k->stride[2]) == hf && (v->stride[1] < v->stride[2]) == hf;
}

ojc_status sdpa_forward_tcgen05(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, ojc_tensor* out, float* lse, const SdpaDims& d) {
  const char* op = "causal_sdpa_forward";
  const bool hf = q->stride[1] < q->stride[2];
  CUtensorMap mq, mk, mv;
  OJC_TRY(make_map(be, op, &mq, q, hf));
  OJC_TRY(make_map(be, op, &mk, k, hf));
  OJC_TRY(make_map(be, op, &mv, v, hf));
  static bool attr = false;
  if (!attr) { OJC_CUDA(be, cudaFuncSetAttribute(sdpa_fwd_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), op); attr = true; }
  FwdArgs args;
  args.out = SdpaView<bf16>{(bf16*)out->data, out->stride[0], out->stride[1], out->stride[2]};
  args.lse = lse; args.heads = d.heads; args.kv_heads = d.kv_heads; args.time = d.time; args.h_first = hf ? 1 : 0; args.scale = d.scale; args.fault = be->fault_dev;
  dim3 grid((d.time + BM - 1) / BM, d.batch * d.heads);
  sdpa_fwd_tcgen05_kernel<<<grid, NTHREADS, SMEM_BYTES, be->stream>>>(mq, mk, mv, args);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

// Dr = rowsum(dO . O) must already be in `dr`. Eligibility is the forward's plus the gradient views.
ojc_status sdpa_backward_tcgen05(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const float* lse, const ojc_tensor* gout,
                                 ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const SdpaDims& d, const float* dr) {
  const char* op = "causal_sdpa_backward";
  const bool hf = q->stride[1] < q->stride[2];
  CUtensorMap mq, mk, mv, mg;
  OJC_TRY(make_map(be, op, &mq, q, hf));
  OJC_TRY(make_map(be, op, &mk, k, hf));
  OJC_TRY(make_map(be, op, &mv, v, hf));
  OJC_TRY(make_map(be, op, &mg, gout, hf));
  static bool attr = false;
  if (!attr) {
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dkv_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM_BYTES), op);
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dq_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM_BYTES), op);
    attr = true;
  }
  BwdArgs a;
  a.lse = lse; a.dr = dr; a.heads = d.heads; a.kv_heads = d.kv_heads; a.time = d.time; a.h_first = hf ? 1 : 0; a.scale = d.scale; a.fault = be->fault_dev;
  a.g0 = SdpaView<bf16>{(bf16*)gk->data, gk->stride[0], gk->stride[1], gk->stride[2]};
  a.g1 = SdpaView<bf16>{(bf16*)gv->data, gv->stride[0], gv->stride[1], gv->stride[2]};
  dim3 grid_k((d.time + BN - 1) / BN, d.batch * d.kv_heads);
  sdpa_bwd_dkv_tcgen05_kernel<<<grid_k, BWD_THREADS, KV_SMEM_BYTES, be->stream>>>(mq, mk, mv, mg, a);
  OJC_LAUNCHED(be, op);
  a.g0 = SdpaView<bf16>{(bf16*)gq->data, gq->stride[0], gq->stride[1], gq->stride[2]};
  dim3 grid_q((d.time + BM - 1) / BM, d.batch * d.heads);
  sdpa_bwd_dq_tcgen05_kernel<<<grid_q, BWD_THREADS, DQ_SMEM_BYTES, be->stream>>>(mq, mk, mv, mg, a);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

bool sdpa_tcgen05_bwd_eligible(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* gout, const ojc_tensor* gq,
                               const ojc_tensor* gk, const ojc_tensor* gv, int64_t window, const SdpaDims& d) {
  if (!sdpa_tcgen05_eligible(be, q, k, v, gout, window, d) || d.time % 4 != 0) return false;
  const bool hf = q->stride[1] < q->stride[2];
  return strides_ok(gq) && strides_ok(gk) && strides_ok(gv) && (gout->stride[1] < gout->stride[2]) == hf;
}
