// Causal attention on the Blackwell tensor cores (tcgen05 + TMEM), head_dim 64 or 128, bf16 operands.
//
// Forward: one CTA owns 128 query rows of one (batch, head) and walks the visible key blocks of 128:
//   warp 4   TMA producer: Q once, then K and V tiles on separate two-stage rings (a K stage is free after its Q K^T, a V
//            stage after its P V), 128-byte swizzle, every CTA fetching its own tiles; the first loads go out before the
//            CTA-wide sync
//   warp 5   allocates 256 TMEM columns and issues the MMAs: S = Q K^T (M128 N128 K64, both K-major) into columns
//            [0,128), then O += P V (M128 N64 K128, P K-major from shared memory, V MN-major) into columns [128,192);
//            S of block j + 1 is issued as soon as the softmax rows hold S of block j in registers
//   warps 0-3  one thread per query row (= TMEM lane): read the S row once and hand the columns back, softmax in the log2
//            domain against a row scale that moves only when the maximum outgrew it by 2^8 (then O is rescaled in place
//            in TMEM), write P as bf16 into the swizzled shared-memory A-operand layout (the one P buffer comes back from
//            the previous P V in two 64-key halves); at the end normalise O from TMEM, store O and lse.
// Blocks are ordered long tiles first inside groups of planes small enough to stay in L2 (tile_order).
// At head_dim 64 two CTAs fit on an SM (112 KB of shared memory, 256 TMEM columns each), so one CTA's softmax overlaps
// the other's MMAs; at head_dim 128 the tiles take 192 KB and one CTA owns the SM. Rows wider than 128 bytes are kept as
// 64-column sub-tiles (one 128-byte swizzle span each), 16 KB apart for 128-row tiles and 8 KB apart for 64-row tiles.
// Every mbarrier wait is bounded; on expiry the CTA raises the fault word, drains and frees its TMEM.
#include <algorithm>

#include "sdpa.cuh"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BN = 128;
constexpr int ST128 = 128 * 128, ST64 = 64 * 128;              // bytes of one 64-column sub-tile of a 128-row / 64-row tile
constexpr int P_BYTES = 128 * BN * 2;                         // 32 KB: P as two 64-key halves
constexpr int NTHREADS = 192, BWD_THREADS = 320;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
constexpr float RESCALE_STEP = 8.0f;                          // log2 units the row maximum may run ahead of the scale in use
constexpr uint32_t HI = desc_hi(1024);                        // every operand here: 8-row groups 1024 bytes apart
constexpr uint32_t KSTEP = 32 >> 4, MNSTEP = 2048 >> 4, ST128_16 = ST128 >> 4, ST64_16 = ST64 >> 4;   // descriptor low-word increments
template <int D> struct Fwd {
  static constexpr int NSUB = D / 64, TILE_BYTES = NSUB * ST128;
  static constexpr int OFF_Q = 0, OFF_K = TILE_BYTES, OFF_V = 3 * TILE_BYTES, OFF_P = 5 * TILE_BYTES, OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;              // D 64: 112 KB (two CTAs per SM); D 128: 192 KB
  static constexpr int CTAS = D == 64 ? 2 : 1;
};
enum { B_QFULL = 0, B_KFULL0, B_KFULL1, B_KEMPTY0, B_KEMPTY1, B_VFULL0, B_VFULL1, B_VEMPTY0, B_VEMPTY1, B_SFULL, B_SFREE, B_PREADY, B_PHALF, B_PVFULL, B_COUNT };

struct FwdArgs {
  SdpaView<bf16> out;
  float* lse;
  int heads, kv_heads, time;
  int planes, group; // batch * heads, and planes per L2 group: the grid is one dimension (tile_order)
  int h_first;      // tensor-map dimension order: 1 = (dh, H, T, B), 0 = (dh, T, H, B)
  float scale;
  uint32_t* fault;
};

// Block order. Planes (batch x head) go in groups small enough for their tensors to stay in L2; inside a group the long
// tiles of all its planes come first, so the blocks that start last are short and the SMs drain together. `rank` counts
// tiles from the longest one.
struct TileOrder { int rank, plane; };
__device__ __forceinline__ TileOrder tile_order(int block, int planes, int group, int tiles) {
  const int g = block / (group * tiles), first = g * group, in_group = min(group, planes - first), within = block - g * group * tiles;
  return TileOrder{within / in_group, first + within % in_group};
}
__host__ inline int planes_per_group(int64_t time, int64_t dim, int planes) {
  const int64_t per_plane = 4 * time * dim * 2;              // q, k, v and one more tensor of the plane, bf16
  return (int)std::max<int64_t>(1, std::min<int64_t>(planes, (32ll << 20) / per_plane));
}

// one `ROWS`-row tile of a head as NSUB 64-column boxes
template <int NSUB, int ROWS>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int h_first, int h, int t0, int b) {
#pragma unroll
  for (int i = 0; i < NSUB; ++i) {
    if (h_first) tma_load_4d(dst + i * ROWS * 128, map, bar, 64 * i, h, t0, b);
    else tma_load_4d(dst + i * ROWS * 128, map, bar, 64 * i, t0, h, b);
  }
}

// The softmax role of one 128-row query tile: thread `tid` owns row q0 + tid (TMEM lane tid). s_addr / o_addr: this thread's
// lane in the S and O accumulators; p_row: its row of the P operand buffer.
template <int D>
__device__ __forceinline__ void softmax_tile(const FwdArgs& args, int b, int h, int q0, int tid, int nblocks, uint32_t s_addr, uint32_t o_addr, uint8_t* p_row,
                                             uint32_t bar_sfull, uint32_t bar_sfree, uint32_t bar_pready, uint32_t bar_phalf, uint32_t bar_pvfull, volatile int* abort_flag) {
  const int row = q0 + tid;
  const float sl2 = args.scale * LOG2E;
  float m = 0.0f, l = 0.0f;                     // m: the maximum the probabilities are scaled by (log2 domain), set by block 0
  bool ok = true;
  for (int j = 0; j < nblocks; ++j) {
    if (!mbar_wait(bar_sfull, j & 1, args.fault, abort_flag)) { ok = false; break; }
    fence_after();
    const int key0 = j * BN;
    const bool masked = key0 + BN > q0 || key0 + BN > args.time;   // only blocks touching the diagonal or the sequence end need masking
    uint32_t r[BN];                                                  // the whole S row of this block: one TMEM pass
#pragma unroll
    for (int c = 0; c < BN / 32; ++c) tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
    tmem_wait_ld();
    // The S columns are free as soon as the row sits in registers: the MMA warp computes the next block's S during this one's softmax.
    fence_before();
    mbar_arrive(bar_sfree);
    if (masked) {
      const int last = min(row, args.time - 1) - key0;              // last visible key of this block, relative
#pragma unroll
      for (int e = 0; e < BN; ++e)
        if (e > last) r[e] = 0xff800000u;                           // -inf: exp2 gives an exact zero
    }
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};    // four chains instead of one 128-deep dependency
#pragma unroll
    for (int e = 0; e < BN; e += 4) {
      mx4[0] = fmaxf(mx4[0], __uint_as_float(r[e])); mx4[1] = fmaxf(mx4[1], __uint_as_float(r[e + 1]));
      mx4[2] = fmaxf(mx4[2], __uint_as_float(r[e + 2])); mx4[3] = fmaxf(mx4[3], __uint_as_float(r[e + 3]));
    }
    float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    mx *= sl2;                                   // the scale is positive: max(s) * scale = max(s * scale)
    // The scale moves only when some row of the warp outgrew it by RESCALE_STEP (the TMEM accesses are warp-wide);
    // block 0 holds key 0, visible to every row, so m is finite from then on.
    const bool grow = j == 0 || mx > m + RESCALE_STEP;
    if (__any_sync(0xffffffffu, grow)) {
      const float m_new = j == 0 ? (mx == -INFINITY ? 0.0f : mx) : fmaxf(m, mx);
      const float corr = j == 0 ? 0.0f : fast_exp2(m - m_new);
      m = m_new;
      l *= corr;
      if (j > 0) {
        // O of blocks 0..j-1 must have landed before it is rescaled in place
        if (!mbar_wait(bar_pvfull, (j - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
          tmem_st32(o_addr + c * 32, o);
        }
        tmem_wait_st();
      }
    }
    float rs4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int ci = 0; ci < BN / 8; ++ci) {
      // P is one buffer: the previous block's P V must have read a 64-key half before this block overwrites it
      if (j > 0 && (ci & 7) == 0) {
        if (!mbar_wait(ci == 0 ? bar_phalf : bar_pvfull, (j - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
      }
      float p[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) { p[e] = fast_exp2(fmaf(__uint_as_float(r[ci * 8 + e]), sl2, -m)); rs4[e & 3] += p[e]; }
      // 16-byte chunk ci of this row's 128 keys; the 128-byte swizzle XORs the chunk index with row % 8
      *reinterpret_cast<uint4*>(p_row + (ci >> 3) * ST128 + (((ci & 7) ^ (tid & 7)) << 4)) =
          make_uint4(pack2_bf16(p[0], p[1]), pack2_bf16(p[2], p[3]), pack2_bf16(p[4], p[5]), pack2_bf16(p[6], p[7]));
    }
    if (!ok) break;
    l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
    fence_before();                              // orders a rescale's TMEM stores before the P V the arrival releases
    fence_async_smem();
    mbar_arrive(bar_pready);
  }
  if (ok && mbar_wait(bar_pvfull, (nblocks - 1) & 1, args.fault, abort_flag)) {
    fence_after();
    const float inv = 1.0f / l;
    bf16* dst = row < args.time ? args.out.row(b, h, row) : nullptr;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(o_addr + c * 32, o);
      tmem_wait_ld();
      if (dst) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(dst + c * 32 + i) =
              make_uint4(pack2_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv), pack2_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                         pack2_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv), pack2_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
      }
    }
    if (dst) {
      args.lse[((int64_t)b * args.heads + h) * args.time + row] = (m + log2f(l)) * LN2;
      if (!(l > 0.0f) || !isfinite(l) || !isfinite(m)) raise_fault(args.fault, OP_SDPA);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(NTHREADS, Fwd<D>::CTAS)
sdpa_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const FwdArgs args) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) { if (threadIdx.x == 0) raise_fault(args.fault, OP_SDPA); return; }   // the swizzled tiles need 1024-byte alignment (whole CTA leaves)
  uint8_t* base_ptr = smem_raw;
  using C = Fwd<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, OFF_Q = C::OFF_Q, OFF_K = C::OFF_K, OFF_V = C::OFF_V, OFF_P = C::OFF_P, OFF_BAR = C::OFF_BAR;
  constexpr uint32_t TILE16 = TILE_BYTES >> 4;
  auto bar = [&](int i) { return base + OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + OFF_BAR + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = gridDim.x / args.planes;
  const TileOrder ord = tile_order(blockIdx.x, args.planes, args.group, tiles);
  const int qt = tiles - 1 - ord.rank;         // late query tiles see the most keys
  const int q0 = qt * BM;
  const int plane = ord.plane, b = plane / args.heads, h = plane % args.heads, hk = h / (args.heads / args.kv_heads);
  const int n_end = min(args.time, q0 + BM);
  const int nblocks = (n_end + BN - 1) / BN;

  // The producer thread sets the barriers up and sends the first loads on their way before the CTA-wide sync, so their
  // latency runs under the TMEM allocation.
  auto load_kv = [&](int j) {
    const int s = j & 1;
    mbar_expect_tx(bar(B_KFULL0 + s), TILE_BYTES);
    load_tile<NSUB, 128>(base + OFF_K + s * TILE_BYTES, &tm_k, bar(B_KFULL0 + s), args.h_first, hk, j * BN, b);
    mbar_expect_tx(bar(B_VFULL0 + s), TILE_BYTES);
    load_tile<NSUB, 128>(base + OFF_V + s * TILE_BYTES, &tm_v, bar(B_VFULL0 + s), args.h_first, hk, j * BN, b);
  };
  if (warp == 4 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
    for (int i = 0; i < B_COUNT; ++i) mbar_init(bar(i), (i == B_PREADY || i == B_SFREE) ? 128 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar(B_QFULL), TILE_BYTES);
    load_tile<NSUB, 128>(base + OFF_Q, &tm_q, bar(B_QFULL), args.h_first, h, q0, b);
    for (int j = 0; j < min(2, nblocks); ++j) load_kv(j);
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // A failed wait has already set the abort flag, which every other wait polls: the loops need no check of their own.
  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer: K and V tiles from block 2 on, two stages each
    if (lane == 0) {
      for (int j = 2; j < nblocks; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        // a K stage is free once the S product that read it finished, a V stage once its P V finished
        if (!mbar_wait(bar(B_KEMPTY0 + s), ph, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(B_KFULL0 + s), TILE_BYTES);
        load_tile<NSUB, 128>(base + OFF_K + s * TILE_BYTES, &tm_k, bar(B_KFULL0 + s), args.h_first, hk, j * BN, b);
        if (!mbar_wait(bar(B_VEMPTY0 + s), ph, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(B_VFULL0 + s), TILE_BYTES);
        load_tile<NSUB, 128>(base + OFF_V + s * TILE_BYTES, &tm_v, bar(B_VFULL0 + s), args.h_first, hk, j * BN, b);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, 0, 0), idesc_pv = make_idesc(BM, D, 0, 1);
      // descriptor low words: K-major operands step 32 bytes per MMA, the MN-major V steps 16 keys = 2048 bytes
      // (V as the MN-major B operand: its 64-wide column blocks are the sub-tiles, ST128 bytes apart)
      const uint32_t q_lo = desc_lo(base + OFF_Q, 0), k_lo = desc_lo(base + OFF_K, 0), p_lo = desc_lo(base + OFF_P, 0), v_lo = desc_lo(base + OFF_V, ST128);
      // S(j) = Q K(j)^T into the one S accumulator; the caller has made sure its columns are free
      auto issue_s = [&](int j) -> bool {
        const uint32_t s = j & 1;
        if (!mbar_wait(bar(B_KFULL0 + s), (j >> 1) & 1, args.fault, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base, q_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, k_lo + s * TILE16 + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(B_SFULL));
        umma_commit(bar(B_KEMPTY0 + s));
        return true;
      };
      bool ok = mbar_wait(bar(B_QFULL), 0, args.fault, abort_flag) && issue_s(0);
      for (int j = 0; j < nblocks && ok; ++j) {
        const uint32_t s = j & 1;
        // S(j + 1) as soon as the softmax rows hold S(j) in registers: it runs under block j's softmax
        if (j + 1 < nblocks) {
          if (!mbar_wait(bar(B_SFREE), j & 1, args.fault, abort_flag)) break;
          fence_after();
          if (!issue_s(j + 1)) break;
        }
        if (!mbar_wait(bar(B_PREADY), j & 1, args.fault, abort_flag)) break;
        if (!mbar_wait(bar(B_VFULL0 + s), (j >> 1) & 1, args.fault, abort_flag)) break;
        fence_after();
        // O += P V: P is two K-major halves of 64 keys (16 KB apart); V is MN-major (one 64-wide block).
        // O stays in TMEM for the whole walk; the softmax rows rescale it in place when their maximum moves.
        // The first half of P is handed back after four of the eight MMAs, so the next block's softmax can start writing.
#pragma unroll
        for (uint32_t kk = 0; kk < BN / 16; ++kk) {
          umma_lh(tmem_base + 128, p_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, v_lo + s * TILE16 + kk * MNSTEP, HI, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          if (kk == BN / 32 - 1) umma_commit(bar(B_PHALF));
        }
        umma_commit(bar(B_VEMPTY0 + s));
        umma_commit(bar(B_PVFULL));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output rows (warps 0..3)
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    softmax_tile<D>(args, b, h, q0, threadIdx.x, nblocks, lane_base, lane_base + 128, base_ptr + OFF_P + threadIdx.x * 128, bar(B_SFULL), bar(B_SFREE), bar(B_PREADY),
                    bar(B_PHALF), bar(B_PVFULL), abort_flag);
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 5) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

// ================================================================================================ forward, two query tiles per CTA
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles and walks the key blocks of 128 once for both:
//   warps 0-3  softmax rows of tile 0, warps 4-7 of tile 1 (one thread per query row; warp w reaches TMEM lanes 32 (w % 4) ..)
//   warp 8     TMA producer: both Q tiles once, then K and V blocks on two-stage rings shared by the two tiles
//   warp 9     allocates all 512 TMEM columns (S0 | S1 | O0 | O1) and issues the MMAs of both tiles in turn
// P never passes through shared memory: a softmax thread packs its row of probabilities to bf16 and stores it with
// tcgen05.st over the first 64 columns of its tile's S accumulator, and O += P V reads P as the A operand from TMEM. The
// MMA warp issues P V of a tile and then that tile's next S (which overwrites the P it has just consumed: the tensor pipe
// runs its instructions in order), so while one tile's rows are in their softmax the pipe works on the other tile.
// Tile 1 sits one key block further down the diagonal than tile 0 and walks one block more.
template <int D> struct Fwd2 {
  static constexpr int NSUB = D / 64, TILE_BYTES = NSUB * ST128;
  static constexpr int OFF_Q = 0, OFF_K = 2 * TILE_BYTES, OFF_V = 4 * TILE_BYTES, OFF_BAR = 6 * TILE_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;                // D 64: 96 KB; D 128: 192 KB
  static constexpr uint32_t COL_S0 = 0, COL_S1 = 128, COL_O0 = 256, COL_O1 = 256 + D;
};
constexpr int FWD2_THREADS = 320;
enum { C_QFULL = 0, C_KFULL0, C_KFULL1, C_KEMPTY0, C_KEMPTY1, C_VFULL0, C_VFULL1, C_VEMPTY0, C_VEMPTY1, C_SFULL0, C_SFULL1, C_PREADY0, C_PREADY1, C_PVFULL0, C_PVFULL1, C_COUNT };

// tcgen05.mma with the A operand in tensor memory (lane = row, two bf16 per 32-bit column, 8 columns per K = 16 step)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %4, 0;\n\tmov.b64 db, {%2, %3};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %5, p;\n\t}"
               ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(hi), "r"(accumulate), "r"(idesc) : "memory");
}

// The softmax role of one query tile (rows q0 .. q0 + 127; thread `t` of the group owns row q0 + t = TMEM lane t).
template <int D>
__device__ __forceinline__ void softmax_tile2(const FwdArgs& args, int b, int h, int q0, int t, int nblocks, uint32_t s_addr, uint32_t o_addr,
                                              uint32_t bar_sfull, uint32_t bar_pready, uint32_t bar_pvfull, volatile int* abort_flag) {
  const int row = q0 + t;
  const float sl2 = args.scale * LOG2E;
  float m = 0.0f, l = 0.0f;
  bool ok = true;
  for (int j = 0; j < nblocks; ++j) {
    if (!mbar_wait(bar_sfull, j & 1, args.fault, abort_flag)) { ok = false; break; }
    fence_after();
    const int key0 = j * BN;
    const bool masked = key0 + BN > q0 || key0 + BN > args.time;
    uint32_t r[BN];
#pragma unroll
    for (int c = 0; c < BN / 32; ++c) tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
    tmem_wait_ld();
    if (masked) {
      const int last = min(row, args.time - 1) - key0;
#pragma unroll
      for (int e = 0; e < BN; ++e)
        if (e > last) r[e] = 0xff800000u;
    }
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < BN; e += 4) {
      mx4[0] = fmaxf(mx4[0], __uint_as_float(r[e])); mx4[1] = fmaxf(mx4[1], __uint_as_float(r[e + 1]));
      mx4[2] = fmaxf(mx4[2], __uint_as_float(r[e + 2])); mx4[3] = fmaxf(mx4[3], __uint_as_float(r[e + 3]));
    }
    float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;
    const bool grow = j == 0 || mx > m + RESCALE_STEP;
    if (__any_sync(0xffffffffu, grow)) {
      const float m_new = j == 0 ? (mx == -INFINITY ? 0.0f : mx) : fmaxf(m, mx);
      const float corr = j == 0 ? 0.0f : fast_exp2(m - m_new);
      m = m_new;
      l *= corr;
      if (j > 0) {
        if (!mbar_wait(bar_pvfull, (j - 1) & 1, args.fault, abort_flag)) { ok = false; break; }   // O of blocks 0..j-1 has landed
        fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
          tmem_st32(o_addr + c * 32, o);
        }
      }
    }
    // P over the first 64 columns of this tile's S (every thread touches its own lane only, and S sits in registers)
    float rs4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t w[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(r[c * 64 + 2 * e]), sl2, -m)), p1 = fast_exp2(fmaf(__uint_as_float(r[c * 64 + 2 * e + 1]), sl2, -m));
        rs4[e & 3] += p0 + p1;
        w[e] = pack2_bf16(p0, p1);
      }
      tmem_st32(s_addr + c * 32, w);
    }
    l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
    tmem_wait_st();
    fence_before();
    mbar_arrive(bar_pready);
  }
  if (ok && nblocks > 0 && mbar_wait(bar_pvfull, (nblocks - 1) & 1, args.fault, abort_flag)) {
    fence_after();
    const float inv = 1.0f / l;
    bf16* dst = row < args.time ? args.out.row(b, h, row) : nullptr;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(o_addr + c * 32, o);
      tmem_wait_ld();
      if (dst) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(dst + c * 32 + i) =
              make_uint4(pack2_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv), pack2_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                         pack2_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv), pack2_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
      }
    }
    if (dst) {
      args.lse[((int64_t)b * args.heads + h) * args.time + row] = (m + log2f(l)) * LN2;
      if (!(l > 0.0f) || !isfinite(l) || !isfinite(m)) raise_fault(args.fault, OP_SDPA);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(FWD2_THREADS, 1)
sdpa_fwd2_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const FwdArgs args) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) { if (threadIdx.x == 0) raise_fault(args.fault, OP_SDPA); return; }
  using C = Fwd2<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES;
  constexpr uint32_t TILE16 = TILE_BYTES >> 4;
  auto bar = [&](int i) { return base + C::OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + C::OFF_BAR + 8 * C_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = gridDim.x / args.planes;                 // 256-row tile pairs per plane
  const TileOrder ord = tile_order(blockIdx.x, args.planes, args.group, tiles);
  const int pt = tiles - 1 - ord.rank;                       // late pairs see the most keys
  const int q0 = pt * 2 * BM;
  const int plane = ord.plane, b = plane / args.heads, h = plane % args.heads, hk = h / (args.heads / args.kv_heads);
  // key blocks each tile walks: up to and including its diagonal block (none for a tile past the end of the sequence)
  const int n0 = (min(args.time, q0 + BM) + BN - 1) / BN;
  const int n1 = q0 + BM < args.time ? (min(args.time, q0 + 2 * BM) + BN - 1) / BN : 0;
  const int nmax = max(n0, n1);

  auto load_kv = [&](int j) {
    const int s = j & 1;
    mbar_expect_tx(bar(C_KFULL0 + s), TILE_BYTES);
    load_tile<NSUB, 128>(base + C::OFF_K + s * TILE_BYTES, &tm_k, bar(C_KFULL0 + s), args.h_first, hk, j * BN, b);
    mbar_expect_tx(bar(C_VFULL0 + s), TILE_BYTES);
    load_tile<NSUB, 128>(base + C::OFF_V + s * TILE_BYTES, &tm_v, bar(C_VFULL0 + s), args.h_first, hk, j * BN, b);
  };
  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
    for (int i = 0; i < C_COUNT; ++i) mbar_init(bar(i), (i == C_PREADY0 || i == C_PREADY1) ? 128 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar(C_QFULL), 2 * TILE_BYTES);
    load_tile<NSUB, 128>(base + C::OFF_Q, &tm_q, bar(C_QFULL), args.h_first, h, q0, b);
    load_tile<NSUB, 128>(base + C::OFF_Q + TILE_BYTES, &tm_q, bar(C_QFULL), args.h_first, h, q0 + BM, b);   // rows past the end read as zeros
    for (int j = 0; j < min(2, nmax); ++j) load_kv(j);
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
      for (int j = 2; j < nmax; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(C_KEMPTY0 + s), ph, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(C_KFULL0 + s), TILE_BYTES);
        load_tile<NSUB, 128>(base + C::OFF_K + s * TILE_BYTES, &tm_k, bar(C_KFULL0 + s), args.h_first, hk, j * BN, b);
        if (!mbar_wait(bar(C_VEMPTY0 + s), ph, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(C_VFULL0 + s), TILE_BYTES);
        load_tile<NSUB, 128>(base + C::OFF_V + s * TILE_BYTES, &tm_v, bar(C_VFULL0 + s), args.h_first, hk, j * BN, b);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, 0, 0), idesc_pv = make_idesc(BM, D, 0, 1);
      const uint32_t q_lo = desc_lo(base + C::OFF_Q, 0), k_lo = desc_lo(base + C::OFF_K, 0), v_lo = desc_lo(base + C::OFF_V, ST128);
      const int nt[2] = {n0, n1};
      const uint32_t col_s[2] = {C::COL_S0, C::COL_S1}, col_o[2] = {C::COL_O0, C::COL_O1};
      // the last tile to read key block j releases its stage: tile 1 whenever it walks that block, tile 0 otherwise
      auto last_user = [&](int g, int j) { return g == 1 ? true : j >= n1; };
      auto issue_s = [&](int g, int j) -> bool {
        const uint32_t s = j & 1;
        if (!mbar_wait(bar(C_KFULL0 + s), (j >> 1) & 1, args.fault, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + col_s[g], q_lo + g * TILE16 + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, k_lo + s * TILE16 + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(C_SFULL0 + g));
        if (last_user(g, j)) umma_commit(bar(C_KEMPTY0 + s));
        return true;
      };
      bool ok = mbar_wait(bar(C_QFULL), 0, args.fault, abort_flag);
      for (int g = 0; g < 2 && ok; ++g) if (nt[g] > 0) ok = issue_s(g, 0);
      for (int j = 0; j < nmax && ok; ++j) {
        const uint32_t s = j & 1;
        for (int g = 0; g < 2 && ok; ++g) {
          if (j >= nt[g]) continue;
          if (!mbar_wait(bar(C_PREADY0 + g), j & 1, args.fault, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar(C_VFULL0 + s), (j >> 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          fence_after();
          // O_g += P_g V: P from tensor memory (8 columns per 16 keys), V MN-major from shared memory
#pragma unroll
          for (uint32_t kk = 0; kk < BN / 16; ++kk)
            umma_ts(tmem_base + col_o[g], tmem_base + col_s[g] + kk * 8, v_lo + s * TILE16 + kk * MNSTEP, HI, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          umma_commit(bar(C_PVFULL0 + g));
          if (last_user(g, j)) umma_commit(bar(C_VEMPTY0 + s));
          // this tile's next S overwrites the P just consumed; the pipe runs the two in issue order
          if (j + 1 < nt[g]) ok = issue_s(g, j + 1);
        }
      }
    }
  } else {
    const int g = warp >> 2, t = threadIdx.x & 127;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    softmax_tile2<D>(args, b, h, q0 + g * BM, t, g == 0 ? n0 : n1, lane_base + (g == 0 ? C::COL_S0 : C::COL_S1), lane_base + (g == 0 ? C::COL_O0 : C::COL_O1),
                     bar(C_SFULL0 + g), bar(C_PREADY0 + g), bar(C_PVFULL0 + g), abort_flag);
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ================================================================================================ forward, persistent CTAs
// The one-tile kernel's roles, kept alive over many query tiles. A CTA takes every gridDim.x-th tile of the long-tiles-first order
// and runs them as one stream of key blocks: the producer keeps loading (the next tile's Q into the second Q buffer, its K and V
// blocks onto the same two-stage rings) while the current tile is still in its last blocks, the MMA thread issues the next tile's first
// S as soon as the softmax rows hold the current tile's last S in registers, and a tile's output rows are normalised and stored while
// the tensor pipe is already on the next tile. TMEM is allocated once, barriers are set up once. P lives in tensor memory beside S
// (S 128 columns, P 64, O D): no shared-memory P buffer, so at head_dim 64 two CTAs share an SM with 96 KB each.
template <int D> struct FwdP {
  static constexpr int NSUB = D / 64, TILE_BYTES = NSUB * ST128;
  static constexpr int OFF_Q = 0, OFF_K = 2 * TILE_BYTES, OFF_V = 4 * TILE_BYTES, OFF_BAR = 6 * TILE_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr uint32_t COL_S = 0, COL_P = 128, COL_O = 192, TMEM_COLS = D == 64 ? 256 : 512;
  static constexpr int CTAS = D == 64 ? 2 : 1;
};
enum { P_QFULL0 = 0, P_QFULL1, P_QEMPTY0, P_QEMPTY1, P_KFULL0, P_KFULL1, P_KEMPTY0, P_KEMPTY1, P_VFULL0, P_VFULL1, P_VEMPTY0, P_VEMPTY1, P_SFULL, P_SFREE, P_PREADY,
       P_PVFULL, P_OFREE, P_COUNT };

// the tile a CTA works on as item `i` of its list, and where it sits
struct TileWalk {
  int q0, b, h, hk, nblocks;
  __device__ __forceinline__ bool set(const FwdArgs& args, int tiles, int total, int item) {
    const int g = blockIdx.x + item * gridDim.x;
    if (g >= total) return false;
    const TileOrder ord = tile_order(g, args.planes, args.group, tiles);
    q0 = (tiles - 1 - ord.rank) * BM;
    b = ord.plane / args.heads; h = ord.plane % args.heads; hk = h / (args.heads / args.kv_heads);
    nblocks = (min(args.time, q0 + BM) + BN - 1) / BN;
    return true;
  }
};

template <int D>
__global__ void __launch_bounds__(NTHREADS, FwdP<D>::CTAS)
sdpa_fwdp_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const FwdArgs args) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) { if (threadIdx.x == 0) raise_fault(args.fault, OP_SDPA); return; }
  using C = FwdP<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES;
  constexpr uint32_t TILE16 = TILE_BYTES >> 4;
  auto bar = [&](int i) { return base + C::OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + C::OFF_BAR + 8 * P_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (args.time + BM - 1) / BM, total = tiles * args.planes;

  if (warp == 4 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
    for (int i = 0; i < P_COUNT; ++i) mbar_init(bar(i), (i == P_PREADY || i == P_SFREE || i == P_OFREE) ? 128 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ producer: Q of tile i into buffer i & 1, K / V of block n into stage n & 1
    if (lane == 0) {
      TileWalk w;
      int n = 0;
      for (int i = 0; w.set(args, tiles, total, i); ++i) {
        const int qs = i & 1;
        if (i >= 2 && !mbar_wait(bar(P_QEMPTY0 + qs), ((i >> 1) & 1) ^ 1, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(P_QFULL0 + qs), TILE_BYTES);
        load_tile<NSUB, 128>(base + C::OFF_Q + qs * TILE_BYTES, &tm_q, bar(P_QFULL0 + qs), args.h_first, w.h, w.q0, w.b);
        bool ok = true;
        for (int j = 0; j < w.nblocks && ok; ++j, ++n) {
          const int s = n & 1;
          const uint32_t ph = ((n >> 1) & 1) ^ 1;
          if (n >= 2 && !mbar_wait(bar(P_KEMPTY0 + s), ph, args.fault, abort_flag)) { ok = false; break; }
          mbar_expect_tx(bar(P_KFULL0 + s), TILE_BYTES);
          load_tile<NSUB, 128>(base + C::OFF_K + s * TILE_BYTES, &tm_k, bar(P_KFULL0 + s), args.h_first, w.hk, j * BN, w.b);
          if (n >= 2 && !mbar_wait(bar(P_VEMPTY0 + s), ph, args.fault, abort_flag)) { ok = false; break; }
          mbar_expect_tx(bar(P_VFULL0 + s), TILE_BYTES);
          load_tile<NSUB, 128>(base + C::OFF_V + s * TILE_BYTES, &tm_v, bar(P_VFULL0 + s), args.h_first, w.hk, j * BN, w.b);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer: S(n + 1) goes out under the softmax of block n, across tile boundaries too
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, BN, 0, 0), idesc_pv = make_idesc(BM, D, 0, 1);
      const uint32_t q_lo = desc_lo(base + C::OFF_Q, 0), k_lo = desc_lo(base + C::OFF_K, 0), v_lo = desc_lo(base + C::OFF_V, ST128);
      // S of block `n` (block j of the tile in Q buffer qs); `last` = the tile's last S: its Q buffer is free afterwards
      auto issue_s = [&](int n, int qs, int qi, int j, bool last) -> bool {
        const uint32_t s = n & 1;
        if (j == 0 && !mbar_wait(bar(P_QFULL0 + qs), (qi >> 1) & 1, args.fault, abort_flag)) return false;
        if (!mbar_wait(bar(P_KFULL0 + s), (n >> 1) & 1, args.fault, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + C::COL_S, q_lo + qs * TILE16 + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, k_lo + s * TILE16 + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(P_SFULL));
        umma_commit(bar(P_KEMPTY0 + s));
        if (last) umma_commit(bar(P_QEMPTY0 + qs));
        return true;
      };
      TileWalk cur, nxt;
      bool have = cur.set(args, tiles, total, 0);
      bool ok = have && issue_s(0, 0, 0, 0, cur.nblocks == 1);
      int n = 0;
      for (int i = 0; have && ok; ++i) {
        const bool more = nxt.set(args, tiles, total, i + 1);
        for (int j = 0; j < cur.nblocks && ok; ++j, ++n) {
          const uint32_t s = n & 1;
          // the next S (of this tile, or block 0 of the next one) as soon as the softmax rows hold S(n) in registers
          const bool within = j + 1 < cur.nblocks;
          if (within || more) {
            if (!mbar_wait(bar(P_SFREE), n & 1, args.fault, abort_flag)) { ok = false; break; }
            fence_after();
            ok = within ? issue_s(n + 1, i & 1, i, j + 1, j + 2 == cur.nblocks) : issue_s(n + 1, (i + 1) & 1, i + 1, 0, nxt.nblocks == 1);
            if (!ok) break;
          }
          if (!mbar_wait(bar(P_PREADY), n & 1, args.fault, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar(P_VFULL0 + s), (n >> 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          // a tile's first P V overwrites O: the previous tile's rows must have read theirs
          if (j == 0 && i > 0 && !mbar_wait(bar(P_OFREE), (i - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          fence_after();
#pragma unroll
          for (uint32_t kk = 0; kk < BN / 16; ++kk)
            umma_ts(tmem_base + C::COL_O, tmem_base + C::COL_P + kk * 8, v_lo + s * TILE16 + kk * MNSTEP, HI, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          umma_commit(bar(P_VEMPTY0 + s));
          umma_commit(bar(P_PVFULL));
        }
        cur = nxt;
        have = more;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output rows (warps 0..3): thread t owns row q0 + t of every tile
    const int t = threadIdx.x;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    const uint32_t s_addr = lane_base + C::COL_S, p_addr = lane_base + C::COL_P, o_addr = lane_base + C::COL_O;
    const float sl2 = args.scale * LOG2E;
    TileWalk w;
    int n = 0;
    bool ok = true;
    for (int i = 0; ok && w.set(args, tiles, total, i); ++i) {
      const int row = w.q0 + t;
      float m = 0.0f, l = 0.0f;
      for (int j = 0; j < w.nblocks; ++j, ++n) {
        if (!mbar_wait(bar(P_SFULL), n & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        const int key0 = j * BN;
        const bool masked = key0 + BN > w.q0 || key0 + BN > args.time;
        uint32_t r[BN];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_wait_ld();
        fence_before();
        mbar_arrive(bar(P_SFREE));               // the S columns are free: the next S runs under this softmax
        if (masked) {
          const int last = min(row, args.time - 1) - key0;
#pragma unroll
          for (int e = 0; e < BN; ++e)
            if (e > last) r[e] = 0xff800000u;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < BN; e += 4) {
          mx4[0] = fmaxf(mx4[0], __uint_as_float(r[e])); mx4[1] = fmaxf(mx4[1], __uint_as_float(r[e + 1]));
          mx4[2] = fmaxf(mx4[2], __uint_as_float(r[e + 2])); mx4[3] = fmaxf(mx4[3], __uint_as_float(r[e + 3]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;
        const bool grow = j == 0 || mx > m + RESCALE_STEP;
        const bool any_grow = __any_sync(0xffffffffu, grow);
        float corr = 1.0f;
        if (any_grow) {
          const float m_new = j == 0 ? (mx == -INFINITY ? 0.0f : mx) : fmaxf(m, mx);
          corr = j == 0 ? 0.0f : fast_exp2(m - m_new);
          m = m_new;
          l *= corr;
        }
        // the probabilities, packed, while the previous P V may still be reading the P columns
        uint32_t pw[BN / 2];
        float rs4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < BN / 2; ++e) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(r[2 * e]), sl2, -m)), p1 = fast_exp2(fmaf(__uint_as_float(r[2 * e + 1]), sl2, -m));
          rs4[e & 3] += p0 + p1;
          pw[e] = pack2_bf16(p0, p1);
        }
        l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
        // P V of the previous block (this tile's or the last of the previous tile) has read P and, for a rescale, has landed in O
        if (n > 0 && !mbar_wait(bar(P_PVFULL), (n - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        if (any_grow && j > 0) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st32(o_addr + c * 32, o);
          }
        }
        tmem_st32(p_addr, *reinterpret_cast<uint32_t(*)[32]>(&pw[0]));
        tmem_st32(p_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pw[32]));
        tmem_wait_st();
        fence_before();
        mbar_arrive(bar(P_PREADY));
      }
      if (!ok) break;
      // this tile's O: read it, hand the columns back, then normalise and store
      if (!mbar_wait(bar(P_PVFULL), (n - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      const float inv = 1.0f / l;
      bf16* dst = row < args.time ? args.out.row(w.b, w.h, row) : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_wait_ld();
        if (c == D / 32 - 1) { fence_before(); mbar_arrive(bar(P_OFREE)); }
        if (dst) {
#pragma unroll
          for (int q = 0; q < 32; q += 8)
            *reinterpret_cast<uint4*>(dst + c * 32 + q) =
                make_uint4(pack2_bf16(__uint_as_float(o[q]) * inv, __uint_as_float(o[q + 1]) * inv), pack2_bf16(__uint_as_float(o[q + 2]) * inv, __uint_as_float(o[q + 3]) * inv),
                           pack2_bf16(__uint_as_float(o[q + 4]) * inv, __uint_as_float(o[q + 5]) * inv), pack2_bf16(__uint_as_float(o[q + 6]) * inv, __uint_as_float(o[q + 7]) * inv));
        }
      }
      if (dst) {
        args.lse[((int64_t)w.b * args.heads + w.h) * args.time + row] = (m + log2f(l)) * LN2;
        if (!(l > 0.0f) || !isfinite(l) || !isfinite(m)) raise_fault(args.fault, OP_SDPA);
      }
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 5) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

// ================================================================================================ backward
// A prepass writes Dr = rowsum(dO . O) and lse * log2(e); then two kernels, each recomputing P from lse (no atomics,
// one writer per gradient element):
//   dK/dV: a CTA owns 128 keys and walks the queries that see them; S^T = K Q^T and dP^T = V dO^T land in TMEM,
//          the threads (one key row each) form P^T and dS^T and write them as swizzled bf16 A operands, and
//          dV += P^T dO, dK += dS^T Q accumulate in TMEM across the whole walk (query heads of a GQA group included).
//   dQ:    a CTA owns 128 queries and walks the keys: S = Q K^T, dP = dO V^T, dS -> shared memory, dQ += dS K in TMEM.
// Both walk in steps of SUB = 64 over three input stages. At head_dim 64 each takes 256 TMEM columns and at most 112 KB of
// shared memory, so two CTAs share an SM: while one CTA's eight compute warps turn a step into P and dS, the other's MMAs
// run, the next step's S / dP MMAs go out as soon as this step's sit in registers, and a CTA's prologue and final stores
// hide behind its neighbour's walk. dS is kept unscaled; the softmax scale multiplies dK and dQ once, on the way out.
struct BwdArgs {
  SdpaView<bf16> g0, g1;          // dK, dV  or  dQ (g1 unused)
  const float* lse;               // natural-log row sums of the forward; the kernels scale them by log2(e) where they read them
  const float* dr;
  int heads, kv_heads, time, h_first;
  int planes, group;              // of this launch: batch * kv_heads (dK/dV) or batch * heads (dQ); planes per L2 group
  float scale;
  uint32_t* fault;
};

// Dr[b,h,t] = sum_d dO . O: D / 8 threads per row, 16-byte loads. Skipped when the caller already has Dr (the gate's
// backward forms the same dot product).
template <int D>
__global__ void sdpa_bwd_prep_kernel(SdpaView<const bf16> out, SdpaView<const bf16> gout, float* __restrict__ dr,
                                     int heads, int time, int64_t rows) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  constexpr int TPR = D / 8;
  const int64_t r = min(gid / TPR, rows - 1);
  const int part = (int)(gid % TPR);
  const int t = (int)(r % time), h = (int)((r / time) % heads), b = (int)(r / ((int64_t)time * heads));
  const uint4 o = *reinterpret_cast<const uint4*>(out.row(b, h, t) + part * 8), g = *reinterpret_cast<const uint4*>(gout.row(b, h, t) + part * 8);
  const uint32_t ow[4] = {o.x, o.y, o.z, o.w}, gw[4] = {g.x, g.y, g.z, g.w};
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    acc += __uint_as_float(ow[i] << 16) * __uint_as_float(gw[i] << 16) + __uint_as_float(ow[i] & 0xffff0000u) * __uint_as_float(gw[i] & 0xffff0000u);
#pragma unroll
  for (int o = 1; o < TPR; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (part == 0 && gid / TPR < rows) dr[r] = acc;
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// COLS accumulator columns of this thread's TMEM lane -> bf16, scaled
template <int COLS>
__device__ __forceinline__ void store_row_bf16(bf16* dst, uint32_t taddr, float mul) {
#pragma unroll
  for (int c = 0; c < COLS / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_wait_ld();
    if (dst) {
#pragma unroll
      for (int i = 0; i < 32; i += 8)
        *reinterpret_cast<uint4*>(dst + c * 32 + i) =
            make_uint4(pack2_bf16(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul), pack2_bf16(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul),
                       pack2_bf16(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul), pack2_bf16(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul));
    }
  }
}

constexpr int SUB = 64;
constexpr int PT_BYTES = 128 * SUB * 2;        // 16 KB: 128 rows x 64 columns of P or dS (one 128-byte swizzled row each)
constexpr int IN_STAGES = 3;          // most q / dO stages the dK/dV kernel rings (its barrier table is laid out for these)
constexpr int DQ_STAGES = 3;          // k / v stages of the dQ kernel

// One step of a compute thread: 32 columns of its row. s, dp: the thread's S and dP values; stats: the columns' (dK/dV) or
// the row's (dQ) statistics, eight columns at a time; vis(e): column e is visible. emit(g, p, ds) takes the packed bf16 results, eight columns
// (one 16-byte chunk each of P and dS) at a time: kept in registers or stored, as the caller's pipeline wants.
template <bool MASKED, class STATS, class VIS, class EMIT>
__device__ __forceinline__ void bwd_step(const uint32_t (&s)[32], const uint32_t (&dp)[32], float sl2, STATS&& stats, VIS&& vis, EMIT&& emit) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float pv[8], dv[8], l2[8], dd[8];
    stats(g, l2, dd);                            // lse * log2(e) and Dr of columns 8g .. 8g + 7
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int c = g * 8 + e;
      const float p = fast_exp2(fmaf(__uint_as_float(s[c]), sl2, -l2[e]));
      const float ds = p * (__uint_as_float(dp[c]) - dd[e]);
      // masked columns: select, never multiply by zero (rows past the sequence end carry whatever the buffers held)
      pv[e] = (!MASKED || vis(c)) ? p : 0.0f;
      dv[e] = (!MASKED || vis(c)) ? ds : 0.0f;
    }
    emit(g, make_uint4(pack2_bf16(pv[0], pv[1]), pack2_bf16(pv[2], pv[3]), pack2_bf16(pv[4], pv[5]), pack2_bf16(pv[6], pv[7])),
         make_uint4(pack2_bf16(dv[0], dv[1]), pack2_bf16(dv[2], dv[3]), pack2_bf16(dv[4], dv[5]), pack2_bf16(dv[6], dv[7])));
  }
}
// 16-byte chunk half * 4 + g of a thread's 128-byte row; the swizzle XORs the chunk index with row % 8
__device__ __forceinline__ void store_chunk(uint8_t* row, const uint4& v, int half, int g, int tid) {
  *reinterpret_cast<uint4*>(row + (((half * 4 + g) ^ (tid & 7)) << 4)) = v;
}

// ---- dK, dV
template <int D> struct Dkv {
  static constexpr int STAGES = D == 64 ? IN_STAGES : 2;       // head_dim 128 (one CTA per SM) measured the same on two as on three
  static constexpr int NSUB = D / 64, TILE_BYTES = NSUB * ST128, STEP_BYTES = NSUB * ST64;   // K / V tile; one step of q or dO
  static constexpr int OFF_K = 0, OFF_V = TILE_BYTES, OFF_Q = 2 * TILE_BYTES, OFF_G = OFF_Q + STAGES * STEP_BYTES, OFF_P = OFF_G + STAGES * STEP_BYTES,
                       OFF_DS = OFF_P + PT_BYTES, OFF_STAT = OFF_DS + PT_BYTES;
  // Row statistics of a step (lse * log2 e and Dr of its 64 queries). One CTA per SM: they ride into shared memory with the
  // step's tiles. Two CTAs per SM: no room is left (112 KB of tiles + barriers fill the SM's half to the last kilobyte), so
  // the compute warps keep them in registers and shuffle them round.
  static constexpr bool STATS_IN_SMEM = D != 64;
  static constexpr int OFF_BAR = OFF_STAT + (STATS_IN_SMEM ? STAGES * 2 * SUB * 4 : 0);
  static constexpr int SMEM_BYTES = OFF_BAR + 128;              // D 64: 112 KB + 128; D 128: 161 KB
  static constexpr int TMEM_COLS = D == 64 ? 256 : 512;         // S^T 64 + dP^T 64 + dV D + dK D
  static constexpr int CTAS = D == 64 ? 2 : 1;
};
enum { KB_KVFULL = 0, KB_INFULL0, KB_INEMPTY0 = KB_INFULL0 + IN_STAGES, KB_SFULL = KB_INEMPTY0 + IN_STAGES, KB_SFREE, KB_PREADY, KB_PFREE, KB_DONE, KB_COUNT };

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, Dkv<D>::CTAS)
sdpa_bwd_dkv_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                            const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) { if (threadIdx.x == 0) raise_fault(args.fault, OP_SDPA); return; }   // the swizzled tiles need 1024-byte alignment (whole CTA leaves)
  uint8_t* base_ptr = smem_raw;
  using C = Dkv<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, STEP_BYTES = C::STEP_BYTES, KV_OFF_K = C::OFF_K, KV_OFF_V = C::OFF_V, KV_OFF_Q = C::OFF_Q, KV_OFF_G = C::OFF_G,
                KV_OFF_P = C::OFF_P, KV_OFF_DS = C::OFF_DS, KV_OFF_STAT = C::OFF_STAT, KV_OFF_BAR = C::OFF_BAR;
  constexpr uint32_t STEP16 = STEP_BYTES >> 4, TCOLS = C::TMEM_COLS;
  auto bar = [&](int i) { return base + KV_OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + KV_OFF_BAR + 8 * KB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileOrder ord = tile_order(blockIdx.x, args.planes, args.group, gridDim.x / args.planes);
  const int k0 = ord.rank * BN;                // early key tiles see the most queries
  const int plane = ord.plane, b = plane / args.kv_heads, hk = plane % args.kv_heads, rep = args.heads / args.kv_heads;
  const int q_subs = (args.time - k0 + SUB - 1) / SUB;      // query steps k0, k0 + 64, ... (k0 is a multiple of 128)
  const int iters = rep * q_subs;

  // step `it` of the walk: query head hk * rep + it / q_subs, queries from k0 + (it % q_subs) * SUB
  auto load_step = [&](int it) {
    const int s = it % C::STAGES, h = hk * rep + it / q_subs, q0 = k0 + (it % q_subs) * SUB;
    // statistics in shared memory ride on the same barrier (time is a multiple of 4, so the copies are whole 16-byte units)
    const uint32_t stat_bytes = C::STATS_IN_SMEM ? (uint32_t)min(SUB, args.time - q0) * 4u : 0u;
    mbar_expect_tx(bar(KB_INFULL0 + s), 2 * STEP_BYTES + 2 * stat_bytes);
    load_tile<NSUB, 64>(base + KV_OFF_Q + s * STEP_BYTES, &tm_q, bar(KB_INFULL0 + s), args.h_first, h, q0, b);
    load_tile<NSUB, 64>(base + KV_OFF_G + s * STEP_BYTES, &tm_g, bar(KB_INFULL0 + s), args.h_first, h, q0, b);
    if (C::STATS_IN_SMEM) {
      const int64_t idx = ((int64_t)b * args.heads + h) * args.time + q0;
      bulk_load(base + KV_OFF_STAT + s * 512, args.lse + idx, stat_bytes, bar(KB_INFULL0 + s));
      bulk_load(base + KV_OFF_STAT + s * 512 + 256, args.dr + idx, stat_bytes, bar(KB_INFULL0 + s));
    }
  };
  // the producer thread sets the barriers up and starts the first loads before the CTA-wide sync
  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_g);
    for (int i = 0; i < KB_COUNT; ++i) mbar_init(bar(i), (i == KB_PREADY || i == KB_SFREE) ? 256 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar(KB_KVFULL), 2 * TILE_BYTES);
    load_tile<NSUB, 128>(base + KV_OFF_K, &tm_k, bar(KB_KVFULL), args.h_first, hk, k0, b);
    load_tile<NSUB, 128>(base + KV_OFF_V, &tm_v, bar(KB_KVFULL), args.h_first, hk, k0, b);
    for (int it = 0; it < min(C::STAGES, iters); ++it) load_step(it);
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TCOLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S^T [0,64), dP^T [64,128), dV [128,128+D), dK [128+D,128+2D)

  if (warp == 8) {
    if (lane == 0) {
      for (int it = C::STAGES; it < iters; ++it) {
        if (!mbar_wait(bar(KB_INEMPTY0 + it % C::STAGES), ((it / C::STAGES) & 1) ^ 1, args.fault, abort_flag)) break;
        load_step(it);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BN, SUB, 0, 0), idesc_o = make_idesc(BN, D, 0, 1);
      const uint32_t k_lo = desc_lo(base + KV_OFF_K, 0), v_lo = desc_lo(base + KV_OFF_V, 0), q_lo = desc_lo(base + KV_OFF_Q, 0), g_lo = desc_lo(base + KV_OFF_G, 0);
      const uint32_t qm_lo = desc_lo(base + KV_OFF_Q, ST64), gm_lo = desc_lo(base + KV_OFF_G, ST64);   // the same tiles as MN-major B operands (64-wide blocks ST64 apart)
      const uint32_t p_lo = desc_lo(base + KV_OFF_P, 0), ds_lo = desc_lo(base + KV_OFF_DS, 0);
      // S^T = K Q^T and dP^T = V dO^T of step i
      auto issue_s = [&](uint32_t i) {
        const uint32_t st = (i % C::STAGES) * STEP16;
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base, k_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, q_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + 64, v_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, g_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(KB_SFULL));
      };
      bool ok = mbar_wait(bar(KB_KVFULL), 0, args.fault, abort_flag) && mbar_wait(bar(KB_INFULL0), 0, args.fault, abort_flag);
      if (ok) { fence_after(); issue_s(0); }
      for (uint32_t it = 0; it < (uint32_t)iters && ok; ++it) {
        // Two CTAs per SM (head_dim 64): the next step's S^T / dP^T go out as soon as every compute thread holds this
        // step's in registers, ahead of this step's dV / dK, so the tensor pipe works through the threads' exp and pack
        // phase. One CTA per SM (head_dim 128): dV / dK first, which hands the input stage back to the loads sooner.
        auto next_s = [&]() -> bool {
          if (it + 1 >= (uint32_t)iters) return true;
          if (C::CTAS == 2 && !mbar_wait(bar(KB_SFREE), it & 1, args.fault, abort_flag)) return false;
          if (!mbar_wait(bar(KB_INFULL0 + (it + 1) % C::STAGES), ((it + 1) / C::STAGES) & 1, args.fault, abort_flag)) return false;
          fence_after();
          issue_s(it + 1);
          return true;
        };
        if (C::CTAS == 2 && !next_s()) break;
        // every compute thread has written P / dS of this step
        if (!mbar_wait(bar(KB_PREADY), it & 1, args.fault, abort_flag)) break;
        fence_after();
        const uint32_t st = (it % C::STAGES) * STEP16;
#pragma unroll
        for (uint32_t kk = 0; kk < SUB / 16; ++kk)  // dV += P^T dO   (dO as the MN-major B operand: 16 queries = 2048 bytes)
          umma_lh(tmem_base + 128, p_lo + kk * KSTEP, gm_lo + st + kk * MNSTEP, HI, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (uint32_t kk = 0; kk < SUB / 16; ++kk)  // dK += dS^T Q
          umma_lh(tmem_base + 128 + D, ds_lo + kk * KSTEP, qm_lo + st + kk * MNSTEP, HI, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(KB_INEMPTY0 + it % C::STAGES));
        umma_commit(bar(KB_PFREE));               // P and dS may be overwritten
        if (it + 1 == (uint32_t)iters) umma_commit(bar(KB_DONE));
        if (C::CTAS == 1 && !next_s()) break;
      }
    }
  } else {
    // two warpgroups share the 128 TMEM lanes (a warp reaches lanes 32 * (warp % 4) ..): group `half` takes 32 of the step's 64 query columns
    const int tid = threadIdx.x & 127, half = warp >> 2, key = k0 + tid;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    uint8_t* p_row = base_ptr + KV_OFF_P + tid * 128;
    uint8_t* ds_row = base_ptr + KV_OFF_DS + tid * 128;
    bool ok = true;
    int q0 = k0;
    // Statistics kept out of shared memory: lane c of a warp holds those of column c of its half, fetched one step
    // ahead, and the warp shuffles them round as the columns come up.
    const float* stat = reinterpret_cast<const float*>(base_ptr + KV_OFF_STAT);   // [stage][lse 64 | dr 64] when in shared memory
    auto stat_of = [&](int it, float& l2, float& dr) {
      const int h = hk * rep + it / q_subs, q = k0 + (it % q_subs) * SUB + half * 32 + lane;
      const bool in = !C::STATS_IN_SMEM && it < iters && q < args.time;
      const int64_t idx = ((int64_t)b * args.heads + h) * args.time + q;
      l2 = in ? args.lse[idx] * LOG2E : INFINITY;
      dr = in ? args.dr[idx] : 0.0f;
    };
    float my_l2, my_dr, next_l2, next_dr;
    stat_of(0, my_l2, my_dr);
    for (int it = 0; it < iters; ++it) {
      stat_of(it + 1, next_l2, next_dr);
      if (!mbar_wait(bar(KB_SFULL), it & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      uint32_t rs[32], rp[32];
      tmem_ld32(lane_base + half * 32, rs);
      tmem_ld32(lane_base + 64 + half * 32, rp);
      tmem_wait_ld();
      if (C::CTAS == 2) { fence_before(); mbar_arrive(bar(KB_SFREE)); }   // the accumulator columns may take the next step
      const int qb = q0 + half * 32;
      const float* st = stat + (it % C::STAGES) * 128 + half * 32;
      auto stats = [&](int g, float (&l2)[8], float (&dd)[8]) {
        if (C::STATS_IN_SMEM) {                    // every thread of the warp reads the same values: 16-byte broadcast loads
          const float4 a = *reinterpret_cast<const float4*>(st + g * 8), b4 = *reinterpret_cast<const float4*>(st + g * 8 + 4);
          const float4 c = *reinterpret_cast<const float4*>(st + SUB + g * 8), d = *reinterpret_cast<const float4*>(st + SUB + g * 8 + 4);
          l2[0] = a.x * LOG2E; l2[1] = a.y * LOG2E; l2[2] = a.z * LOG2E; l2[3] = a.w * LOG2E;
          l2[4] = b4.x * LOG2E; l2[5] = b4.y * LOG2E; l2[6] = b4.z * LOG2E; l2[7] = b4.w * LOG2E;
          dd[0] = c.x; dd[1] = c.y; dd[2] = c.z; dd[3] = c.w; dd[4] = d.x; dd[5] = d.y; dd[6] = d.z; dd[7] = d.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) { l2[e] = __shfl_sync(0xffffffffu, my_l2, g * 8 + e); dd[e] = __shfl_sync(0xffffffffu, my_dr, g * 8 + e); }
        }
      };
      auto vis = [&](int c) { return key < args.time && qb + c < args.time && key <= qb + c; };
      const bool masked = q0 < k0 + BN || q0 + SUB > args.time || k0 + BN > args.time;   // diagonal steps or a ragged end
      // P and dS are free once the previous step's dV / dK MMAs have read them. With two CTAs per SM those run behind the
      // next S^T / dP^T, so the results wait in registers and the wait comes last; with one CTA per SM they were issued before
      // this step's S^T, whose commit (SFULL) covers them, and each chunk is stored as it is formed.
      if (C::CTAS == 2) {
        uint4 pp[4], dsp[4];
        auto keep = [&](int g, const uint4& p, const uint4& ds) { pp[g] = p; dsp[g] = ds; };
        if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, keep); else bwd_step<false>(rs, rp, sl2, stats, vis, keep);
        if (it > 0 && !mbar_wait(bar(KB_PFREE), (it - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
#pragma unroll
        for (int g = 0; g < 4; ++g) { store_chunk(p_row, pp[g], half, g, tid); store_chunk(ds_row, dsp[g], half, g, tid); }
      } else {
        auto put = [&](int g, const uint4& p, const uint4& ds) { store_chunk(p_row, p, half, g, tid); store_chunk(ds_row, ds, half, g, tid); };
        if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, put); else bwd_step<false>(rs, rp, sl2, stats, vis, put);
      }
      fence_async_smem();
      mbar_arrive(bar(KB_PREADY));
      my_l2 = next_l2; my_dr = next_dr;
      q0 += SUB;
      if (q0 >= args.time) q0 = k0;
    }
    if (ok && mbar_wait(bar(KB_DONE), 0, args.fault, abort_flag)) {
      fence_after();
      if (half == 0) store_row_bf16<D>(key < args.time ? args.g1.row(b, hk, key) : nullptr, lane_base + 128, 1.0f);     // dV
      else store_row_bf16<D>(key < args.time ? args.g0.row(b, hk, key) : nullptr, lane_base + 128 + D, args.scale);         // dK
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TCOLS) : "memory");
  }
}

// ---- dQ
template <int D> struct Dq {
  static constexpr int NSUB = D / 64, TILE_BYTES = NSUB * ST128, STEP_BYTES = NSUB * ST64;   // q / dO tile; one step of k or v
  static constexpr int OFF_Q = 0, OFF_G = TILE_BYTES, OFF_K = 2 * TILE_BYTES, OFF_V = OFF_K + DQ_STAGES * STEP_BYTES, OFF_DS = OFF_V + DQ_STAGES * STEP_BYTES,
                       OFF_BAR = OFF_DS + PT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128 + 1024;       // D 64: 97 KB (two CTAs per SM); D 128: 177 KB
  static constexpr int CTAS = D == 64 ? 2 : 1;
};
enum { QB_QDFULL = 0, QB_INFULL0, QB_INEMPTY0 = QB_INFULL0 + DQ_STAGES, QB_SFULL = QB_INEMPTY0 + DQ_STAGES, QB_SFREE, QB_PREADY, QB_PFREE, QB_DONE, QB_COUNT };

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, Dq<D>::CTAS)
sdpa_bwd_dq_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                           const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  using C = Dq<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, STEP_BYTES = C::STEP_BYTES, DQ_OFF_Q = C::OFF_Q, DQ_OFF_G = C::OFF_G, DQ_OFF_K = C::OFF_K, DQ_OFF_V = C::OFF_V,
                DQ_OFF_DS = C::OFF_DS, DQ_OFF_BAR = C::OFF_BAR;
  constexpr uint32_t STEP16 = STEP_BYTES >> 4;
  auto bar = [&](int i) { return base + DQ_OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + DQ_OFF_BAR + 8 * QB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileOrder ord = tile_order(blockIdx.x, args.planes, args.group, gridDim.x / args.planes);
  const int qt = gridDim.x / args.planes - 1 - ord.rank;
  const int q0 = qt * BM;
  const int plane = ord.plane, b = plane / args.heads, h = plane % args.heads, hk = h / (args.heads / args.kv_heads);
  const int n_end = min(args.time, q0 + BM);
  const int iters = (n_end + SUB - 1) / SUB;     // key steps 0, 64, ...

  auto load_step = [&](int it) {
    const int s = it % DQ_STAGES;
    mbar_expect_tx(bar(QB_INFULL0 + s), 2 * STEP_BYTES);
    load_tile<NSUB, 64>(base + DQ_OFF_K + s * STEP_BYTES, &tm_k, bar(QB_INFULL0 + s), args.h_first, hk, it * SUB, b);
    load_tile<NSUB, 64>(base + DQ_OFF_V + s * STEP_BYTES, &tm_v, bar(QB_INFULL0 + s), args.h_first, hk, it * SUB, b);
  };
  // the producer thread sets the barriers up and starts the first loads before the CTA-wide sync
  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_g);
    for (int i = 0; i < QB_COUNT; ++i) mbar_init(bar(i), (i == QB_PREADY || i == QB_SFREE) ? 256 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar(QB_QDFULL), 2 * TILE_BYTES);
    load_tile<NSUB, 128>(base + DQ_OFF_Q, &tm_q, bar(QB_QDFULL), args.h_first, h, q0, b);
    load_tile<NSUB, 128>(base + DQ_OFF_G, &tm_g, bar(QB_QDFULL), args.h_first, h, q0, b);
    for (int it = 0; it < min(DQ_STAGES, iters); ++it) load_step(it);
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S [0,64), dP [64,128), dQ [128,128+D)

  if (warp == 8) {
    if (lane == 0) {
      for (int it = DQ_STAGES; it < iters; ++it) {
        if (!mbar_wait(bar(QB_INEMPTY0 + it % DQ_STAGES), ((it / DQ_STAGES) & 1) ^ 1, args.fault, abort_flag)) break;
        load_step(it);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, SUB, 0, 0), idesc_o = make_idesc(BM, D, 0, 1);
      const uint32_t q_lo = desc_lo(base + DQ_OFF_Q, 0), g_lo = desc_lo(base + DQ_OFF_G, 0), k_lo = desc_lo(base + DQ_OFF_K, 0), v_lo = desc_lo(base + DQ_OFF_V, 0);
      const uint32_t km_lo = desc_lo(base + DQ_OFF_K, ST64), ds_lo = desc_lo(base + DQ_OFF_DS, 0);
      // S = Q K^T and dP = dO V^T of step i
      auto issue_s = [&](uint32_t i) {
        const uint32_t st = (i % DQ_STAGES) * STEP16;
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base, q_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, k_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + 64, g_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, v_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(QB_SFULL));
      };
      bool ok = mbar_wait(bar(QB_QDFULL), 0, args.fault, abort_flag) && mbar_wait(bar(QB_INFULL0), 0, args.fault, abort_flag);
      if (ok) { fence_after(); issue_s(0); }
      for (uint32_t it = 0; it < (uint32_t)iters && ok; ++it) {
        // the next step's S / dP: ahead of this step's dQ with two CTAs per SM, after it with one (see the dK/dV kernel)
        auto next_s = [&]() -> bool {
          if (it + 1 >= (uint32_t)iters) return true;
          if (C::CTAS == 2 && !mbar_wait(bar(QB_SFREE), it & 1, args.fault, abort_flag)) return false;
          if (!mbar_wait(bar(QB_INFULL0 + (it + 1) % DQ_STAGES), ((it + 1) / DQ_STAGES) & 1, args.fault, abort_flag)) return false;
          fence_after();
          issue_s(it + 1);
          return true;
        };
        if (C::CTAS == 2 && !next_s()) break;
        if (!mbar_wait(bar(QB_PREADY), it & 1, args.fault, abort_flag)) break;
        fence_after();
        const uint32_t st = (it % DQ_STAGES) * STEP16;
#pragma unroll
        for (uint32_t kk = 0; kk < SUB / 16; ++kk)  // dQ += dS K   (K as the MN-major B operand: 16 keys = 2048 bytes)
          umma_lh(tmem_base + 128, ds_lo + kk * KSTEP, km_lo + st + kk * MNSTEP, HI, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(QB_INEMPTY0 + it % DQ_STAGES));
        umma_commit(bar(QB_PFREE));               // dS may be overwritten
        if (it + 1 == (uint32_t)iters) umma_commit(bar(QB_DONE));
        if (C::CTAS == 1 && !next_s()) break;
      }
    }
  } else {
    const int tid = threadIdx.x & 127, half = warp >> 2, row = q0 + tid;   // warpgroup `half` takes 32 of the step's 64 key columns
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    const int64_t idx = ((int64_t)b * args.heads + h) * args.time + row;
    const float lse_row = row < args.time ? args.lse[idx] * LOG2E : INFINITY, dr_row = row < args.time ? args.dr[idx] : 0.0f;
    uint8_t* ds_row = base_ptr + DQ_OFF_DS + tid * 128;
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      const int key0 = it * SUB + half * 32;
      if (!mbar_wait(bar(QB_SFULL), it & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      uint32_t rs[32], rp[32];
      tmem_ld32(lane_base + half * 32, rs);
      tmem_ld32(lane_base + 64 + half * 32, rp);
      tmem_wait_ld();
      if (C::CTAS == 2) { fence_before(); mbar_arrive(bar(QB_SFREE)); }
      auto stats = [&](int, float (&l2)[8], float (&dd)[8]) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { l2[e] = lse_row; dd[e] = dr_row; }
      };
      auto vis = [&](int c) { return key0 + c <= row && key0 + c < args.time; };
      const bool masked = it * SUB + SUB > q0 || it * SUB + SUB > args.time;
      if (C::CTAS == 2) {                           // as in the dK/dV kernel: keep, wait late, store
        uint4 dsp[4];
        auto keep = [&](int g, const uint4&, const uint4& ds) { dsp[g] = ds; };
        if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, keep); else bwd_step<false>(rs, rp, sl2, stats, vis, keep);
        if (it > 0 && !mbar_wait(bar(QB_PFREE), (it - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
#pragma unroll
        for (int g = 0; g < 4; ++g) store_chunk(ds_row, dsp[g], half, g, tid);
      } else {
        auto put = [&](int g, const uint4&, const uint4& ds) { store_chunk(ds_row, ds, half, g, tid); };
        if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, put); else bwd_step<false>(rs, rp, sl2, stats, vis, put);
      }
      fence_async_smem();
      mbar_arrive(bar(QB_PREADY));
    }
    if (ok && mbar_wait(bar(QB_DONE), 0, args.fault, abort_flag)) {
      fence_after();
      store_row_bf16<D / 2>(row < args.time ? args.g0.row(b, h, row) + half * (D / 2) : nullptr, lane_base + 128 + half * (D / 2), args.scale);
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

// ================================================================================================ backward, persistent CTAs
// The two backward kernels with their roles kept alive over many tiles, as the persistent forward kernel: a CTA takes every
// gridDim.x-th tile of the long-walks-first order and runs them as one stream of 64-wide steps. The step ring never drains between
// tiles, the tile the CTA keeps (K and V, or Q and dO) is reloaded as soon as the last S-type product that reads it has finished
// (under that step's exp phase, its accumulating products and the tile's final stores), the next tile's first S-type products go out
// under the current tile's last step, and the accumulators are handed back as soon as the compute threads hold them in registers,
// so their conversion and stores run under the next tile's walk. TMEM and the barriers are set up once per CTA.
enum { QP_QDFULL = 0, QP_QDEMPTY, QP_INFULL0, QP_INEMPTY0 = QP_INFULL0 + DQ_STAGES, QP_SFULL = QP_INEMPTY0 + DQ_STAGES, QP_SFREE, QP_PREADY, QP_PFREE, QP_DONE, QP_ACCFREE,
       QP_COUNT };

struct DqWalk {
  int q0, b, h, hk, iters;
  __device__ __forceinline__ bool set(const BwdArgs& args, int tiles, int total, int item) {
    const int g = blockIdx.x + item * gridDim.x;
    if (g >= total) return false;
    const TileOrder ord = tile_order(g, args.planes, args.group, tiles);
    q0 = (tiles - 1 - ord.rank) * BM;
    b = ord.plane / args.heads; h = ord.plane % args.heads; hk = h / (args.heads / args.kv_heads);
    iters = (min(args.time, q0 + BM) + SUB - 1) / SUB;
    return true;
  }
};

// COLS accumulator columns of this thread's TMEM lane into registers
template <int COLS>
__device__ __forceinline__ void load_acc(uint32_t taddr, uint32_t (&r)[COLS]) {
#pragma unroll
  for (int c = 0; c < COLS / 32; ++c) tmem_ld32(taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
  tmem_wait_ld();
}
template <int COLS>
__device__ __forceinline__ void store_acc_bf16(bf16* dst, const uint32_t (&r)[COLS], float mul) {
  if (!dst) return;
#pragma unroll
  for (int i = 0; i < COLS; i += 8)
    *reinterpret_cast<uint4*>(dst + i) =
        make_uint4(pack2_bf16(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul), pack2_bf16(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul),
                   pack2_bf16(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul), pack2_bf16(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul));
}

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, Dq<D>::CTAS)
sdpa_bwd_dq_p_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  using C = Dq<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, STEP_BYTES = C::STEP_BYTES;
  constexpr uint32_t STEP16 = STEP_BYTES >> 4;
  static_assert(QP_COUNT * 8 + 8 <= 128, "barrier table");
  auto bar = [&](int i) { return base + C::OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + C::OFF_BAR + 8 * QP_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (args.time + BM - 1) / BM, total = tiles * args.planes;

  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_g);
    for (int i = 0; i < QP_COUNT; ++i) mbar_init(bar(i), (i == QP_PREADY || i == QP_SFREE || i == QP_ACCFREE) ? 256 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S [0,64), dP [64,128), dQ [128,128+D)

  if (warp == 8) {
    if (lane == 0) {
      DqWalk w;
      int gs = 0;
      bool ok = true;
      for (int item = 0; ok && w.set(args, tiles, total, item); ++item) {
        // the Q / dO tile is free once the previous tile's last S / dP have read it
        if (item > 0 && !mbar_wait(bar(QP_QDEMPTY), (item - 1) & 1, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(QP_QDFULL), 2 * TILE_BYTES);
        load_tile<NSUB, 128>(base + C::OFF_Q, &tm_q, bar(QP_QDFULL), args.h_first, w.h, w.q0, w.b);
        load_tile<NSUB, 128>(base + C::OFF_G, &tm_g, bar(QP_QDFULL), args.h_first, w.h, w.q0, w.b);
        for (int it = 0; it < w.iters; ++it, ++gs) {
          const int s = gs % DQ_STAGES;
          if (gs >= DQ_STAGES && !mbar_wait(bar(QP_INEMPTY0 + s), ((gs / DQ_STAGES) & 1) ^ 1, args.fault, abort_flag)) { ok = false; break; }
          mbar_expect_tx(bar(QP_INFULL0 + s), 2 * STEP_BYTES);
          load_tile<NSUB, 64>(base + C::OFF_K + s * STEP_BYTES, &tm_k, bar(QP_INFULL0 + s), args.h_first, w.hk, it * SUB, w.b);
          load_tile<NSUB, 64>(base + C::OFF_V + s * STEP_BYTES, &tm_v, bar(QP_INFULL0 + s), args.h_first, w.hk, it * SUB, w.b);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, SUB, 0, 0), idesc_o = make_idesc(BM, D, 0, 1);
      const uint32_t q_lo = desc_lo(base + C::OFF_Q, 0), g_lo = desc_lo(base + C::OFF_G, 0), k_lo = desc_lo(base + C::OFF_K, 0), v_lo = desc_lo(base + C::OFF_V, 0);
      const uint32_t km_lo = desc_lo(base + C::OFF_K, ST64), ds_lo = desc_lo(base + C::OFF_DS, 0);
      // S = Q K^T and dP = dO V^T of global step n; `last`: the tile's last such pair, after which Q / dO may be replaced
      auto issue_s = [&](uint32_t n, bool last) {
        const uint32_t st = (n % DQ_STAGES) * STEP16;
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base, q_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, k_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + 64, g_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, v_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(QP_SFULL));
        if (last) umma_commit(bar(QP_QDEMPTY));
      };
      DqWalk cur, nxt;
      bool have = cur.set(args, tiles, total, 0);
      bool ok = have && mbar_wait(bar(QP_QDFULL), 0, args.fault, abort_flag) && mbar_wait(bar(QP_INFULL0), 0, args.fault, abort_flag);
      if (ok) { fence_after(); issue_s(0, cur.iters == 1); }
      uint32_t gs = 0;
      for (int item = 0; have && ok; ++item) {
        const bool more = nxt.set(args, tiles, total, item + 1);
        for (int it = 0; it < cur.iters && ok; ++it, ++gs) {
          // the next step's S / dP (this tile's, or the first of the next tile): ahead of this step's dQ with two CTAs per SM, after it with one
          auto next_s = [&]() -> bool {
            const bool within = it + 1 < cur.iters;
            if (!within && !more) return true;
            if (C::CTAS == 2 && !mbar_wait(bar(QP_SFREE), gs & 1, args.fault, abort_flag)) return false;
            const uint32_t n = gs + 1;
            if (!within && !mbar_wait(bar(QP_QDFULL), (item + 1) & 1, args.fault, abort_flag)) return false;
            if (!mbar_wait(bar(QP_INFULL0 + n % DQ_STAGES), (n / DQ_STAGES) & 1, args.fault, abort_flag)) return false;
            fence_after();
            issue_s(n, within ? it + 2 == cur.iters : nxt.iters == 1);
            return true;
          };
          if (C::CTAS == 2 && !next_s()) { ok = false; break; }
          if (!mbar_wait(bar(QP_PREADY), gs & 1, args.fault, abort_flag)) { ok = false; break; }
          // a tile's first dQ product overwrites the accumulator: the previous tile's rows must hold theirs in registers
          if (it == 0 && item > 0 && !mbar_wait(bar(QP_ACCFREE), (item - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          fence_after();
          const uint32_t st = (gs % DQ_STAGES) * STEP16;
#pragma unroll
          for (uint32_t kk = 0; kk < SUB / 16; ++kk)
            umma_lh(tmem_base + 128, ds_lo + kk * KSTEP, km_lo + st + kk * MNSTEP, HI, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
          umma_commit(bar(QP_INEMPTY0 + gs % DQ_STAGES));
          umma_commit(bar(QP_PFREE));
          if (it + 1 == cur.iters) umma_commit(bar(QP_DONE));
          if (C::CTAS == 1 && !next_s()) { ok = false; break; }
        }
        cur = nxt;
        have = more;
      }
    }
  } else {
    const int tid = threadIdx.x & 127, half = warp >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    uint8_t* ds_row = base_ptr + C::OFF_DS + tid * 128;
    DqWalk w;
    uint32_t gs = 0;
    bool ok = true;
    for (int item = 0; ok && w.set(args, tiles, total, item); ++item) {
      const int row = w.q0 + tid;
      const int64_t idx = ((int64_t)w.b * args.heads + w.h) * args.time + row;
      const float lse_row = row < args.time ? args.lse[idx] * LOG2E : INFINITY, dr_row = row < args.time ? args.dr[idx] : 0.0f;
      for (int it = 0; it < w.iters; ++it, ++gs) {
        const int key0 = it * SUB + half * 32;
        if (!mbar_wait(bar(QP_SFULL), gs & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        uint32_t rs[32], rp[32];
        tmem_ld32(lane_base + half * 32, rs);
        tmem_ld32(lane_base + 64 + half * 32, rp);
        tmem_wait_ld();
        if (C::CTAS == 2) { fence_before(); mbar_arrive(bar(QP_SFREE)); }
        auto stats = [&](int, float (&l2)[8], float (&dd)[8]) {
#pragma unroll
          for (int e = 0; e < 8; ++e) { l2[e] = lse_row; dd[e] = dr_row; }
        };
        auto vis = [&](int c) { return key0 + c <= row && key0 + c < args.time; };
        const bool masked = it * SUB + SUB > w.q0 || it * SUB + SUB > args.time;
        if (C::CTAS == 2) {
          uint4 dsp[4];
          auto keep = [&](int g, const uint4&, const uint4& ds) { dsp[g] = ds; };
          if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, keep); else bwd_step<false>(rs, rp, sl2, stats, vis, keep);
          if (gs > 0 && !mbar_wait(bar(QP_PFREE), (gs - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
#pragma unroll
          for (int g = 0; g < 4; ++g) store_chunk(ds_row, dsp[g], half, g, tid);
        } else {
          auto put = [&](int g, const uint4&, const uint4& ds) { store_chunk(ds_row, ds, half, g, tid); };
          if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, put); else bwd_step<false>(rs, rp, sl2, stats, vis, put);
        }
        fence_async_smem();
        mbar_arrive(bar(QP_PREADY));
      }
      if (!ok) break;
      if (!mbar_wait(bar(QP_DONE), item & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      uint32_t acc[D / 2];
      load_acc<D / 2>(lane_base + 128 + half * (D / 2), acc);
      fence_before();
      mbar_arrive(bar(QP_ACCFREE));              // the accumulator may take the next tile while these rows are converted and stored
      store_acc_bf16<D / 2>(row < args.time ? args.g0.row(w.b, w.h, row) + half * (D / 2) : nullptr, acc, args.scale);
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

enum { KP_KVFULL = 0, KP_KVEMPTY, KP_INFULL0, KP_INEMPTY0 = KP_INFULL0 + IN_STAGES, KP_SFULL = KP_INEMPTY0 + IN_STAGES, KP_SFREE, KP_PREADY, KP_PFREE, KP_DONE, KP_ACCFREE,
       KP_COUNT };

struct DkvWalk {
  int k0, b, hk, q_subs, iters;
  __device__ __forceinline__ bool set(const BwdArgs& args, int tiles, int total, int item) {
    const int g = blockIdx.x + item * gridDim.x;
    if (g >= total) return false;
    const TileOrder ord = tile_order(g, args.planes, args.group, tiles);
    k0 = ord.rank * BN;                          // early key tiles see the most queries
    b = ord.plane / args.kv_heads; hk = ord.plane % args.kv_heads;
    q_subs = (args.time - k0 + SUB - 1) / SUB;
    iters = (args.heads / args.kv_heads) * q_subs;
    return true;
  }
};

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, Dkv<D>::CTAS)
sdpa_bwd_dkv_p_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) { if (threadIdx.x == 0) raise_fault(args.fault, OP_SDPA); return; }
  uint8_t* base_ptr = smem_raw;
  using C = Dkv<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, STEP_BYTES = C::STEP_BYTES;
  constexpr uint32_t STEP16 = STEP_BYTES >> 4, TCOLS = C::TMEM_COLS;
  static_assert(KP_COUNT * 8 + 8 <= 128, "barrier table");
  auto bar = [&](int i) { return base + C::OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + C::OFF_BAR + 8 * KP_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (args.time + BN - 1) / BN, total = tiles * args.planes, rep = args.heads / args.kv_heads;

  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_g);
    for (int i = 0; i < KP_COUNT; ++i) mbar_init(bar(i), (i == KP_PREADY || i == KP_SFREE || i == KP_ACCFREE) ? 256 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TCOLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S^T [0,64), dP^T [64,128), dV [128,128+D), dK [128+D,128+2D)

  if (warp == 8) {
    if (lane == 0) {
      DkvWalk w;
      int gs = 0;
      bool ok = true;
      for (int item = 0; ok && w.set(args, tiles, total, item); ++item) {
        if (item > 0 && !mbar_wait(bar(KP_KVEMPTY), (item - 1) & 1, args.fault, abort_flag)) break;
        mbar_expect_tx(bar(KP_KVFULL), 2 * TILE_BYTES);
        load_tile<NSUB, 128>(base + C::OFF_K, &tm_k, bar(KP_KVFULL), args.h_first, w.hk, w.k0, w.b);
        load_tile<NSUB, 128>(base + C::OFF_V, &tm_v, bar(KP_KVFULL), args.h_first, w.hk, w.k0, w.b);
        for (int it = 0; it < w.iters; ++it, ++gs) {
          const int s = gs % C::STAGES, h = w.hk * rep + it / w.q_subs, q0 = w.k0 + (it % w.q_subs) * SUB;
          if (gs >= C::STAGES && !mbar_wait(bar(KP_INEMPTY0 + s), ((gs / C::STAGES) & 1) ^ 1, args.fault, abort_flag)) { ok = false; break; }
          const uint32_t stat_bytes = C::STATS_IN_SMEM ? (uint32_t)min(SUB, args.time - q0) * 4u : 0u;
          mbar_expect_tx(bar(KP_INFULL0 + s), 2 * STEP_BYTES + 2 * stat_bytes);
          load_tile<NSUB, 64>(base + C::OFF_Q + s * STEP_BYTES, &tm_q, bar(KP_INFULL0 + s), args.h_first, h, q0, w.b);
          load_tile<NSUB, 64>(base + C::OFF_G + s * STEP_BYTES, &tm_g, bar(KP_INFULL0 + s), args.h_first, h, q0, w.b);
          if (C::STATS_IN_SMEM) {
            const int64_t idx = ((int64_t)w.b * args.heads + h) * args.time + q0;
            bulk_load(base + C::OFF_STAT + s * 512, args.lse + idx, stat_bytes, bar(KP_INFULL0 + s));
            bulk_load(base + C::OFF_STAT + s * 512 + 256, args.dr + idx, stat_bytes, bar(KP_INFULL0 + s));
          }
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BN, SUB, 0, 0), idesc_o = make_idesc(BN, D, 0, 1);
      const uint32_t k_lo = desc_lo(base + C::OFF_K, 0), v_lo = desc_lo(base + C::OFF_V, 0), q_lo = desc_lo(base + C::OFF_Q, 0), g_lo = desc_lo(base + C::OFF_G, 0);
      const uint32_t qm_lo = desc_lo(base + C::OFF_Q, ST64), gm_lo = desc_lo(base + C::OFF_G, ST64);
      const uint32_t p_lo = desc_lo(base + C::OFF_P, 0), ds_lo = desc_lo(base + C::OFF_DS, 0);
      auto issue_s = [&](uint32_t n, bool last) {
        const uint32_t st = (n % C::STAGES) * STEP16;
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base, k_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, q_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + 64, v_lo + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, g_lo + st + (kk >> 2) * ST64_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(KP_SFULL));
        if (last) umma_commit(bar(KP_KVEMPTY));
      };
      DkvWalk cur, nxt;
      bool have = cur.set(args, tiles, total, 0);
      bool ok = have && mbar_wait(bar(KP_KVFULL), 0, args.fault, abort_flag) && mbar_wait(bar(KP_INFULL0), 0, args.fault, abort_flag);
      if (ok) { fence_after(); issue_s(0, cur.iters == 1); }
      uint32_t gs = 0;
      for (int item = 0; have && ok; ++item) {
        const bool more = nxt.set(args, tiles, total, item + 1);
        for (int it = 0; it < cur.iters && ok; ++it, ++gs) {
          auto next_s = [&]() -> bool {
            const bool within = it + 1 < cur.iters;
            if (!within && !more) return true;
            if (C::CTAS == 2 && !mbar_wait(bar(KP_SFREE), gs & 1, args.fault, abort_flag)) return false;
            const uint32_t n = gs + 1;
            if (!within && !mbar_wait(bar(KP_KVFULL), (item + 1) & 1, args.fault, abort_flag)) return false;
            if (!mbar_wait(bar(KP_INFULL0 + n % C::STAGES), (n / C::STAGES) & 1, args.fault, abort_flag)) return false;
            fence_after();
            issue_s(n, within ? it + 2 == cur.iters : nxt.iters == 1);
            return true;
          };
          if (C::CTAS == 2 && !next_s()) { ok = false; break; }
          if (!mbar_wait(bar(KP_PREADY), gs & 1, args.fault, abort_flag)) { ok = false; break; }
          if (it == 0 && item > 0 && !mbar_wait(bar(KP_ACCFREE), (item - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          fence_after();
          const uint32_t st = (gs % C::STAGES) * STEP16;
#pragma unroll
          for (uint32_t kk = 0; kk < SUB / 16; ++kk)  // dV += P^T dO
            umma_lh(tmem_base + 128, p_lo + kk * KSTEP, gm_lo + st + kk * MNSTEP, HI, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
          for (uint32_t kk = 0; kk < SUB / 16; ++kk)  // dK += dS^T Q
            umma_lh(tmem_base + 128 + D, ds_lo + kk * KSTEP, qm_lo + st + kk * MNSTEP, HI, idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
          umma_commit(bar(KP_INEMPTY0 + gs % C::STAGES));
          umma_commit(bar(KP_PFREE));
          if (it + 1 == cur.iters) umma_commit(bar(KP_DONE));
          if (C::CTAS == 1 && !next_s()) { ok = false; break; }
        }
        cur = nxt;
        have = more;
      }
    }
  } else {
    const int tid = threadIdx.x & 127, half = warp >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    uint8_t* p_row = base_ptr + C::OFF_P + tid * 128;
    uint8_t* ds_row = base_ptr + C::OFF_DS + tid * 128;
    const float* stat = reinterpret_cast<const float*>(base_ptr + C::OFF_STAT);
    DkvWalk w, wn;
    // statistics kept in registers (two CTAs per SM): lane c of a warp holds those of column c of its half, fetched one step ahead
    auto stat_of = [&](const DkvWalk& t, bool valid, int it, float& l2, float& dr) {
      const int h = t.hk * rep + it / t.q_subs, q = t.k0 + (it % t.q_subs) * SUB + half * 32 + lane;
      const bool in = !C::STATS_IN_SMEM && valid && q < args.time;
      const int64_t idx = ((int64_t)t.b * args.heads + h) * args.time + q;
      l2 = in ? args.lse[idx] * LOG2E : INFINITY;
      dr = in ? args.dr[idx] : 0.0f;
    };
    uint32_t gs = 0;
    bool ok = true, have = w.set(args, tiles, total, 0);
    float my_l2 = INFINITY, my_dr = 0.0f, next_l2, next_dr;
    if (have) stat_of(w, true, 0, my_l2, my_dr);
    for (int item = 0; ok && have; ++item) {
      const bool more = wn.set(args, tiles, total, item + 1);
      const int key = w.k0 + tid;
      int q0 = w.k0;
      for (int it = 0; it < w.iters; ++it, ++gs) {
        if (it + 1 < w.iters) stat_of(w, true, it + 1, next_l2, next_dr); else stat_of(wn, more, 0, next_l2, next_dr);
        if (!mbar_wait(bar(KP_SFULL), gs & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        uint32_t rs[32], rp[32];
        tmem_ld32(lane_base + half * 32, rs);
        tmem_ld32(lane_base + 64 + half * 32, rp);
        tmem_wait_ld();
        if (C::CTAS == 2) { fence_before(); mbar_arrive(bar(KP_SFREE)); }
        const int qb = q0 + half * 32;
        const float* st = stat + (gs % C::STAGES) * 128 + half * 32;
        auto stats = [&](int g, float (&l2)[8], float (&dd)[8]) {
          if (C::STATS_IN_SMEM) {
            const float4 a = *reinterpret_cast<const float4*>(st + g * 8), b4 = *reinterpret_cast<const float4*>(st + g * 8 + 4);
            const float4 c = *reinterpret_cast<const float4*>(st + SUB + g * 8), d = *reinterpret_cast<const float4*>(st + SUB + g * 8 + 4);
            l2[0] = a.x * LOG2E; l2[1] = a.y * LOG2E; l2[2] = a.z * LOG2E; l2[3] = a.w * LOG2E;
            l2[4] = b4.x * LOG2E; l2[5] = b4.y * LOG2E; l2[6] = b4.z * LOG2E; l2[7] = b4.w * LOG2E;
            dd[0] = c.x; dd[1] = c.y; dd[2] = c.z; dd[3] = c.w; dd[4] = d.x; dd[5] = d.y; dd[6] = d.z; dd[7] = d.w;
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { l2[e] = __shfl_sync(0xffffffffu, my_l2, g * 8 + e); dd[e] = __shfl_sync(0xffffffffu, my_dr, g * 8 + e); }
          }
        };
        auto vis = [&](int c) { return key < args.time && qb + c < args.time && key <= qb + c; };
        const bool masked = q0 < w.k0 + BN || q0 + SUB > args.time || w.k0 + BN > args.time;
        if (C::CTAS == 2) {
          uint4 pp[4], dsp[4];
          auto keep = [&](int g, const uint4& p, const uint4& ds) { pp[g] = p; dsp[g] = ds; };
          if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, keep); else bwd_step<false>(rs, rp, sl2, stats, vis, keep);
          if (gs > 0 && !mbar_wait(bar(KP_PFREE), (gs - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
#pragma unroll
          for (int g = 0; g < 4; ++g) { store_chunk(p_row, pp[g], half, g, tid); store_chunk(ds_row, dsp[g], half, g, tid); }
        } else {
          auto put = [&](int g, const uint4& p, const uint4& ds) { store_chunk(p_row, p, half, g, tid); store_chunk(ds_row, ds, half, g, tid); };
          if (masked) bwd_step<true>(rs, rp, sl2, stats, vis, put); else bwd_step<false>(rs, rp, sl2, stats, vis, put);
        }
        fence_async_smem();
        mbar_arrive(bar(KP_PREADY));
        my_l2 = next_l2; my_dr = next_dr;
        q0 += SUB;
        if (q0 >= args.time) q0 = w.k0;
      }
      if (!ok) break;
      if (!mbar_wait(bar(KP_DONE), item & 1, args.fault, abort_flag)) { ok = false; break; }
      fence_after();
      uint32_t acc[D];
      load_acc<D>(lane_base + 128 + (half == 0 ? 0 : D), acc);
      fence_before();
      mbar_arrive(bar(KP_ACCFREE));
      if (half == 0) store_acc_bf16<D>(key < args.time ? args.g1.row(w.b, w.hk, key) : nullptr, acc, 1.0f);              // dV
      else store_acc_bf16<D>(key < args.time ? args.g0.row(w.b, w.hk, key) : nullptr, acc, args.scale);                 // dK
      w = wn;
      have = more;
    }
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TCOLS) : "memory");
  }
}

#include "sdpa_bwd_wide.cuh"

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A [B, H, T, dh] view (any batch / head / time strides, dh contiguous) as a 4-D tensor map whose boxes are `rows` time steps x 64
// columns of one head (one 128-byte swizzle span per row).
ojc_status make_map(ojc_backend* be, const char* op, CUtensorMap* map, const ojc_tensor* t, bool h_first, uint32_t rows = 128) {
  const uint64_t B = t->shape[0], H = t->shape[1], T = t->shape[2], dh = t->shape[3];
  cuuint64_t gdim[4], gstride[3];
  cuuint32_t box[4], estride[4] = {1, 1, 1, 1};
  gdim[0] = dh; box[0] = 64;
  if (h_first) { gdim[1] = H; gstride[0] = t->stride[1] * 2; box[1] = 1; gdim[2] = T; gstride[1] = t->stride[2] * 2; box[2] = rows; }
  else { gdim[1] = T; gstride[0] = t->stride[2] * 2; box[1] = rows; gdim[2] = H; gstride[1] = t->stride[1] * 2; box[2] = 1; }
  gdim[3] = B; gstride[2] = t->stride[0] * 2; box[3] = 1;
  CUresult r = ((EncodeTiledFn)be->tmap_encode)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t->data, gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ojc_fail(OJC_ERR_BACKEND, op, "cuTensorMapEncodeTiled refused an attention operand (code " + std::to_string((int)r) + ")");
  return OJC_OK;
}

int g_sdpa_forward_variant = 0;   // ojc_sdpa_forward_variant: 0 the library's choice, 1 one CTA per tile, 2 persistent kernels on three CTAs

bool strides_ok(const ojc_tensor* t) {
  return (reinterpret_cast<uintptr_t>(t->data) & 15) == 0 && t->stride[3] == 1 && t->stride[0] % 8 == 0 && t->stride[1] % 8 == 0 && t->stride[2] % 8 == 0 &&
         t->stride[0] > 0 && t->stride[1] > 0 && t->stride[2] > 0;
}

}  // namespace

bool sdpa_tcgen05_eligible(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, int64_t window, const SdpaDims& d) {
  if (!be->tmap_encode || q->dtype != OJC_BF16 || (d.dim != 64 && d.dim != 128) || window >= 0) return false;
  if (!strides_ok(q) || !strides_ok(k) || !strides_ok(v) || !strides_ok(out)) return false;
  // one dimension order for all three maps: heads inside time, or time inside heads
  const bool hf = q->stride[1] < q->stride[2];
  return (k->stride[1] < k->stride[2]) == hf && (v->stride[1] < v->stride[2]) == hf;
}

template <int D>
static ojc_status launch_fwd2(ojc_backend* be, const char* op, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FwdArgs& args, dim3 grid) {
  static PerDeviceFlag attr_of;
  bool& attr = attr_of[be->device];
  if (!attr) { OJC_CUDA(be, cudaFuncSetAttribute(sdpa_fwd2_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2<D>::SMEM_BYTES), op); attr = true; }
  sdpa_fwd2_tcgen05_kernel<D><<<grid, FWD2_THREADS, Fwd2<D>::SMEM_BYTES, be->stream>>>(mq, mk, mv, args);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

template <int D>
static ojc_status launch_fwdp(ojc_backend* be, const char* op, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FwdArgs& args, int total_tiles) {
  static PerDeviceFlag attr_of;
  bool& attr = attr_of[be->device];
  if (!attr) { OJC_CUDA(be, cudaFuncSetAttribute(sdpa_fwdp_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdP<D>::SMEM_BYTES), op); attr = true; }
  const int grid = std::min(total_tiles, g_sdpa_forward_variant == 2 ? 3 : be->sm_count * FwdP<D>::CTAS);
  sdpa_fwdp_tcgen05_kernel<D><<<grid, NTHREADS, FwdP<D>::SMEM_BYTES, be->stream>>>(mq, mk, mv, args);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

template <int D>
static ojc_status launch_fwd(ojc_backend* be, const char* op, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FwdArgs& args, dim3 grid) {
  static PerDeviceFlag attr_of;
  bool& attr = attr_of[be->device];
  if (!attr) { OJC_CUDA(be, cudaFuncSetAttribute(sdpa_fwd_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd<D>::SMEM_BYTES), op); attr = true; }
  sdpa_fwd_tcgen05_kernel<D><<<grid, NTHREADS, Fwd<D>::SMEM_BYTES, be->stream>>>(mq, mk, mv, args);
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

ojc_status sdpa_forward_tcgen05(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, ojc_tensor* out, float* lse, const SdpaDims& d) {
  const char* op = "causal_sdpa_forward";
  const bool hf = q->stride[1] < q->stride[2];
  CUtensorMap mq, mk, mv;
  OJC_TRY(make_map(be, op, &mq, q, hf));
  OJC_TRY(make_map(be, op, &mk, k, hf));
  OJC_TRY(make_map(be, op, &mv, v, hf));
  FwdArgs args;
  args.out = SdpaView<bf16>{(bf16*)out->data, out->stride[0], out->stride[1], out->stride[2]};
  args.lse = lse; args.heads = d.heads; args.kv_heads = d.kv_heads; args.time = d.time; args.h_first = hf ? 1 : 0; args.scale = d.scale; args.fault = be->fault_dev;
  args.planes = d.batch * d.heads;
  args.group = planes_per_group(d.time, d.dim, args.planes);
  // Two query tiles per CTA (P in tensor memory) where it measured faster: head_dim 128, where one CTA owns the SM either way
  // ([8,16,4096,128]: 671 us against 686 us). At head_dim 64 two one-tile CTAs share an SM and overlap each other's softmax, and
  // the short walks of T = 1024 favour them (162 us against 181 us at B 32, H 12).
  if (d.dim == 128 && d.time > BM && g_sdpa_forward_variant != 1) {
    dim3 grid2((unsigned)(((d.time + 2 * BM - 1) / (2 * BM)) * args.planes));
    return d.dim == 64 ? launch_fwd2<64>(be, op, mq, mk, mv, args, grid2) : launch_fwd2<128>(be, op, mq, mk, mv, args, grid2);
  }
  dim3 grid((unsigned)(((d.time + BM - 1) / BM) * args.planes));
  if (d.dim == 64 && g_sdpa_forward_variant != 1 && (g_sdpa_forward_variant == 2 || grid.x > (unsigned)(be->sm_count * FwdP<64>::CTAS)))
    return launch_fwdp<64>(be, op, mq, mk, mv, args, (int)grid.x);
  return d.dim == 64 ? launch_fwd<64>(be, op, mq, mk, mv, args, grid) : launch_fwd<128>(be, op, mq, mk, mv, args, grid);
}

template <int D>
static ojc_status launch_bwd(ojc_backend* be, const char* op, const ojc_tensor* out, const ojc_tensor* gout, float* dr_work, int64_t rows,
                             const CUtensorMap (&m)[8], BwdArgs a, const ojc_tensor* gq, const ojc_tensor* gk, const ojc_tensor* gv, const SdpaDims& d) {
  static PerDeviceFlag attr_of;
  bool& attr = attr_of[be->device];
  if (!attr) {
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dkv_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Dkv<D>::SMEM_BYTES), op);
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dq_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Dq<D>::SMEM_BYTES), op);
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dkv_p_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Dkv<D>::SMEM_BYTES), op);
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dq_p_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Dq<D>::SMEM_BYTES), op);
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dkv_w_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvW<D>::SMEM_BYTES), op);
    OJC_CUDA(be, cudaFuncSetAttribute(sdpa_bwd_dq_w_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqW<D>::SMEM_BYTES), op);
    attr = true;
  }
  if (dr_work) {   // the caller has no Dr of its own
    sdpa_bwd_prep_kernel<D><<<(unsigned)((rows * (D / 8) + 255) / 256), 256, 0, be->stream>>>(
        SdpaView<const bf16>{(const bf16*)out->data, out->stride[0], out->stride[1], out->stride[2]},
        SdpaView<const bf16>{(const bf16*)gout->data, gout->stride[0], gout->stride[1], gout->stride[2]}, dr_work, d.heads, d.time, rows);
    OJC_LAUNCHED(be, op);
  }
  a.g0 = SdpaView<bf16>{(bf16*)gk->data, gk->stride[0], gk->stride[1], gk->stride[2]};
  a.g1 = SdpaView<bf16>{(bf16*)gv->data, gv->stride[0], gv->stride[1], gv->stride[2]};
  a.planes = d.batch * d.kv_heads;
  a.group = planes_per_group(d.time, d.dim, a.planes);
  dim3 grid_k((unsigned)(((d.time + BN - 1) / BN) * a.planes));
  // persistent CTAs at head_dim 64 once there are more tiles than CTA slots (B 32 x H 12 x T 1024: 411 us against 423 us for both kernels;
  // at head_dim 128, one CTA per SM, they measured slower: [8,16,4096,128] 3264 us against 3127 us)
  // the library's choice: persistent CTAs walking in 128-wide steps, P and dS in tensor memory (one CTA per SM)
  // At head_dim 128 they measured 1.4 to 1.55 times faster than the 64-wide kernels from T 512 to T 8192 ([8,16,4096,128]: 2039 us
  // against 3128 us). At head_dim 64 the 64-wide kernels, two CTAs per SM, stay about 5% ahead at every length tried (T 512 to 4096):
  // there the accumulating products are N = 64 either way, and the second CTA hides tile switches that one CTA's pipeline shows.
  const int v = g_sdpa_forward_variant;
  const bool wide = v == 3 || v == 5 || (v == 0 && D == 128);
  const unsigned wide_cap = g_sdpa_forward_variant == 3 ? 3u : (unsigned)be->sm_count;
  if (wide) {
    sdpa_bwd_dkv_w_kernel<D><<<std::min<unsigned>(grid_k.x, wide_cap), BWD_THREADS, DkvW<D>::SMEM_BYTES, be->stream>>>(m[0], m[1], m[2], m[3], a);
    OJC_LAUNCHED(be, op);
    a.g0 = SdpaView<bf16>{(bf16*)gq->data, gq->stride[0], gq->stride[1], gq->stride[2]};
    a.planes = d.batch * d.heads;
    a.group = planes_per_group(d.time, d.dim, a.planes);
    const unsigned tiles_q = (unsigned)(((d.time + BM - 1) / BM) * a.planes);
    sdpa_bwd_dq_w_kernel<D><<<std::min<unsigned>(tiles_q, wide_cap), BWD_THREADS, DqW<D>::SMEM_BYTES, be->stream>>>(m[0], m[1], m[2], m[3], a);
    OJC_LAUNCHED(be, op);
    return OJC_OK;
  }
  const bool persist_k = g_sdpa_forward_variant == 2 || (D == 64 && g_sdpa_forward_variant != 1 && (int)grid_k.x > be->sm_count * Dkv<D>::CTAS);
  if (persist_k) sdpa_bwd_dkv_p_kernel<D><<<g_sdpa_forward_variant == 2 ? std::min<unsigned>(grid_k.x, 3u) : (unsigned)(be->sm_count * Dkv<D>::CTAS), BWD_THREADS, Dkv<D>::SMEM_BYTES, be->stream>>>(m[4], m[1], m[2], m[7], a);
  else sdpa_bwd_dkv_tcgen05_kernel<D><<<grid_k, BWD_THREADS, Dkv<D>::SMEM_BYTES, be->stream>>>(m[4], m[1], m[2], m[7], a);   // q, dO in 64-row steps
  OJC_LAUNCHED(be, op);
  a.g0 = SdpaView<bf16>{(bf16*)gq->data, gq->stride[0], gq->stride[1], gq->stride[2]};
  a.planes = d.batch * d.heads;
  a.group = planes_per_group(d.time, d.dim, a.planes);
  dim3 grid_q((unsigned)(((d.time + BM - 1) / BM) * a.planes));
  const bool persist_q = g_sdpa_forward_variant == 2 || (D == 64 && g_sdpa_forward_variant != 1 && (int)grid_q.x > be->sm_count * Dq<D>::CTAS);
  if (persist_q) sdpa_bwd_dq_p_kernel<D><<<g_sdpa_forward_variant == 2 ? std::min<unsigned>(grid_q.x, 3u) : (unsigned)(be->sm_count * Dq<D>::CTAS), BWD_THREADS, Dq<D>::SMEM_BYTES, be->stream>>>(m[0], m[5], m[6], m[3], a);
  else sdpa_bwd_dq_tcgen05_kernel<D><<<grid_q, BWD_THREADS, Dq<D>::SMEM_BYTES, be->stream>>>(m[0], m[5], m[6], m[3], a);      // k, v in 64-row steps
  OJC_LAUNCHED(be, op);
  return OJC_OK;
}

// `work` holds B * H * T floats for Dr = rowsum(dO . O), filled by the prepass, unless the caller passes `dr_given` (Dr it
// already has, [B, H, T]). Eligibility is the forward's plus the gradient views.
ojc_status sdpa_backward_tcgen05(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const float* lse,
                                 const ojc_tensor* gout, ojc_tensor* gq, ojc_tensor* gk, ojc_tensor* gv, const SdpaDims& d, float* work, const float* dr_given) {
  const char* op = "causal_sdpa_backward";
  const int64_t rows = (int64_t)d.batch * d.heads * d.time;
  const bool hf = q->stride[1] < q->stride[2];
  // maps 0-3: q, k, v, dO in 128-row tiles (the operand a CTA keeps); 4-7: the same in 64-row steps (the one it walks)
  CUtensorMap m[8];
  const ojc_tensor* src[4] = {q, k, v, gout};
  for (int i = 0; i < 4; ++i) { OJC_TRY(make_map(be, op, &m[i], src[i], hf)); OJC_TRY(make_map(be, op, &m[4 + i], src[i], hf, SUB)); }
  BwdArgs a;
  a.lse = lse; a.dr = dr_given ? dr_given : work; a.heads = d.heads; a.kv_heads = d.kv_heads; a.time = d.time; a.h_first = hf ? 1 : 0; a.scale = d.scale; a.fault = be->fault_dev;
  float* prep = dr_given ? nullptr : work;
  return d.dim == 64 ? launch_bwd<64>(be, op, out, gout, prep, rows, m, a, gq, gk, gv, d) : launch_bwd<128>(be, op, out, gout, prep, rows, m, a, gq, gk, gv, d);
}

bool sdpa_tcgen05_bwd_eligible(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* gout, const ojc_tensor* gq,
                               const ojc_tensor* gk, const ojc_tensor* gv, int64_t window, const SdpaDims& d) {
  if (!sdpa_tcgen05_eligible(be, q, k, v, gout, window, d) || d.time % 4 != 0) return false;
  const bool hf = q->stride[1] < q->stride[2];
  return strides_ok(gq) && strides_ok(gk) && strides_ok(gv) && (gout->stride[1] < gout->stride[2]) == hf;
}

// Instrumentation (no counterpart in the reference): 0 = the library's choice (forward: two query tiles per CTA at head_dim 128, persistent
// CTAs at head_dim 64; backward: the 128-wide persistent kernels at head_dim 128, the 64-wide persistent ones at head_dim 64 once there
// are more tiles than CTA slots), 1 = always one CTA per tile (to time the others against it), 2 = the 64-wide persistent kernels on a
// grid of at most three CTAs, whatever the size (so that small test shapes walk several tiles per CTA), 3 = the 128-wide backward kernels
// on at most three CTAs (likewise), 4 = the 64-wide backward kernels by their own rule, 5 = the 128-wide backward kernels at any head_dim.
extern "C" ojc_status ojc_sdpa_forward_variant(int32_t variant) { g_sdpa_forward_variant = variant >= 0 && variant <= 5 ? variant : 0; return OJC_OK; }

