// bf16 x bf16 -> f32 GEMM on the Blackwell tensor cores (sm_100a).
//
//   C[m,n] = alpha * A[m,k] . B[k,n]  (+ residual)  (+ C)
//
// A persistent kernel, one CTA per SM, ten warps with fixed roles:
//   warp 0   TMA producer: cp.async.bulk.tensor loads of A and B tiles (128-byte
//            swizzle, each CTA fetching its own tiles) into a 4-stage shared-memory ring
//   warp 1   allocates tensor memory and issues tcgen05.mma (one thread);
//            accumulators live in TMEM, double-buffered (2 x 256 columns) so
//            the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2-9  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM
//            lanes and half of the columns), scale, write 32 x 128-byte blocks
//            into swizzled staging rows and hand them to TMA tile stores (the
//            adding form for C += ...); with a residual operand the block goes
//            through padded staging rows and coalesced f32 loads / stores instead
// Tile 128 x 256 x 64; either operand may be K-major or MN-major in memory, so
// x.W^T, g.W and g^T.x all run on the same kernel without transposed copies.
// When the output has too few tiles to fill the GPU the reduction axis is
// split; partial tiles go to workspace and are summed in split order by a
// second kernel (deterministic; no float atomics).
//
// Every mbarrier wait is bounded by a wall-clock limit: when it runs out the
// kernel raises the fault word, stops issuing work, lets its copies land,
// frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "gemm.cuh"
#include "swiglu_math.cuh"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2, B_TILE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int STAGE_LD = 20;                      // floats per staged epilogue row (16 + 4 of padding), residual path
constexpr int EPI_WARP_BYTES = 32 * 128;          // per epilogue warp: 32 rows of 128 bytes (one swizzled TMA-store box)
constexpr int EPI_STAGE_BYTES = 8 * EPI_WARP_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + EPI_STAGE_BYTES + 256 /*barriers*/;
static_assert(32 * STAGE_LD * 4 <= EPI_WARP_BYTES, "the padded residual-path rows share the store staging");
constexpr int EPI_WARPS = 8;                     // two warps per TMEM lane quarter, each draining half of the columns
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
static_assert(SMEM_BYTES <= 232448, "shared memory per CTA");

struct TcArgs {
  void* c; int c_bf16; int64_t ldc;
  int m, n, k;
  int a_mn_major, b_mn_major;
  float alpha; int accumulate; const float* residual;
  int splits, kblocks_per_split;
  float* partial;           // [splits][m][n] when splits > 1
  uint32_t* fault;
  int batch;                // independent matrices: a unit is (matrix, tile, split); batch > 1 needs tma_store and splits == 1
  int tma_store;            // finished blocks leave through TMA tile stores (no residual operand; split partials need m % 32 == 0)
  const bf16* ns_src; int64_t ns_ld, ns_bs; float ns_src_mul, ns_acc_mul;   // Newton-Schulz combine epilogue (NsCombine); ns_src null: none
  const bf16* sw_au; int64_t sw_ld;   // SwiGLU-backward epilogue (SwigluGrad): a at column 0, u at column n of rows sw_ld wide; null: none
  int sw_f;                 // SwiGLU-forward epilogue (SwigluForward): the hidden width F; C is (a | u), n = 2 F
  int tiles_n_fast;         // tile order: 1 = neighbouring CTAs share an A row block (few column tiles), 0 = they share a B column block
};

// Stores of finished 32-row blocks: TMA tile stores out of swizzled staging rows (the hardware clips at the matrix edge),
// or the adding form for C += tile.
// (every map is 3-D: columns, rows, matrix of the batch)
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Drains one warp's share of a finished accumulator tile: TMEM lanes [32 quarter, +32) x columns [col_begin, col_end)
// starting at `tsrc`, destined for rows row_base.. and columns col_tile0.. of matrix bz of C (or of the split's partial).
__device__ __forceinline__ void drain_tile(const TcArgs& args, const CUtensorMap& tmap_c, uint32_t tsrc, int row_base, int col_tile0, int split, int bz, int lane,
                                           int col_begin, int col_end, uint8_t* stage_bytes, uint32_t stage_addr) {
  float* stage = reinterpret_cast<float*>(stage_bytes);
  if (args.tma_store) {
    // Each lane owns one accumulator row: it writes 128 bytes of it (64 bf16 or 32 f32 columns) into the warp's
    // swizzled staging box, and lane 0 hands the 32 x 128-byte box to the TMA unit.
    const bool bf = args.c_bf16 && args.splits == 1;
    const int step = bf ? 64 : 32;
    const int y = (args.splits > 1 ? split * args.m : 0) + row_base;
#pragma unroll 1
    for (int c0 = col_begin; c0 < col_end; c0 += step) {
      uint32_t r[32], r2[32];
      tmem_ld32(tsrc + c0, r);
      if (bf) tmem_ld32(tsrc + c0 + 32, r2);
      tmem_wait_ld();
      if (lane == 0) bulk_wait_read();       // the previous box has left the staging rows
      __syncwarp();
      uint8_t* rowp = stage_bytes + lane * 128;
      const float al = args.splits > 1 ? 1.0f : args.alpha;
      if (bf && args.ns_src) {
        // C = bf16(bf16(src_mul * src) + bf16(acc_mul * bf16(acc))): this lane's row, 64 columns from c0
        const int grow = row_base + lane, gcol = col_tile0 + c0;
        const bf16* srow = args.ns_src + (int64_t)bz * args.ns_bs + (int64_t)grow * args.ns_ld + gcol;
        const bool whole = grow < args.m && gcol + 64 <= args.n;
        auto rb = [](float x) { return __uint_as_float(pack2_bf16(0.0f, x) & 0xffff0000u); };
        bool bad = false;
#pragma unroll
        for (int ci = 0; ci < 8; ++ci) {
          const uint32_t* v = ci < 4 ? &r[ci * 8] : &r2[(ci - 4) * 8];
          float sv[8];
          if (whole) {
            const uint4 t = *reinterpret_cast<const uint4*>(srow + ci * 8);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) { sv[2 * e] = __uint_as_float(w[e] << 16); sv[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) sv[e] = (grow < args.m && gcol + ci * 8 + e < args.n) ? __bfloat162float(srow[ci * 8 + e]) : 0.0f;
          }
          float o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            o[e] = rb(rb(args.ns_src_mul * sv[e]) + rb(args.ns_acc_mul * rb(__uint_as_float(v[e]))));
            bad |= !isfinite(o[e]);
          }
          *reinterpret_cast<uint4*>(rowp + ((ci ^ (lane & 7)) << 4)) =
              make_uint4(pack2_bf16(o[0], o[1]), pack2_bf16(o[2], o[3]), pack2_bf16(o[4], o[5]), pack2_bf16(o[6], o[7]));
        }
        if (bad && grow < args.m) raise_fault(args.fault, OP_MUON);
      } else if (bf) {
#pragma unroll
        for (int ci = 0; ci < 8; ++ci) {
          const uint32_t* v = ci < 4 ? &r[ci * 8] : &r2[(ci - 4) * 8];
          *reinterpret_cast<uint4*>(rowp + ((ci ^ (lane & 7)) << 4)) =
              make_uint4(pack2_bf16(al * __uint_as_float(v[0]), al * __uint_as_float(v[1])), pack2_bf16(al * __uint_as_float(v[2]), al * __uint_as_float(v[3])),
                         pack2_bf16(al * __uint_as_float(v[4]), al * __uint_as_float(v[5])), pack2_bf16(al * __uint_as_float(v[6]), al * __uint_as_float(v[7])));
        }
      } else {
#pragma unroll
        for (int ci = 0; ci < 8; ++ci)
          *reinterpret_cast<float4*>(rowp + ((ci ^ (lane & 7)) << 4)) =
              make_float4(al * __uint_as_float(r[ci * 4]), al * __uint_as_float(r[ci * 4 + 1]), al * __uint_as_float(r[ci * 4 + 2]), al * __uint_as_float(r[ci * 4 + 3]));
      }
      fence_async_smem();
      __syncwarp();
      const int x = col_tile0 + c0;
      if (lane == 0 && x < args.n && row_base < args.m) {
        if (args.accumulate && args.splits == 1) tma_reduce_add_3d(&tmap_c, stage_addr, x, y, bz);
        else tma_store_3d(&tmap_c, stage_addr, x, y, bz);
        bulk_commit();
      }
    }
    return;
  }
#pragma unroll 1
  for (int c0 = col_begin; c0 < col_end; c0 += 32) {
    uint32_t r[32];
    __syncwarp();
    tmem_ld32(tsrc + c0, r);
    tmem_wait_ld();
    const int col0 = col_tile0 + c0;
    // residual path: each thread holds one accumulator row; pass the block, 16 columns at a time, through this warp's
    // padded staging rows so the global accesses are row-contiguous across lanes (4 lanes x 16 bytes per row).
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (half) __syncwarp();
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4*>(stage + lane * STAGE_LD + j) = make_float4(__uint_as_float(r[half * 16 + j]), __uint_as_float(r[half * 16 + j + 1]),
                                                                               __uint_as_float(r[half * 16 + j + 2]), __uint_as_float(r[half * 16 + j + 3]));
      __syncwarp();
      const int cc = (lane & 3) * 4, gcol = col0 + half * 16 + cc;
      if (gcol >= args.n) continue;
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int rr = it * 8 + (lane >> 2), grow = row_base + rr;
        if (grow >= args.m) continue;
        float4 v = *reinterpret_cast<const float4*>(stage + rr * STAGE_LD + cc);
        if (args.splits > 1) {
          *reinterpret_cast<float4*>(args.partial + ((int64_t)split * args.m + grow) * args.n + gcol) = v;
          continue;
        }
        const int64_t o = (int64_t)grow * args.ldc + gcol;
        v.x *= args.alpha; v.y *= args.alpha; v.z *= args.alpha; v.w *= args.alpha;
        if (args.residual) { const float4 t = *reinterpret_cast<const float4*>(args.residual + o); v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w; }
        if (!args.c_bf16) {
          float* dst = reinterpret_cast<float*>(args.c) + o;
          if (args.accumulate) { const float4 t = *reinterpret_cast<const float4*>(dst); v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w; }
          *reinterpret_cast<float4*>(dst) = v;
        } else {
          *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(args.c) + o) = make_uint2(pack2_bf16(v.x, v.y), pack2_bf16(v.z, v.w));
        }
      }
    }
  }
}

// SwiGLU backward on 64 columns of this warp's share of a finished accumulator: the accumulator is g, the gradient of
// m = bf16(silu(a)) * u, rounded to bf16 as a stored g would be. a and u of the same 32 rows x 64 columns sit in the warp's two staging
// boxes, lane = row (swizzled 128-byte rows, put there by the caller); each lane turns its row into g_a and g_u in place, 16 bytes at a
// time, and the boxes leave as two TMA stores: g_a to columns x.., g_u to columns n + x.. of the output rows.
__device__ __forceinline__ void drain_swiglu_backward(const TcArgs& args, const CUtensorMap& tmap_c, uint32_t tsrc, int row_base, int x, int c0, int bz, int lane,
                                                      uint8_t* stage_bytes, uint32_t stage_addr) {
  uint8_t* rowp = stage_bytes + lane * 128;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t r[32];
    tmem_ld32(tsrc + c0 + half * 32, r);
    tmem_wait_ld();
#pragma unroll
    for (int cj = 0; cj < 4; ++cj) {
      const int off = ((half * 4 + cj) ^ (lane & 7)) << 4;
      const uint32_t* v = &r[cj * 8];
      const uint4 qa = *reinterpret_cast<const uint4*>(rowp + off), qu = *reinterpret_cast<const uint4*>(rowp + EPI_WARP_BYTES + off);
      const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wu[4] = {qu.x, qu.y, qu.z, qu.w};
      float ga[8], gu[8];
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        float g0 = __uint_as_float(v[e]), g1 = __uint_as_float(v[e + 1]);
        swiglu::round2_bf16(g0, g1);
        swiglu::backward_pair(__uint_as_float(wa[e >> 1] << 16), __uint_as_float(wa[e >> 1] & 0xffff0000u), __uint_as_float(wu[e >> 1] << 16),
                              __uint_as_float(wu[e >> 1] & 0xffff0000u), g0, g1, ga[e], ga[e + 1], gu[e], gu[e + 1]);
      }
      *reinterpret_cast<uint4*>(rowp + off) = make_uint4(pack2_bf16(ga[0], ga[1]), pack2_bf16(ga[2], ga[3]), pack2_bf16(ga[4], ga[5]), pack2_bf16(ga[6], ga[7]));
      *reinterpret_cast<uint4*>(rowp + EPI_WARP_BYTES + off) = make_uint4(pack2_bf16(gu[0], gu[1]), pack2_bf16(gu[2], gu[3]), pack2_bf16(gu[4], gu[5]), pack2_bf16(gu[6], gu[7]));
    }
  }
  fence_async_smem();
  __syncwarp();
  if (lane == 0 && x < args.n && row_base < args.m) {
    tma_store_3d(&tmap_c, stage_addr, x, row_base, bz);
    tma_store_3d(&tmap_c, stage_addr + EPI_WARP_BYTES, args.n + x, row_base, bz);
    bulk_commit();
  }
}

// SwiGLU forward on a finished two-SM accumulator whose 256 columns are gate columns [j0, j0 + 128) followed by up columns
// [F + j0, F + j0 + 128) of the (a | u) row: this warp takes 64 gate columns and the 64 up columns that go with them, rounds both
// to bf16 (what the stored a and u hold), and sends out three boxes in turn through its staging rows: a, u and
// m = bf16(silu(a)) * u. The same bits as the product followed by the row kernel.
__device__ __forceinline__ void drain_swiglu_forward(const TcArgs& args, const CUtensorMap& tmap_c, const CUtensorMap& tmap_m, uint32_t tsrc, int row_base, int j0,
                                                     int bz, int lane, int half, uint8_t* stage_bytes, uint32_t stage_addr) {
  const int j = j0 + half * 64;
  uint4 second[8], third[8];
  uint8_t* rowp = stage_bytes + lane * 128;
  if (lane == 0) bulk_wait_read();           // the previous tile's last box has left the staging rows
  __syncwarp();
#pragma unroll
  for (int part = 0; part < 2; ++part) {
    uint32_t ra[32], ru[32];
    tmem_ld32(tsrc + half * 64 + part * 32, ra);
    tmem_ld32(tsrc + 128 + half * 64 + part * 32, ru);
    tmem_wait_ld();
#pragma unroll
    for (int cj = 0; cj < 4; ++cj) {
      const int ci = part * 4 + cj;
      float a[8], u[8], m[8];
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        a[e] = __uint_as_float(ra[cj * 8 + e]); a[e + 1] = __uint_as_float(ra[cj * 8 + e + 1]);
        u[e] = __uint_as_float(ru[cj * 8 + e]); u[e + 1] = __uint_as_float(ru[cj * 8 + e + 1]);
        swiglu::round2_bf16(a[e], a[e + 1]);
        swiglu::round2_bf16(u[e], u[e + 1]);
        swiglu::forward_pair(a[e], a[e + 1], u[e], u[e + 1], m[e], m[e + 1]);
      }
      *reinterpret_cast<uint4*>(rowp + ((ci ^ (lane & 7)) << 4)) = make_uint4(pack2_bf16(a[0], a[1]), pack2_bf16(a[2], a[3]), pack2_bf16(a[4], a[5]), pack2_bf16(a[6], a[7]));
      second[ci] = make_uint4(pack2_bf16(u[0], u[1]), pack2_bf16(u[2], u[3]), pack2_bf16(u[4], u[5]), pack2_bf16(u[6], u[7]));
      third[ci] = make_uint4(pack2_bf16(m[0], m[1]), pack2_bf16(m[2], m[3]), pack2_bf16(m[4], m[5]), pack2_bf16(m[6], m[7]));
    }
  }
  const bool issue = lane == 0 && j < args.sw_f && row_base < args.m;
  fence_async_smem();
  __syncwarp();
  if (issue) { tma_store_3d(&tmap_c, stage_addr, j, row_base, bz); bulk_commit(); bulk_wait_read(); }
  __syncwarp();
#pragma unroll
  for (int ci = 0; ci < 8; ++ci) *reinterpret_cast<uint4*>(rowp + ((ci ^ (lane & 7)) << 4)) = second[ci];
  fence_async_smem();
  __syncwarp();
  if (issue) { tma_store_3d(&tmap_c, stage_addr, args.sw_f + j, row_base, bz); bulk_commit(); bulk_wait_read(); }
  __syncwarp();
#pragma unroll
  for (int ci = 0; ci < 8; ++ci) *reinterpret_cast<uint4*>(rowp + ((ci ^ (lane & 7)) << 4)) = third[ci];
  fence_async_smem();
  __syncwarp();
  if (issue) { tma_store_3d(&tmap_m, stage_addr, j, row_base, bz); bulk_commit(); }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c,
               const TcArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;               // 128-byte swizzle atoms repeat every 1024 bytes
  const uint32_t epi_base = tiles_base + STAGES * STAGE_BYTES;       // 1024-aligned: the store boxes are swizzled too
  const uint32_t bar_base = epi_base + EPI_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bar_base - raw) + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_ptr = smem_raw + (epi_base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (args.m + BM - 1) / BM, tiles_n = (args.n + BN - 1) / BN;
  const int units_per_matrix = tiles_m * tiles_n * args.splits, units = units_per_matrix * args.batch;
  const int kblocks_total = (args.k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched with programmatic stream serialization: everything above (barriers, tensor memory) may run while the kernel before this
  // one in the stream is still finishing on other SMs; nothing below touches global memory before that kernel is complete. The
  // trigger lets the kernel after this one do the same with its own prologue once this one's CTAs start leaving.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x) {
        const int bz = u / units_per_matrix, ub = u - bz * units_per_matrix;
        const int split = ub % args.splits, tile = ub / args.splits;
        const int tm = args.tiles_n_fast ? tile / tiles_n : tile % tiles_m, tn = args.tiles_n_fast ? tile % tiles_n : tile / tiles_m;
        const int kb0 = split * args.kblocks_per_split, kb1 = min(kblocks_total, kb0 + args.kblocks_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, args.fault, abort_flag)) break;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const uint32_t a_dst = tiles_base + s * STAGE_BYTES, b_dst = a_dst + A_TILE_BYTES;
          if (!args.a_mn_major) tma_load_3d(a_dst, &tmap_a, full_bar(s), kb * BK, tm * BM, bz);
          else for (int j = 0; j < BM / 64; ++j) tma_load_3d(a_dst + j * (BK * 128), &tmap_a, full_bar(s), tm * BM + j * 64, kb * BK, bz);
          if (!args.b_mn_major) tma_load_3d(b_dst, &tmap_b, full_bar(s), kb * BK, tn * BN, bz);
          else for (int j = 0; j < BN / 64; ++j) tma_load_3d(b_dst + j * (BK * 128), &tmap_b, full_bar(s), tn * BN + j * 64, kb * BK, bz);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, BN, args.a_mn_major, args.b_mn_major);
      // K-major: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO), one MMA step = 32 bytes along the row.
      // MN-major: 64-element column blocks BK*128 bytes apart (LBO), 8-row K groups 1024 bytes apart (SBO), one MMA step = 2 groups.
      const uint32_t a_lbo = args.a_mn_major ? BK * 128 : 0, b_lbo = args.b_mn_major ? BK * 128 : 0;
      const uint32_t a_step = args.a_mn_major ? 2048 : 32, b_step = args.b_mn_major ? 2048 : 32;
      uint32_t it = 0, local = 0;
      for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x, ++local) {
        const int split = (u % units_per_matrix) % args.splits;
        const int kb0 = split * args.kblocks_per_split, kb1 = min(kblocks_total, kb0 + args.kblocks_per_split);
        const int acc = local & 1;
        if (!mbar_wait(tempty_bar(acc), ((local >> 1) & 1) ^ 1, args.fault, abort_flag)) break;
        fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar(s), (it / STAGES) & 1, args.fault, abort_flag)) { ok = false; break; }
          fence_after();
          const uint32_t a_src = tiles_base + s * STAGE_BYTES, b_src = a_src + A_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = make_desc(a_src + kk * a_step, a_lbo, 1024);
            const uint64_t db = make_desc(b_src + kk * b_step, b_lbo, 1024);
            umma(tmem_d, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(s));      // frees the stage when these MMAs have read it
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));      // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;         // TMEM lanes [32 * quarter, +32) are this warp's
    const int col_begin = ((warp - 2) >> 2) * (BN / 2), col_end = col_begin + BN / 2;
    uint8_t* stage_bytes = epi_ptr + (warp - 2) * EPI_WARP_BYTES;
    const uint32_t stage_addr = epi_base + (warp - 2) * EPI_WARP_BYTES;
    uint32_t local = 0;
    for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x, ++local) {
      const int bz = u / units_per_matrix, ub = u - bz * units_per_matrix;
      const int split = ub % args.splits, tile = ub / args.splits;
      const int tm = args.tiles_n_fast ? tile / tiles_n : tile % tiles_m, tn = args.tiles_n_fast ? tile % tiles_n : tile / tiles_m;
      const int acc = local & 1;
      if (!mbar_wait(tfull_bar(acc), (local >> 1) & 1, args.fault, abort_flag)) break;
      fence_after();
      const int row_base = tm * BM + quarter * 32;
      const uint32_t tsrc = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      drain_tile(args, tmap_c, tsrc, row_base, tn * BN, split, bz, lane, col_begin, col_end, stage_bytes, stage_addr);
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (args.tma_store && lane == 0) bulk_wait_all();   // the staging rows must outlive the last store's read; its writes finish before the grid does
  }
  // Teardown: on an aborted run give copies in flight time to land before the shared memory goes away.
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The two-SM form: a cluster of two CTAs owns a 256 x 256 tile. Each CTA stages its own 128 rows of A and 128 columns
// of B (32 KB per stage instead of 48 KB, six stages), one thread of the even CTA issues tcgen05.mma.cta_group::2
// (M 256, N 256) and each SM's tensor core accumulates its 128 rows x 256 columns in its own TMEM. A third less
// operand traffic from L2 per FLOP than the one-SM tile, and a deeper ring in the same shared memory.
//   full[s]   (even CTA's copy) one arrive + the bytes of both CTAs' loads
//   empty[s]  (each CTA's copy) the MMA thread's commit reaches both copies
//   tfull[a]  (each CTA's copy) likewise; tempty[a] (even CTA's copy) collects the 16 epilogue warps of both CTAs
// EPI selects the epilogue compiled in (kernels of their own, so the plain products keep their registers and their ring):
// 0 plain; 1 SwiGLU backward (SwigluGrad): two staging boxes per epilogue warp and a five-stage ring; 2 SwiGLU forward (SwigluForward).
constexpr int BM2 = 256, BN2 = 256;
constexpr int A2_TILE_BYTES = 128 * BK * 2, B2_TILE_BYTES = 128 * BK * 2, STAGE2_BYTES = A2_TILE_BYTES + B2_TILE_BYTES;
// The backward epilogue has two staging boxes per warp (a and u come in through them, g_a and g_u leave through them) and a
// five-stage ring; the ring's depth matters more than anything else here: with three stages the main loop alone took 12.2k cycles per
// tile of 12 k-blocks against about 7.5k with six (a TMA load from L2 takes 2-3k cycles; a stage is consumed in 512).
__host__ __device__ constexpr int stages2(int epi) { return epi == 1 ? 5 : 6; }
__host__ __device__ constexpr int epi_boxes(int epi) { return epi == 1 ? 2 : 1; }
__host__ __device__ constexpr int smem2_bytes(int epi) { return stages2(epi) * STAGE2_BYTES + 1024 + epi_boxes(epi) * EPI_STAGE_BYTES + 256; }
static_assert(smem2_bytes(0) <= 232448 && smem2_bytes(1) <= 232448 && smem2_bytes(2) <= 232448, "shared memory per CTA");
static_assert(8 * (2 * stages2(0) + 5) <= 256, "barrier area");

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c,
                const __grid_constant__ CUtensorMap tmap_m, const TcArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;               // the same offset in both CTAs (same kernel, same layout)
  constexpr int STAGES2 = stages2(EPI);
  const uint32_t epi_base = tiles_base + STAGES2 * STAGE2_BYTES;
  const uint32_t bar_base = epi_base + epi_boxes(EPI) * EPI_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES2 + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES2 + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES2 + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bar_base - raw) + 8 * (2 * STAGES2 + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_ptr = smem_raw + (epi_base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                          // 0: the CTA that issues the MMAs
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_m = (args.m + BM2 - 1) / BM2, tiles_n = (args.n + BN2 - 1) / BN2;
  const int units_per_matrix = tiles_m * tiles_n * args.splits, units = units_per_matrix * args.batch;
  const int kblocks_total = (args.k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 2 * EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the same warp of both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  cluster_sync_all();                                               // both CTAs' barriers exist before anyone arrives on a peer's
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched with programmatic stream serialization: everything above (barriers, tensor memory) may run while the kernel before this
  // one in the stream is still finishing on other SMs; nothing below touches global memory before that kernel is complete. The
  // trigger lets the kernel after this one do the same with its own prologue once this one's CTAs start leaving.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (each CTA loads its own halves)
    if (lane == 0) {
      uint32_t it = 0;
      for (int u = pair; u < units; u += npairs) {
        const int bz = u / units_per_matrix, ub = u - bz * units_per_matrix;
        const int split = ub % args.splits, tile = ub / args.splits;
        const int tm = args.tiles_n_fast ? tile / tiles_n : tile % tiles_m, tn = args.tiles_n_fast ? tile % tiles_n : tile / tiles_m;
        const int kb0 = split * args.kblocks_per_split, kb1 = min(kblocks_total, kb0 + args.kblocks_per_split);
        // SwiGLU forward: the even CTA brings 128 gate columns and the odd one the 128 up columns that go with them
        const int row0 = tm * BM2 + (int)rank * 128, col0 = EPI == 2 ? (int)rank * args.sw_f + tn * 128 : tn * BN2 + (int)rank * 128;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES2;
          if (!mbar_wait(empty_bar(s), ((it / STAGES2) & 1) ^ 1, args.fault, abort_flag)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE2_BYTES);
          const uint32_t a_dst = tiles_base + s * STAGE2_BYTES, b_dst = a_dst + A2_TILE_BYTES;
          if (!args.a_mn_major) tma_load_3d_pair(a_dst, &tmap_a, full_bar(s), kb * BK, row0, bz);
          else for (int j = 0; j < 2; ++j) tma_load_3d_pair(a_dst + j * (BK * 128), &tmap_a, full_bar(s), row0 + j * 64, kb * BK, bz);
          if (!args.b_mn_major) tma_load_3d_pair(b_dst, &tmap_b, full_bar(s), kb * BK, col0, bz);
          else for (int j = 0; j < 2; ++j) tma_load_3d_pair(b_dst + j * (BK * 128), &tmap_b, full_bar(s), col0 + j * 64, kb * BK, bz);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(BM2, BN2, args.a_mn_major, args.b_mn_major);
      const uint32_t a_lbo = args.a_mn_major ? BK * 128 : 0, b_lbo = args.b_mn_major ? BK * 128 : 0;
      const uint32_t a_step = args.a_mn_major ? 2048 : 32, b_step = args.b_mn_major ? 2048 : 32;
      uint32_t it = 0, local = 0;
      for (int u = pair; u < units; u += npairs, ++local) {
        const int split = (u % units_per_matrix) % args.splits;
        const int kb0 = split * args.kblocks_per_split, kb1 = min(kblocks_total, kb0 + args.kblocks_per_split);
        const int acc = local & 1;
        if (!mbar_wait(tempty_bar(acc), ((local >> 1) & 1) ^ 1, args.fault, abort_flag)) break;
        fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN2;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES2;
          if (!mbar_wait(full_bar(s), (it / STAGES2) & 1, args.fault, abort_flag)) { ok = false; break; }
          fence_after();
          const uint32_t a_src = tiles_base + s * STAGE2_BYTES, b_src = a_src + A2_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_pair(tmem_d, make_desc(a_src + kk * a_step, a_lbo, 1024), make_desc(b_src + kk * b_step, b_lbo, 1024), idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          umma_commit_pair(empty_bar(s));      // frees the stage in both CTAs when these MMAs have read it
        }
        if (!ok) break;
        umma_commit_pair(tfull_bar(acc));      // accumulators complete in both CTAs
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9 of both CTAs)
    const int quarter = warp & 3;
    const int col_begin = ((warp - 2) >> 2) * (BN2 / 2), col_end = col_begin + BN2 / 2;
    uint8_t* stage_bytes = epi_ptr + (warp - 2) * epi_boxes(EPI) * EPI_WARP_BYTES;
    const uint32_t stage_addr = epi_base + (warp - 2) * epi_boxes(EPI) * EPI_WARP_BYTES;
    auto unit_tile = [&](int u, int* tm, int* tn, int* split, int* bz) {
      *bz = u / units_per_matrix;
      const int ub = u - *bz * units_per_matrix, tile = ub / args.splits;
      *split = ub % args.splits;
      *tm = args.tiles_n_fast ? tile / tiles_n : tile % tiles_m; *tn = args.tiles_n_fast ? tile % tiles_n : tile / tiles_m;
    };
    // EPI 1: a and u for rows [32 quarter, +32) x 64 columns of a step are read one step ahead with plain 16-byte loads, eight lanes
    // to a row (whole 128-byte lines; a lane per row would touch 32 lines per instruction and bind on L1 wavefronts), and wait in
    // registers: the first step's while the unit's products still run, the next one's while this one is worked on. Out-of-range
    // rows and columns read as zero and are clipped on the way out.
    uint4 la[8], lu[8];
    auto fetch_inputs = [&](int u, int c0) {
      int tm, tn, split, bz;
      unit_tile(u, &tm, &tn, &split, &bz);
      const int x = tn * BN2 + c0, y = tm * BM2 + (int)rank * 128 + quarter * 32 + (lane >> 3);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const bool in = y + 4 * k < args.m && x < args.n;
        const uint4* p = reinterpret_cast<const uint4*>(args.sw_au + (in ? (int64_t)(y + 4 * k) * args.sw_ld + x : 0)) + (lane & 7);
        la[k] = make_uint4(0, 0, 0, 0); lu[k] = make_uint4(0, 0, 0, 0);
        if (in) { la[k] = __ldg(p); lu[k] = __ldg(p + args.n / 8); }
      }
    };
    if (EPI == 1 && pair < units) fetch_inputs(pair, col_begin);
    uint32_t local = 0;
    for (int u = pair; u < units; u += npairs, ++local) {
      int tm, tn, split, bz;
      unit_tile(u, &tm, &tn, &split, &bz);
      const int acc = local & 1;
      if (!mbar_wait(tfull_bar(acc), (local >> 1) & 1, args.fault, abort_flag)) break;
      fence_after();
      const int row_base = tm * BM2 + (int)rank * 128 + quarter * 32;
      const uint32_t tsrc = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN2;
      if constexpr (EPI == 2) drain_swiglu_forward(args, tmap_c, tmap_m, tsrc, row_base, tn * 128, bz, lane, (warp - 2) >> 2, stage_bytes, stage_addr);
      else if constexpr (EPI == 1) {
#pragma unroll 1
        for (int c0 = col_begin; c0 < col_end; c0 += 64) {
          if (lane == 0) bulk_wait_read();       // the previous step's two boxes have left the staging rows
          __syncwarp();
          // the fetched 16-byte pieces go to their rows' places in the boxes (row 4 k + lane / 8, piece lane % 8): lane = row from here on
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int row = 4 * k + (lane >> 3), off = row * 128 + (((lane & 7) ^ (row & 7)) << 4);
            *reinterpret_cast<uint4*>(stage_bytes + off) = la[k];
            *reinterpret_cast<uint4*>(stage_bytes + EPI_WARP_BYTES + off) = lu[k];
          }
          __syncwarp();
          if (c0 + 64 < col_end) fetch_inputs(u, c0 + 64);
          else if (u + npairs < units) fetch_inputs(u + npairs, col_begin);
          drain_swiglu_backward(args, tmap_c, tsrc, row_base, tn * BN2 + c0, c0, bz, lane, stage_bytes, stage_addr);
        }
      }
      else drain_tile(args, tmap_c, tsrc, row_base, tn * BN2, split, bz, lane, col_begin, col_end, stage_bytes, stage_addr);
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_even_cta(tempty_bar(acc));
    }
    if (args.tma_store && lane == 0) bulk_wait_all();
  }
  // Teardown: neither CTA may leave while its partner can still reach its shared memory, barriers or tensor memory.
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Sum the split-K partials in split order, then apply alpha / residual / accumulate. n is a multiple of 8, so rows split
// into whole float4 groups.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, void* c, int c_bf16, int64_t ldc, int m, int n, float alpha,
                                     int accumulate, const float* __restrict__ residual) {
  pdl_trigger();
  const int n4 = n >> 2;
  const int64_t total4 = (int64_t)m * n4, plane4 = total4;
  const float4* part4 = reinterpret_cast<const float4*>(partial);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 acc = part4[i];
    for (int s = 1; s < splits; ++s) { const float4 t = part4[(int64_t)s * plane4 + i]; acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w; }
    const int64_t row = i / n4, o = row * ldc + (i - row * n4) * 4;
    float4 v = make_float4(alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w);
    if (residual) { const float4 t = *reinterpret_cast<const float4*>(residual + o); v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w; }
    if (c_bf16) {
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(c) + o) = make_uint2(pack2_bf16(v.x, v.y), pack2_bf16(v.z, v.w));
    } else {
      float* dst = reinterpret_cast<float*>(c) + o;
      if (accumulate) { const float4 t = *reinterpret_cast<const float4*>(dst); v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w; }
      *reinterpret_cast<float4*>(dst) = v;
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// inner = extent of the contiguous axis, outer = the other one, ld = elements between outer steps; `batch` matrices
// `batch_stride` elements apart form the third dimension (1 and any stride for a single matrix).
ojc_status make_tmap(ojc_backend* be, const char* op, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                     uint32_t box_outer, bool f32 = false, uint64_t batch = 1, uint64_t batch_stride = 0) {
  if (!be->tmap_encode) return ojc_fail(OJC_ERR_BACKEND, op, "cuTensorMapEncodeTiled is not available from this driver");
  const uint64_t es = f32 ? 4 : 2;
  if (batch <= 1) { batch = 1; batch_stride = ld * outer; }
  cuuint64_t gdim[3] = {inner, outer, batch};
  cuuint64_t gstride[2] = {ld * es, batch_stride * es};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estride[3] = {1, 1, 1};
  CUresult r = ((EncodeTiledFn)be->tmap_encode)(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), gdim, gstride, box, estride,
                                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ojc_fail(OJC_ERR_BACKEND, op, "cuTensorMapEncodeTiled refused the operand (code " + std::to_string((int)r) + ")");
  return OJC_OK;
}

bool operand_ok(const GemmOperand& o, bool is_a, int* mn_major, int64_t* ld) {
  if (o.dtype != OJC_BF16 || (reinterpret_cast<uintptr_t>(o.ptr) & 15)) return false;
  // A(i,k): K-major when cs == 1; B(k,j): K-major when rs == 1.
  const int64_t k_stride = is_a ? o.cs : o.rs, mn_stride = is_a ? o.rs : o.cs;
  if (k_stride == 1) { *mn_major = 0; *ld = mn_stride; }
  else if (mn_stride == 1) { *mn_major = 1; *ld = k_stride; }
  else return false;
  return *ld % 8 == 0 && *ld > 0;
}

}  // namespace

namespace {
// How many CTA pairs of the two-SM kernel the device runs at once (0: the cluster launch is not available); found once per device.
ojc_status two_sm_pairs(ojc_backend* be, const char* op, int* pairs) {
  static PerDeviceInt max_pairs_of(-1);
  int& max_pairs = max_pairs_of[be->device];
  if (max_pairs < 0) {
    OJC_CUDA(be, cudaFuncSetAttribute(gemm_tc2_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2_bytes(0)), op);
    OJC_CUDA(be, cudaFuncSetAttribute(gemm_tc2_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2_bytes(1)), op);
    OJC_CUDA(be, cudaFuncSetAttribute(gemm_tc2_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2_bytes(2)), op);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension; attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3((unsigned)(be->sm_count & ~1)); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = smem2_bytes(1); cfg.attrs = attr; cfg.numAttrs = 1;
    int n_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&n_clusters, gemm_tc2_kernel<1>, &cfg) != cudaSuccess) { cudaGetLastError(); n_clusters = 0; }
    max_pairs = n_clusters;
  }
  *pairs = max_pairs;
  return OJC_OK;
}
}  // namespace

bool gemm_tc_swiglu_backward_eligible(ojc_backend* be, int64_t m, int64_t n) {
  int pairs = 0;
  if (two_sm_pairs(be, "linear_backward", &pairs) != OJC_OK || pairs <= 0) return false;
  return m >= BM2 && n >= BN2 && n % 64 == 0;
}
bool gemm_tc_swiglu_forward_eligible(ojc_backend* be, int64_t m, int64_t n, int64_t ldm, const void* mptr) {
  int pairs = 0;
  if (two_sm_pairs(be, "linear_forward", &pairs) != OJC_OK || pairs <= 0) return false;
  return m >= BM2 && n >= BN2 && n % 256 == 0 && ldm % 8 == 0 && ldm >= n / 2 && (reinterpret_cast<uintptr_t>(mptr) & 15) == 0;
}

bool gemm_tc_eligible(const GemmOperand& a, const GemmOperand& b, const void* c, int32_t c_dtype, int64_t ldc, int64_t m, int64_t n, int64_t k) {
  int amn, bmn; int64_t lda, ldb;
  if (!operand_ok(a, true, &amn, &lda) || !operand_ok(b, false, &bmn, &ldb)) return false;
  if (m < 1 || n < 1 || k < 1 || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return false;
  if (n % 8 != 0 || ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(c) & 15)) return false;
  // An MN-major operand's contiguous extent is its TMA inner dimension: keep whole 16-byte rows.
  if (amn && m % 8 != 0) return false;
  if (bmn && n % 8 != 0) return false;
  if (!amn && k % 8 != 0) return false;
  if (!bmn && k % 8 != 0) return false;
  return c_dtype == OJC_F32 || c_dtype == OJC_BF16;
}

ojc_status gemm_tc(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                   int64_t n, int64_t k, float alpha, bool accumulate, const float* residual) {
  return gemm_tc_batched(be, op, a, b, c, c_dtype, ldc, m, n, k, 1, 0, 0, 0, alpha, accumulate, residual);
}

// `batch` independent products of the same shape; matrix i of A / B / C starts a_bs / b_bs / c_bs elements after matrix i - 1.
ojc_status gemm_tc_batched(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                           int64_t n, int64_t k, int64_t batch, int64_t a_bs, int64_t b_bs, int64_t c_bs, float alpha, bool accumulate, const float* residual,
                           const NsCombine* combine, bool allow_split, const SwigluGrad* swiglu_grad, const SwigluForward* swiglu_fwd) {
  if (swiglu_fwd && !gemm_tc_swiglu_forward_eligible(be, m, n, swiglu_fwd->ldm, swiglu_fwd->m))
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "the SwiGLU forward epilogue needs two-SM tiles (256 rows or more), a hidden width that is a multiple of 128 and an aligned bf16 m");
  if (swiglu_fwd && (c_dtype != OJC_BF16 || alpha != 1.0f || accumulate || residual || combine || swiglu_grad || batch != 1))
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "the SwiGLU forward epilogue needs a single bf16 product, alpha 1, no accumulation");
  if (swiglu_fwd) allow_split = false;
  if (swiglu_grad && !gemm_tc_swiglu_backward_eligible(be, m, n))
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "the SwiGLU backward epilogue needs two-SM tiles (256 rows and 256 columns or more) and a width that is a multiple of 64");
  if (swiglu_grad && (c_dtype != OJC_BF16 || alpha != 1.0f || accumulate || residual || combine || batch != 1 || n % 64 != 0 || swiglu_grad->ld % 8 != 0 ||
                      swiglu_grad->ld < 2 * n || ldc < 2 * n || ((uintptr_t)swiglu_grad->au & 15) != 0))
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "the SwiGLU epilogue needs bf16 (a | u) rows and output rows at least 2 n wide, n a multiple of 64, alpha 1, no accumulation");
  if (swiglu_grad) allow_split = false;
  if (!gemm_tc_eligible(a, b, c, c_dtype, ldc, m, n, k)) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "operands break the tensor-core kernel's alignment rules");
  if (combine && (c_dtype != OJC_BF16 || alpha != 1.0f || accumulate || residual || combine->src_ld % 8 != 0 || combine->src_bs % 8 != 0 || ((uintptr_t)combine->src & 15) != 0 || n < 64))
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "the combine epilogue needs a bf16 output, alpha 1, no accumulation and an aligned source");
  if (accumulate && c_dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "accumulation needs an F32 output");
  if (batch < 1 || batch > 65535) return ojc_fail(OJC_ERR_SHAPE, op, "batch count out of range");
  if (batch > 1 && (a_bs % 8 != 0 || b_bs % 8 != 0 || c_bs % 8 != 0 || residual || n < 64))
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "a batched product needs 16-byte aligned matrix strides, no residual operand and at least 64 output columns");
  int amn, bmn; int64_t lda, ldb;
  operand_ok(a, true, &amn, &lda); operand_ok(b, false, &bmn, &ldb);
  // Two-SM tiles (256 x 256 per CTA pair) whenever the output is at least one such tile; the one-SM kernel keeps the rest.
  int max_pairs = 0;
  OJC_TRY(two_sm_pairs(be, op, &max_pairs));
  const bool two_sm = max_pairs > 0 && m >= BM2 && n >= BN2;
  const int tile_m = two_sm ? BM2 : BM, tile_n = two_sm ? BN2 : BN, workers = two_sm ? max_pairs : be->sm_count;
  CUtensorMap ta, tb;
  if (!amn) OJC_TRY(make_tmap(be, op, &ta, a.ptr, (uint64_t)k, (uint64_t)m, (uint64_t)lda, 64, 128, false, batch, a_bs));
  else OJC_TRY(make_tmap(be, op, &ta, a.ptr, (uint64_t)m, (uint64_t)k, (uint64_t)lda, 64, BK, false, batch, a_bs));
  if (!bmn) OJC_TRY(make_tmap(be, op, &tb, b.ptr, (uint64_t)k, (uint64_t)n, (uint64_t)ldb, 64, two_sm ? 128 : BN, false, batch, b_bs));
  else OJC_TRY(make_tmap(be, op, &tb, b.ptr, (uint64_t)n, (uint64_t)k, (uint64_t)ldb, 64, BK, false, batch, b_bs));

  static PerDeviceFlag attr_set_of;
  bool& attr_set = attr_set_of[be->device];
  if (!attr_set) {
    OJC_CUDA(be, cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), op);
    attr_set = true;
  }
  const int tiles = (int)(((m + tile_m - 1) / tile_m) * ((n + tile_n - 1) / tile_n) * batch);   // units before any split
  const int kblocks = (int)((k + BK - 1) / BK);
  // Split the reduction axis when the output tiles alone leave SMs idle: estimate each split count's time as the math at
  // the wave efficiency its units reach plus the partial round trip through memory, and take the cheapest (each split
  // keeps at least 8 k-blocks).
  int splits = 1;
  if (kblocks >= 16 && batch == 1 && !combine && allow_split) {
    const double flops = 2.0 * (double)m * (double)n * (double)k;
    double best = 1e30;
    for (int sp = 1; sp <= 16 && kblocks / sp >= 8; ++sp) {
      const int units = tiles * sp, waves = (units + workers - 1) / workers;
      const double eff = (double)units / ((double)waves * workers);
      const double t = flops / (1.5e15 * eff) + (sp > 1 ? (double)sp * (double)m * (double)n * 8.0 / 6.0e12 : 0.0);
      if (t < best * 0.97) { best = t; splits = sp; }
    }
  }
  int per = (kblocks + splits - 1) / splits;
  splits = (kblocks + per - 1) / per;
  TcArgs args;
  args.c = c; args.c_bf16 = c_dtype == OJC_BF16; args.ldc = ldc;
  args.m = (int)m; args.n = (int)n; args.k = (int)k;
  args.a_mn_major = amn; args.b_mn_major = bmn;
  args.alpha = alpha; args.accumulate = accumulate ? 1 : 0; args.residual = residual;
  args.splits = splits; args.kblocks_per_split = per; args.partial = nullptr; args.fault = be->fault_dev; args.batch = (int)batch;
  args.ns_src = combine ? (const bf16*)combine->src : nullptr; args.ns_ld = combine ? combine->src_ld : 0; args.ns_bs = combine ? combine->src_bs : 0;
  args.ns_src_mul = combine ? combine->src_mul : 0.0f; args.ns_acc_mul = combine ? combine->acc_mul : 0.0f;
  args.sw_au = swiglu_grad ? (const bf16*)swiglu_grad->au : nullptr; args.sw_ld = swiglu_grad ? swiglu_grad->ld : 0;
  args.sw_f = swiglu_fwd ? (int)(n / 2) : 0;
  if (splits > 1) {
    void* ws = nullptr;
    OJC_TRY(ojc_scratch(be, (uint64_t)splits * m * n * 4, &ws));
    args.partial = (float*)ws;
  }
  // Neighbouring CTAs work on neighbouring tiles: walk the shorter tile axis fastest so the long operand streams from HBM once.
  args.tiles_n_fast = ((n + tile_n - 1) / tile_n) <= ((m + tile_m - 1) / tile_m) ? 1 : 0;
  args.tma_store = (!residual && (splits == 1 || m % 32 == 0) && n >= 64) ? 1 : 0;   // narrower outputs than a store box take the row path
  CUtensorMap tc = ta;   // unused unless tma_store
  if (args.tma_store) {
    if (splits > 1) OJC_TRY(make_tmap(be, op, &tc, args.partial, (uint64_t)n, (uint64_t)splits * (uint64_t)m, (uint64_t)n, 32, 32, true));
    else if (args.c_bf16) OJC_TRY(make_tmap(be, op, &tc, c, (uint64_t)(swiglu_grad ? 2 * n : n), (uint64_t)m, (uint64_t)ldc, 64, 32, false, batch, c_bs));
    else OJC_TRY(make_tmap(be, op, &tc, c, (uint64_t)n, (uint64_t)m, (uint64_t)ldc, 32, 32, true, batch, c_bs));
  } else if (batch > 1) {
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, "a batched product needs the tile-store epilogue");
  }
  CUtensorMap tm = tc;   // the SwiGLU forward epilogue's third output
  if (swiglu_fwd) OJC_TRY(make_tmap(be, op, &tm, swiglu_fwd->m, (uint64_t)(n / 2), (uint64_t)m, (uint64_t)swiglu_fwd->ldm, 64, 32));
  int grid = tiles * splits < workers ? tiles * splits : workers;
  if (two_sm) grid *= 2;
  ojc_backend::GemmSample sample{nullptr, nullptr, 2.0 * (double)m * (double)n * (double)k * (double)batch, swiglu_grad != nullptr || swiglu_fwd != nullptr};
  if (be->profile_gemm) {
    if (!be->event_pool.empty()) { sample.start = be->event_pool.back().first; sample.stop = be->event_pool.back().second; be->event_pool.pop_back(); }
    else { OJC_CUDA(be, cudaEventCreate(&sample.start), op); OJC_CUDA(be, cudaEventCreate(&sample.stop), op); }
    OJC_CUDA(be, cudaEventRecord(sample.start, be->stream), op);
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(NUM_THREADS); cfg.stream = be->stream; cfg.attrs = pdl; cfg.numAttrs = 1;
  cudaError_t launched;
  if (swiglu_fwd) { cfg.dynamicSmemBytes = smem2_bytes(2); launched = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<2>, ta, tb, tc, tm, args); }
  else if (swiglu_grad) { cfg.dynamicSmemBytes = smem2_bytes(1); launched = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<1>, ta, tb, tc, tm, args); }
  else if (two_sm) { cfg.dynamicSmemBytes = smem2_bytes(0); launched = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<0>, ta, tb, tc, tm, args); }
  else { cfg.dynamicSmemBytes = SMEM_BYTES; launched = cudaLaunchKernelEx(&cfg, gemm_tc_kernel, ta, tb, tc, args); }
  OJC_CUDA(be, launched, op);
  OJC_LAUNCHED(be, op);
  if (be->profile_gemm) {
    OJC_CUDA(be, cudaEventRecord(sample.stop, be->stream), op);
    be->gemm_samples.push_back(sample);
  }
  if (splits > 1) {
    splitk_reduce_kernel<<<elementwise_grid(be, m * n / 4, 256), 256, 0, be->stream>>>(args.partial, splits, c, args.c_bf16, ldc, (int)m, (int)n, alpha,
                                                                                   args.accumulate, residual);
    OJC_LAUNCHED(be, op);
  }
  return OJC_OK;
}

ojc_status gemm_auto(ojc_backend* be, const char* op, const GemmOperand& a, const GemmOperand& b, void* c, int32_t c_dtype, int64_t ldc, int64_t m,
                     int64_t n, int64_t k, float alpha, bool accumulate, const float* residual) {
  if (a.dtype == OJC_BF16 && b.dtype == OJC_BF16 && gemm_tc_eligible(a, b, c, c_dtype, ldc, m, n, k) && !(accumulate && c_dtype != OJC_F32))
    return gemm_tc(be, op, a, b, c, c_dtype, ldc, m, n, k, alpha, accumulate, residual);
  return gemm_f32(be, op, a, b, c, c_dtype, ldc, m, n, k, alpha, accumulate, residual);
}

// ------------------------------------------------------------------------------------------------ bounded-wait self-test
namespace {
// The wait every tensor-pipeline role uses, on a barrier nothing ever arrives on, with a caller-chosen limit: the wait must give
// up, raise the wait fault and let the CTA leave in order (no trap, no spin past the limit).
__global__ void bounded_wait_selftest_kernel(long long limit_cycles, uint32_t* fault, int* gave_up) {
  __shared__ __align__(8) uint64_t barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) { tc::mbar_init(tc::smem_u32(&barrier), 1); abort_flag = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  __syncthreads();
  const bool ok = tc::mbar_wait_limit(tc::smem_u32(&barrier), 0, fault, &abort_flag, limit_cycles);
  if (!ok) atomicAdd(gave_up, 1);
  __syncthreads();
}
}  // namespace

extern "C" ojc_status ojc_selftest_bounded_wait(ojc_backend* be, uint64_t limit_cycles, int32_t* threads_that_gave_up) {
  const char* op = "selftest_bounded_wait";
  OJC_ALIVE(be, op);
  if (limit_cycles == 0 || limit_cycles > 200000000ull) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "the limit must be between 1 and 2e8 cycles (about a tenth of a second)");
  void* counter = nullptr;
  OJC_TRY(ojc_alloc(be, 4, &counter));
  ojc_status st = ojc_fill_zero(be, counter, 4);
  if (st == OJC_OK) {
    bounded_wait_selftest_kernel<<<1, 64, 0, be->stream>>>((long long)limit_cycles, be->fault_dev, (int*)counter);
    st = ojc_cuda_check(be, cudaGetLastError(), op);
  }
  int32_t host = 0;
  ojc_status rd = st == OJC_OK ? ojc_download(be, &host, counter, 4) : st;    // the sync point: reports the wait fault as WaitTimeout
  if (threads_that_gave_up) *threads_that_gave_up = host;
  ojc_free(be, counter);
  return rd;
}
