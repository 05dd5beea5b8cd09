// bf16 x bf16 -> f32 GEMM on the Blackwell tensor cores (sm_100a).
//
//   C[m,n] = alpha * A[m,k] . B[k,n]  (+ residual)  (+ C)
//
// A persistent kernel, one CTA per SM, ten warps with fixed roles:
//   warp 0   TMA producer: cp.async.bulk.tensor loads of A and B tiles (128-byte
//            swizzle, no cluster multicast) into a 4-stage shared-memory ring
//   warp 1   allocates tensor memory and issues tcgen05.mma (one thread);
//            accumulators live in TMEM, double-buffered (2 x 256 columns) so
//            the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2-9  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM
//            lanes and half of the columns), scale / add residual / accumulate,
//            store f32 (through padded staging rows, coalesced) or bf16
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

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2, B_TILE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int STAGE_LD = 20;                      // floats per staged epilogue row (16 + 4 of padding)
constexpr int EPI_STAGE_BYTES = 8 * 32 * STAGE_LD * 4;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ + EPI_STAGE_BYTES;
#ifndef OJC_DIRECT_BF16
#define OJC_DIRECT_BF16 1
#endif
constexpr int EPI_WARPS = 8;                     // two warps per TMEM lane quarter, each draining half of the columns
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
static_assert(SMEM_BYTES <= 232448, "shared memory per CTA");
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;

struct TcArgs {
  void* c; int c_bf16; int64_t ldc;
  int m, n, k;
  int a_mn_major, b_mn_major;
  float alpha; int accumulate; const float* residual;
  int splits, kblocks_per_split;
  float* partial;           // [splits][m][n] when splits > 1
  uint32_t* fault;
  int epi_warps;            // 4: bf16 rows stored directly by one warp per lane quarter; 8: staged f32 path, two warps per quarter
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t global_ns() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false (and the fault word raised) when the limit runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t* fault, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  // the SM cycle counter bounds the wait (cheap to read; at most ~2 GHz, so the limit is at least two seconds)
  const long long start = clock64();
  while (true) {
#pragma unroll 1
    for (int spin = 0; spin < 32; ++spin) if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > WAIT_LIMIT_CYCLES) { *abort_flag = 1; raise_fault(fault, OP_GEMM_WAIT); return false; }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor (128-byte swizzle). Bits: [0,14) start >> 4, [16,30) leading byte offset >> 4,
// [32,46) stride byte offset >> 4, [46,48) version = 1, [61,64) layout type = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor, kind::f16: D f32 (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), transpose bits 15/16
// for MN-major operands, N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__device__ __forceinline__ uint32_t make_idesc(int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
      "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const TcArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;               // 128-byte swizzle atoms repeat every 1024 bytes
  const uint32_t bar_base = tiles_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bar_base - raw) + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stage_all = reinterpret_cast<float*>(smem_raw + (bar_base - raw) + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (args.m + BM - 1) / BM, tiles_n = (args.n + BN - 1) / BN;
  const int units = tiles_m * tiles_n * args.splits;
  const int kblocks_total = (args.k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), args.epi_warps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x) {
        const int split = u % args.splits, tile = u / args.splits;
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        const int kb0 = split * args.kblocks_per_split, kb1 = min(kblocks_total, kb0 + args.kblocks_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, args.fault, abort_flag)) break;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const uint32_t a_dst = tiles_base + s * STAGE_BYTES, b_dst = a_dst + A_TILE_BYTES;
          if (!args.a_mn_major) tma_load_2d(a_dst, &tmap_a, full_bar(s), kb * BK, tm * BM);
          else for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmap_a, full_bar(s), tm * BM + j * 64, kb * BK);
          if (!args.b_mn_major) tma_load_2d(b_dst, &tmap_b, full_bar(s), kb * BK, tn * BN);
          else for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmap_b, full_bar(s), tn * BN + j * 64, kb * BK);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(args.a_mn_major, args.b_mn_major);
      // K-major: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO), one MMA step = 32 bytes along the row.
      // MN-major: 64-element column blocks BK*128 bytes apart (LBO), 8-row K groups 1024 bytes apart (SBO), one MMA step = 2 groups.
      const uint32_t a_lbo = args.a_mn_major ? BK * 128 : 0, b_lbo = args.b_mn_major ? BK * 128 : 0;
      const uint32_t a_step = args.a_mn_major ? 2048 : 32, b_step = args.b_mn_major ? 2048 : 32;
      uint32_t it = 0, local = 0;
      for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x, ++local) {
        const int split = u % args.splits;
        const int kb0 = split * args.kblocks_per_split, kb1 = min(kblocks_total, kb0 + args.kblocks_per_split);
        const int acc = local & 1;
        if (!mbar_wait(tempty_bar(acc), ((local >> 1) & 1) ^ 1, args.fault, abort_flag)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar(s), (it / STAGES) & 1, args.fault, abort_flag)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
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
  } else if (warp < 2 + args.epi_warps) {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;         // TMEM lanes [32 * quarter, +32) are this warp's
    float* stage = stage_all + (warp - 2) * 32 * STAGE_LD;
    const int col_begin = args.epi_warps == 4 ? 0 : ((warp - 2) >> 2) * (BN / 2), col_end = args.epi_warps == 4 ? BN : col_begin + BN / 2;
    uint32_t local = 0;
    for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x, ++local) {
      const int split = u % args.splits, tile = u / args.splits;
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int acc = local & 1;
      if (!mbar_wait(tfull_bar(acc), (local >> 1) & 1, args.fault, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row_base = tm * BM + quarter * 32;
#pragma unroll 1
      for (int c0 = col_begin; c0 < col_end; c0 += 32) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col0 = tn * BN + c0;
        if (OJC_DIRECT_BF16 && args.c_bf16 && args.splits == 1 && !args.residual) {
          // bf16 output: each thread writes 64 contiguous bytes of its own row (two full 32-byte sectors)
          const int row = row_base + lane;
          if (row < args.m && col0 < args.n) {
            bf16* dst = reinterpret_cast<bf16*>(args.c) + (int64_t)row * args.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j >= args.n) break;
              uint4 t;
              t.x = (uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j])) | ((uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j + 1])) << 16);
              t.y = (uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j + 2])) | ((uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j + 3])) << 16);
              t.z = (uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j + 4])) | ((uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j + 5])) << 16);
              t.w = (uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j + 6])) | ((uint32_t)f32_to_bf16_bits(args.alpha * __uint_as_float(r[j + 7])) << 16);
              *reinterpret_cast<uint4*>(dst + j) = t;
            }
          }
          continue;
        }
        // f32 output: each thread holds one accumulator row; pass the block, 16 columns at a time, through this warp's
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
              uint2 t;
              t.x = (uint32_t)f32_to_bf16_bits(v.x) | ((uint32_t)f32_to_bf16_bits(v.y) << 16);
              t.y = (uint32_t)f32_to_bf16_bits(v.z) | ((uint32_t)f32_to_bf16_bits(v.w) << 16);
              *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(args.c) + o) = t;
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }
  // Teardown: on an aborted run give copies in flight time to land before the shared memory goes away.
  if (*abort_flag) __nanosleep(200000);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Sum the split-K partials in split order, then apply alpha / residual / accumulate.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, void* c, int c_bf16, int64_t ldc, int m, int n, float alpha,
                                     int accumulate, const float* __restrict__ residual) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)m * n, stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    float acc = 0.0f;
    for (int s = 0; s < splits; ++s) acc += partial[(int64_t)s * total + i];
    const int64_t o = (i / n) * ldc + (i % n);
    float v = alpha * acc;
    if (residual) v += residual[o];
    if (c_bf16) { reinterpret_cast<bf16*>(c)[o] = __float2bfloat16_rn(v); }
    else { float* dst = reinterpret_cast<float*>(c) + o; *dst = accumulate ? *dst + v : v; }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// inner = extent of the contiguous axis, outer = the other one, ld = elements between outer steps.
ojc_status make_tmap(ojc_backend* be, const char* op, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                     uint32_t box_outer) {
  if (!be->tmap_encode) return ojc_fail(OJC_ERR_BACKEND, op, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estride[2] = {1, 1};
  CUresult r = ((EncodeTiledFn)be->tmap_encode)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
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
  if (!gemm_tc_eligible(a, b, c, c_dtype, ldc, m, n, k)) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "operands break the tensor-core kernel's alignment rules");
  if (accumulate && c_dtype != OJC_F32) return ojc_fail(OJC_ERR_DTYPE, op, "accumulation needs an F32 output");
  int amn, bmn; int64_t lda, ldb;
  operand_ok(a, true, &amn, &lda); operand_ok(b, false, &bmn, &ldb);
  CUtensorMap ta, tb;
  if (!amn) OJC_TRY(make_tmap(be, op, &ta, a.ptr, (uint64_t)k, (uint64_t)m, (uint64_t)lda, 64, BM));
  else OJC_TRY(make_tmap(be, op, &ta, a.ptr, (uint64_t)m, (uint64_t)k, (uint64_t)lda, 64, BK));
  if (!bmn) OJC_TRY(make_tmap(be, op, &tb, b.ptr, (uint64_t)k, (uint64_t)n, (uint64_t)ldb, 64, BN));
  else OJC_TRY(make_tmap(be, op, &tb, b.ptr, (uint64_t)n, (uint64_t)k, (uint64_t)ldb, 64, BK));

  static bool attr_set = false;
  if (!attr_set) {
    OJC_CUDA(be, cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), op);
    attr_set = true;
  }
  const int tiles = (int)(((m + BM - 1) / BM) * ((n + BN - 1) / BN));
  const int kblocks = (int)((k + BK - 1) / BK);
  int splits = 1;
  if (tiles * 2 <= be->sm_count && kblocks >= 16) {
    splits = be->sm_count / tiles;
    if (splits > kblocks / 8) splits = kblocks / 8;
    if (splits < 1) splits = 1;
  }
  int per = (kblocks + splits - 1) / splits;
  splits = (kblocks + per - 1) / per;
  TcArgs args;
  args.c = c; args.c_bf16 = c_dtype == OJC_BF16; args.ldc = ldc;
  args.m = (int)m; args.n = (int)n; args.k = (int)k;
  args.a_mn_major = amn; args.b_mn_major = bmn;
  args.alpha = alpha; args.accumulate = accumulate ? 1 : 0; args.residual = residual;
  args.splits = splits; args.kblocks_per_split = per; args.partial = nullptr; args.fault = be->fault_dev;
  args.epi_warps = (OJC_DIRECT_BF16 && args.c_bf16 && splits == 1 && !residual) ? 4 : EPI_WARPS;
  if (splits > 1) {
    void* ws = nullptr;
    OJC_TRY(ojc_scratch(be, (uint64_t)splits * m * n * 4, &ws));
    args.partial = (float*)ws;
  }
  int grid = tiles * splits < be->sm_count ? tiles * splits : be->sm_count;
  ojc_backend::GemmSample sample{nullptr, nullptr, 2.0 * (double)m * (double)n * (double)k};
  if (be->profile_gemm) {
    if (!be->event_pool.empty()) { sample.start = be->event_pool.back().first; sample.stop = be->event_pool.back().second; be->event_pool.pop_back(); }
    else { OJC_CUDA(be, cudaEventCreate(&sample.start), op); OJC_CUDA(be, cudaEventCreate(&sample.stop), op); }
    OJC_CUDA(be, cudaEventRecord(sample.start, be->stream), op);
  }
  gemm_tc_kernel<<<grid, NUM_THREADS, SMEM_BYTES, be->stream>>>(ta, tb, args);
  OJC_LAUNCHED(be, op);
  if (be->profile_gemm) {
    OJC_CUDA(be, cudaEventRecord(sample.stop, be->stream), op);
    be->gemm_samples.push_back(sample);
  }
  if (splits > 1) {
    splitk_reduce_kernel<<<elementwise_grid(be, m * n, 256), 256, 0, be->stream>>>(args.partial, splits, c, args.c_bf16, ldc, (int)m, (int)n, alpha,
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
