// Attention backward in 128-wide steps with P and dS kept in tensor memory (included by sdpa_tc5.cu, inside its namespace).
//
// The 64-wide kernels issue every product as tcgen05.mma instructions of N = 64, and an instruction of N <= 128 occupies the issue
// slot for about 96 cycles whatever its width. Here a step is 128 keys (dQ) or 128 queries (dK/dV): the S-type products are N = 128,
// the accumulating products run K = 128 deep, and a step takes a third fewer instructions per element. P and dS never pass through
// shared memory: a compute thread packs its row to bf16 and stores it with tcgen05.st over accumulator columns it has already read,
// and the accumulating products take that as their A operand.
//
// One persistent CTA per SM, ten warps:
//   warp 8     TMA producer: the tile the CTA keeps (Q and dO, or K and V; two buffers at head_dim 64), and rings of the tiles it walks.
//              It also works out where each tile of the CTA's list sits (plane, head, position, number of steps: half a dozen integer
//              divisions) and publishes that four tiles ahead through a ring of descriptors in shared memory, so that neither the MMA
//              thread nor the compute threads spend a tile switch on index arithmetic
//   warp 9     allocates all 512 TMEM columns and issues the MMAs. The roles meet once per step: when the compute threads have
//              finished step n (barrier CDONE) the MMA thread issues, back to back, the products that depend on it and the S-type
//              products of the steps ahead, so the tensor pipe works through them while the threads are in step n + 1.
//   warps 0-7  compute: thread t of a warpgroup owns TMEM lane t (a query row for dQ, a key row for dK/dV); warpgroup `half` takes
//              64 of the step's 128 columns. Phase 1 turns S into P (the exponentials, the bulk of the work) while the pipe is still
//              producing dP; phase 2 forms dS = P (dP - Dr).
// A tile's accumulators are read, handed back (ACCFREE) and stored by the compute threads right after they have handed over the next
// tile's first step, so the tile's last accumulating product has finished by then and the walk does not stall at a tile boundary.
// Every mbarrier wait is bounded; on expiry the CTA raises the fault word, drains and frees its TMEM.

constexpr int WB = 128;
// Ring of tile descriptors, and how far ahead of its own tile the producer publishes. The producer can start tile t once the S-type
// products of tile t - 2 are out (t - 1 with one buffer for the kept tile); the role furthest behind, the accumulating products'
// cursor, may then still stand on tile t - 3 when tiles are one step long, about to read descriptor t - 2. Publishing t + 4 into the
// slot of t - 4 therefore never touches a descriptor still to be read, and never runs a slot's barrier two phases ahead of a reader.
constexpr int DESC_SLOTS = 8, DESC_AHEAD = 4;

__device__ __forceinline__ void tmem_st_packed(uint32_t taddr, const uint32_t (&r)[32]) { tmem_st32(taddr, r); }


// Phase 1 of a compute thread: its 64 columns of S (or S^T) into P = exp2(S scale log2e - lse log2e). ROWSTAT: one statistic for the
// whole row (dQ); otherwise the columns' statistics, from shared memory (dK/dV). Visible columns are lo <= i < hi; MASKED is a
// compile-time switch so that the steps below the diagonal (most of them) carry no comparisons at all.
template <bool MASKED, bool ROWSTAT>
__device__ __forceinline__ void wide_phase1(uint32_t s_addr, float sl2, float lse_row, const float* stat, int lo, int hi, float (&p)[64]) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t rs[32];
    tmem_ld32(s_addr + c * 32, rs);
    tmem_wait_ld();
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float l2[4] = {lse_row, lse_row, lse_row, lse_row};
      if (!ROWSTAT) {
        const float4 l4 = *reinterpret_cast<const float4*>(stat + c * 32 + g * 4);
        l2[0] = l4.x * LOG2E; l2[1] = l4.y * LOG2E; l2[2] = l4.z * LOG2E; l2[3] = l4.w * LOG2E;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = c * 32 + g * 4 + e;
        const float v = fast_exp2(fmaf(__uint_as_float(rs[g * 4 + e]), sl2, -l2[e]));
        p[i] = (!MASKED || (i >= lo && i < hi)) ? v : 0.0f;
      }
    }
  }
}
// Phase 2: dS = P (dP - Dr) of the same 64 columns, packed to bf16 pairs. Masked columns select zero, never multiply by it (rows and
// columns past the sequence end carry whatever the buffers held).
template <bool MASKED, bool ROWSTAT>
__device__ __forceinline__ void wide_phase2(uint32_t dp_addr, float dr_row, const float* stat_dr, int lo, int hi, const float (&p)[64], uint32_t (&dsw)[32]) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t rp[32];
    tmem_ld32(dp_addr + c * 32, rp);
    tmem_wait_ld();
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float dd[4] = {dr_row, dr_row, dr_row, dr_row};
      if (!ROWSTAT) {
        const float4 d4 = *reinterpret_cast<const float4*>(stat_dr + c * 32 + g * 4);
        dd[0] = d4.x; dd[1] = d4.y; dd[2] = d4.z; dd[3] = d4.w;
      }
      float ds[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = c * 32 + g * 4 + e;
        const float v = p[i] * (__uint_as_float(rp[g * 4 + e]) - dd[e]);
        ds[e] = (!MASKED || (i >= lo && i < hi)) ? v : 0.0f;
      }
      dsw[c * 16 + g * 2] = pack2_bf16(ds[0], ds[1]);
      dsw[c * 16 + g * 2 + 1] = pack2_bf16(ds[2], ds[3]);
    }
  }
}

// ---- dQ
template <int D> struct DqW {
  static constexpr int NSUB = D / 64, TILE_BYTES = NSUB * ST128;    // a 128-row tile of q, dO, k or v
  static constexpr int NQD = D == 64 ? 2 : 1;                       // buffers for the Q / dO tile the CTA keeps
  // K lives from its S (two steps ahead) to its dQ, V only for its dP; a stage freed by a product must be refilled (about a microsecond
  // from L2) before the product two or three steps on needs it, so head_dim 64, with room to spare and short steps, rings one deeper
  static constexpr int KS = D == 64 ? 4 : 3, VS = D == 64 ? 3 : 2;
  static constexpr int OFF_Q = 0, OFF_G = NQD * TILE_BYTES, OFF_K = 2 * NQD * TILE_BYTES, OFF_V = OFF_K + KS * TILE_BYTES, OFF_BAR = OFF_V + VS * TILE_BYTES;
  static constexpr int OFF_DESC = OFF_BAR + 512;                    // barriers and the TMEM slot, then the ring of tile descriptors
  static constexpr int SMEM_BYTES = OFF_DESC + DESC_SLOTS * 32 + 1024;   // D 64: 178 KB; D 128: 226 KB
  static constexpr int COL_S = 0, COL_DP = 256, COL_DQ = 384;       // S (two buffers of 128 columns; dS over the first 32 of each half), dP, dQ
};
enum { WQ_QDFULL0 = 0, WQ_QDEMPTY0 = 2, WQ_KFULL0 = 4, WQ_KEMPTY0 = 8, WQ_VFULL0 = 12, WQ_VEMPTY0 = 15, WQ_SFULL0 = 18, WQ_DPFULL = 20, WQ_CDONE, WQ_DONE, WQ_ACCFREE, WQ_DESC0, WQ_COUNT = WQ_DESC0 + DESC_SLOTS };

// Where a tile sits: pos = its first query (dQ) or key (dK/dV) row; h = the query head (dQ only); blocks = 128-wide query blocks
// per head of the walk (dK/dV only); iters = steps of the walk; valid = 0 past the end of the CTA's list.
struct TileDesc { int pos, b, h, hk, iters, blocks, valid, pad; };

__device__ __forceinline__ TileDesc dq_tile(const BwdArgs& args, int tiles, int total, int item) {
  TileDesc d = {0, 0, 0, 0, 0, 0, 0, 0};
  const int g = blockIdx.x + item * gridDim.x;
  if (g >= total) return d;
  const TileOrder ord = tile_order(g, args.planes, args.group, tiles);
  d.pos = (tiles - 1 - ord.rank) * BM;
  d.b = ord.plane / args.heads; d.h = ord.plane % args.heads; d.hk = d.h / (args.heads / args.kv_heads);
  d.iters = (min(args.time, d.pos + BM) + WB - 1) / WB;
  d.valid = 1;
  return d;
}
__device__ __forceinline__ TileDesc dkv_tile(const BwdArgs& args, int tiles, int total, int item) {
  TileDesc d = {0, 0, 0, 0, 0, 0, 0, 0};
  const int g = blockIdx.x + item * gridDim.x;
  if (g >= total) return d;
  const TileOrder ord = tile_order(g, args.planes, args.group, tiles);
  d.pos = ord.rank * BN;                         // early key tiles see the most queries
  d.b = ord.plane / args.kv_heads; d.hk = ord.plane % args.kv_heads;
  d.blocks = (args.time - d.pos + WB - 1) / WB;
  d.iters = (args.heads / args.kv_heads) * d.blocks;
  d.valid = 1;
  return d;
}
// The producer thread writes descriptor `item` into slot item % 8 and arrives on the slot's barrier (release); a reader waits for
// the slot's phase item / 8 (acquire) and copies the descriptor out.
__device__ __forceinline__ void publish_desc(uint8_t* ring, uint32_t bar0, int item, const TileDesc& d) {
  int4* slot = reinterpret_cast<int4*>(ring + (item % DESC_SLOTS) * 32);
  slot[0] = make_int4(d.pos, d.b, d.h, d.hk);
  slot[1] = make_int4(d.iters, d.blocks, d.valid, 0);
  mbar_arrive(bar0 + 8u * (item % DESC_SLOTS));
}
__device__ __forceinline__ bool read_desc(const uint8_t* ring, uint32_t bar0, int item, TileDesc& d, uint32_t* fault, volatile int* abort_flag) {
  if (!mbar_wait(bar0 + 8u * (item % DESC_SLOTS), (item / DESC_SLOTS) & 1, fault, abort_flag)) { d.valid = 0; return false; }
  const int4* slot = reinterpret_cast<const int4*>(ring + (item % DESC_SLOTS) * 32);
  const int4 a = slot[0], c = slot[1];
  d.pos = a.x; d.b = a.y; d.h = a.z; d.hk = a.w; d.iters = c.x; d.blocks = c.y; d.valid = c.z; d.pad = 0;
  return true;
}
// where one role stands in the CTA's stream of steps: step n of the stream is step j of tile `item`
struct StepCursor {
  TileDesc d;
  int item, j;
  uint32_t n;
  bool valid;
  __device__ __forceinline__ bool start(const uint8_t* ring, uint32_t bar0, uint32_t* fault, volatile int* abort_flag) {
    item = 0; j = 0; n = 0;
    const bool ok = read_desc(ring, bar0, 0, d, fault, abort_flag);
    valid = ok && d.valid;
    return ok;
  }
  __device__ __forceinline__ bool advance(const uint8_t* ring, uint32_t bar0, uint32_t* fault, volatile int* abort_flag) {
    ++n;
    if (++j < d.iters) return true;
    ++item; j = 0;
    const bool ok = read_desc(ring, bar0, item, d, fault, abort_flag);
    valid = ok && d.valid;
    return ok;
  }
  __device__ __forceinline__ bool last() const { return j + 1 == d.iters; }
};

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
sdpa_bwd_dq_w_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  using C = DqW<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, NQD = C::NQD, KS = C::KS, VS = C::VS;
  constexpr uint32_t TILE16 = TILE_BYTES >> 4;
  static_assert(WQ_COUNT * 8 + 8 <= 512, "barrier table");
  uint8_t* ring = base_ptr + C::OFF_DESC;
  const uint32_t desc_bar = base + C::OFF_BAR + 8u * WQ_DESC0;
  auto bar = [&](int i) { return base + C::OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + C::OFF_BAR + 8 * WQ_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (args.time + BM - 1) / BM, total = tiles * args.planes;

  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_g);
    for (int i = 0; i < WQ_COUNT; ++i) mbar_init(bar(i), (i == WQ_CDONE || i == WQ_ACCFREE) ? 256 : 1);
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
      for (int i = 0; i < DESC_AHEAD; ++i) publish_desc(ring, desc_bar, i, dq_tile(args, tiles, total, i));
      uint32_t n = 0;
      bool ok = true;
      for (int item = 0; ok; ++item) {
        const TileDesc w = dq_tile(args, tiles, total, item);
        if (!w.valid) break;
        const int qb = item % NQD;
        // a Q / dO buffer is free once the last S and dP of the tile that used it have read it
        if (item >= NQD && !mbar_wait(bar(WQ_QDEMPTY0 + qb), ((item / NQD) - 1) & 1, args.fault, abort_flag)) break;
        publish_desc(ring, desc_bar, item + DESC_AHEAD, dq_tile(args, tiles, total, item + DESC_AHEAD));
        mbar_expect_tx(bar(WQ_QDFULL0 + qb), 2 * TILE_BYTES);
        load_tile<NSUB, 128>(base + C::OFF_Q + qb * TILE_BYTES, &tm_q, bar(WQ_QDFULL0 + qb), args.h_first, w.h, w.pos, w.b);
        load_tile<NSUB, 128>(base + C::OFF_G + qb * TILE_BYTES, &tm_g, bar(WQ_QDFULL0 + qb), args.h_first, w.h, w.pos, w.b);
        for (int j = 0; j < w.iters; ++j, ++n) {
          const int ks = n % KS, vs = n % VS;
          if (n >= KS && !mbar_wait(bar(WQ_KEMPTY0 + ks), ((n / KS) - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          mbar_expect_tx(bar(WQ_KFULL0 + ks), TILE_BYTES);
          load_tile<NSUB, 128>(base + C::OFF_K + ks * TILE_BYTES, &tm_k, bar(WQ_KFULL0 + ks), args.h_first, w.hk, j * WB, w.b);
          if (n >= VS && !mbar_wait(bar(WQ_VEMPTY0 + vs), ((n / VS) - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          mbar_expect_tx(bar(WQ_VFULL0 + vs), TILE_BYTES);
          load_tile<NSUB, 128>(base + C::OFF_V + vs * TILE_BYTES, &tm_v, bar(WQ_VFULL0 + vs), args.h_first, w.hk, j * WB, w.b);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BM, WB, 0, 0), idesc_o = make_idesc(BM, D, 0, 1);
      const uint32_t q_lo = desc_lo(base + C::OFF_Q, 0), g_lo = desc_lo(base + C::OFF_G, 0), k_lo = desc_lo(base + C::OFF_K, 0), v_lo = desc_lo(base + C::OFF_V, 0);
      const uint32_t km_lo = desc_lo(base + C::OFF_K, ST128);
      using Cur = StepCursor;
      // S = Q K^T of the cursor's step, into S buffer n % 2
      auto issue_s = [&](const Cur& c) -> bool {
        const uint32_t qd = (uint32_t)(c.item % NQD) * TILE16, ks = (c.n % KS) * TILE16;
        if (c.j == 0 && !mbar_wait(bar(WQ_QDFULL0 + c.item % NQD), (c.item / NQD) & 1, args.fault, abort_flag)) return false;
        if (!mbar_wait(bar(WQ_KFULL0 + c.n % KS), (c.n / KS) & 1, args.fault, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + C::COL_S + (c.n & 1) * WB, q_lo + qd + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, k_lo + ks + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(WQ_SFULL0 + (c.n & 1)));
        return true;
      };
      // dP = dO V^T of the cursor's step; the tile's last one frees its Q / dO buffer (its S went out earlier)
      auto issue_dp = [&](const Cur& c) -> bool {
        const uint32_t qd = (uint32_t)(c.item % NQD) * TILE16, vs = (c.n % VS) * TILE16;
        if (!mbar_wait(bar(WQ_VFULL0 + c.n % VS), (c.n / VS) & 1, args.fault, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + C::COL_DP, g_lo + qd + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, v_lo + vs + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(WQ_DPFULL));
        umma_commit(bar(WQ_VEMPTY0 + c.n % VS));
        if (c.last()) umma_commit(bar(WQ_QDEMPTY0 + c.item % NQD));
        return true;
      };
      // dQ += dS K of the cursor's step: dS from tensor memory (each half's 64 keys packed over the first 32 columns of its S columns),
      // K as the MN-major B operand (16 keys = 2048 bytes)
      auto issue_dq = [&](const Cur& c) -> bool {
        // a tile's first dQ product overwrites the accumulator: the previous tile's rows must hold theirs in registers
        if (c.j == 0 && c.item > 0 && !mbar_wait(bar(WQ_ACCFREE), (c.item - 1) & 1, args.fault, abort_flag)) return false;
        const uint32_t ks = (c.n % KS) * TILE16, ds = tmem_base + C::COL_S + (c.n & 1) * WB;
#pragma unroll
        for (uint32_t kk = 0; kk < WB / 16; ++kk)
          umma_ts(tmem_base + C::COL_DQ, ds + (kk >> 2) * 64 + (kk & 3) * 8, km_lo + ks + kk * MNSTEP, HI, idesc_o, (c.j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(WQ_KEMPTY0 + c.n % KS));
        if (c.last()) umma_commit(bar(WQ_DONE));
        return true;
      };
      auto next = [&](Cur& c) { return c.advance(ring, desc_bar, args.fault, abort_flag); };
      Cur cs, cp, cq;
      bool ok = cs.start(ring, desc_bar, args.fault, abort_flag) && cs.valid;
      cp = cs; cq = cs;
      if (ok) ok = issue_s(cs) && next(cs);
      if (ok && cs.valid) ok = issue_s(cs) && next(cs);
      if (ok) ok = issue_dp(cp) && next(cp);
      while (ok && cq.valid) {
        if (!mbar_wait(bar(WQ_CDONE), cq.n & 1, args.fault, abort_flag)) break;
        fence_after();
        if (cp.valid && !(issue_dp(cp) && next(cp))) break;
        if (!(issue_dq(cq) && next(cq))) break;
        if (cs.valid && !(issue_s(cs) && next(cs))) break;
      }
    }
  } else {
    const int tid = threadIdx.x & 127, half = warp >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    TileDesc w, wn;
    uint32_t n = 0;
    bool ok = true, fin = false;
    int fin_item = 0, fin_b = 0, fin_h = 0, fin_row = 0;
    // the finished tile's dQ: wait for its last product, read this thread's half of the row, hand the accumulator back, store
    auto finalize = [&]() -> bool {
      if (!mbar_wait(bar(WQ_DONE), fin_item & 1, args.fault, abort_flag)) return false;
      fence_after();
      bf16* dst = fin_row < args.time ? args.g0.row(fin_b, fin_h, fin_row) + half * (D / 2) : nullptr;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t acc[32];
        load_acc<32>(lane_base + C::COL_DQ + half * (D / 2) + c * 32, acc);
        if (c + 1 == D / 64) { fence_before(); mbar_arrive(bar(WQ_ACCFREE)); }
        store_acc_bf16<32>(dst ? dst + c * 32 : nullptr, acc, args.scale);
      }
      fin = false;
      return true;
    };
    // The row's statistics are fetched one tile ahead, so their latency sits under the previous tile's walk (the loaded values are
    // not touched until the tile switch: a thread stalls at the first use of a load, not at the load).
    auto stat_of = [&](const TileDesc& t, float& lse, float& dr) {
      const int r = t.pos + tid;
      const int64_t idx = ((int64_t)t.b * args.heads + t.h) * args.time + r;
      lse = INFINITY; dr = 0.0f;
      if (t.valid && r < args.time) { lse = args.lse[idx]; dr = args.dr[idx]; }
    };
    ok = read_desc(ring, desc_bar, 0, w, args.fault, abort_flag);
    float lse_row = INFINITY, dr_row = 0.0f, lse_next, dr_next;
    if (ok && w.valid) { stat_of(w, lse_row, dr_row); lse_row *= LOG2E; }
    for (int item = 0; ok && w.valid; ++item) {
      if (!read_desc(ring, desc_bar, item + 1, wn, args.fault, abort_flag)) { ok = false; break; }
      stat_of(wn, lse_next, dr_next);
      const int row = w.pos + tid;
      for (int j = 0; j < w.iters; ++j, ++n) {
        const int key0 = j * WB + half * 64;
        const uint32_t s_addr = lane_base + C::COL_S + (n & 1) * WB + half * 64;
        if (!mbar_wait(bar(WQ_SFULL0 + (n & 1)), (n >> 1) & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        const bool masked = j * WB + WB > w.pos || j * WB + WB > args.time;
        // visible columns of this half: key <= row and key < time, as a range of column indices
        const int lo = 0, hi = min(row - key0 + 1, args.time - key0);
        float p[64];
        if (masked) wide_phase1<true, true>(s_addr, sl2, lse_row, nullptr, lo, hi, p); else wide_phase1<false, true>(s_addr, sl2, lse_row, nullptr, lo, hi, p);
        if (!mbar_wait(bar(WQ_DPFULL), n & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        // phase 2: dS over this half's first 32 S columns (all of them read above)
        uint32_t dsw[32];
        if (masked) wide_phase2<true, true>(lane_base + C::COL_DP + half * 64, dr_row, nullptr, lo, hi, p, dsw);
        else wide_phase2<false, true>(lane_base + C::COL_DP + half * 64, dr_row, nullptr, lo, hi, p, dsw);
        tmem_st_packed(s_addr, dsw);
        tmem_wait_st();
        fence_before();
        mbar_arrive(bar(WQ_CDONE));
        // the previous tile's dQ, after this tile's first step has been handed over: its last product has long finished, and the MMA
        // thread needs the accumulator back only for this step's dQ product, which it issues after the next step's dP
        if (fin && !finalize()) { ok = false; break; }
      }
      if (!ok) break;
      fin = true; fin_item = item; fin_b = w.b; fin_h = w.h; fin_row = row;
      w = wn; lse_row = lse_next * LOG2E; dr_row = dr_next;
    }
    if (ok && fin) finalize();
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- dK, dV
template <int D> struct DkvW {
  static constexpr int NSUB = D / 64, TILE_BYTES = NSUB * ST128;
  static constexpr int NKV = D == 64 ? 2 : 1;                       // buffers for the K / V tile the CTA keeps
  static constexpr int NS = D == 64 ? 2 : 1;                        // S^T buffers: two at head_dim 64; at 128 the accumulators leave room for one
  // Q lives from its S^T to its dK, dO from its dP^T to its dV; deep enough that a freed stage is refilled (about a microsecond from
  // L2) before the step that needs it
  static constexpr int QS = D == 64 ? 4 : 3, GS = D == 64 ? 3 : 2;
  static constexpr int OFF_K = 0, OFF_V = NKV * TILE_BYTES, OFF_Q = 2 * NKV * TILE_BYTES, OFF_G = OFF_Q + QS * TILE_BYTES, OFF_STAT = OFF_G + GS * TILE_BYTES,
                       OFF_BAR = OFF_STAT + GS * 1024;              // per dO stage: lse of its 128 queries, then their Dr
  static constexpr int OFF_DESC = OFF_BAR + 512;                    // barriers and the TMEM slot, then the ring of tile descriptors
  static constexpr int SMEM_BYTES = OFF_DESC + DESC_SLOTS * 32;     // D 64: 179.75 KB; D 128: 226.75 KB (the launch asks for 1024-byte alignment)
  static_assert(SMEM_BYTES <= 232448, "shared memory per CTA");
  static constexpr int COL_S = 0, COL_DP = NS * WB, COL_DV = COL_DP + WB, COL_DK = COL_DV + D;   // 512 columns either way
};
enum { WK_KVFULL0 = 0, WK_KVEMPTY0 = 2, WK_QFULL0 = 4, WK_QEMPTY0 = 8, WK_GFULL0 = 12, WK_GEMPTY0 = 15, WK_SFULL0 = 18, WK_DPFULL = 20, WK_CDONE, WK_DONE, WK_ACCFREE, WK_DESC0, WK_COUNT = WK_DESC0 + DESC_SLOTS };

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
sdpa_bwd_dkv_w_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_g, const BwdArgs args) {
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) { if (threadIdx.x == 0) raise_fault(args.fault, OP_SDPA); return; }   // the swizzled tiles need 1024-byte alignment (whole CTA leaves)
  uint8_t* base_ptr = smem_raw;
  using C = DkvW<D>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, NKV = C::NKV, NS = C::NS, QS = C::QS, GS = C::GS;
  constexpr uint32_t TILE16 = TILE_BYTES >> 4;
  static_assert(WK_COUNT * 8 + 8 <= 512, "barrier table");
  uint8_t* ring = base_ptr + C::OFF_DESC;
  const uint32_t desc_bar = base + C::OFF_BAR + 8u * WK_DESC0;
  static_assert(C::COL_DK + D <= 512, "tensor memory columns");
  auto bar = [&](int i) { return base + C::OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + C::OFF_BAR + 8 * WK_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (args.time + BN - 1) / BN, total = tiles * args.planes;

  if (warp == 8 && lane == 0) {
    prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_g);
    for (int i = 0; i < WK_COUNT; ++i) mbar_init(bar(i), (i == WK_CDONE || i == WK_ACCFREE) ? 256 : 1);
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
      for (int i = 0; i < DESC_AHEAD; ++i) publish_desc(ring, desc_bar, i, dkv_tile(args, tiles, total, i));
      const int rep = args.heads / args.kv_heads;
      uint32_t n = 0;
      bool ok = true;
      for (int item = 0; ok; ++item) {
        const TileDesc w = dkv_tile(args, tiles, total, item);
        if (!w.valid) break;
        const int kb = item % NKV;
        if (item >= NKV && !mbar_wait(bar(WK_KVEMPTY0 + kb), ((item / NKV) - 1) & 1, args.fault, abort_flag)) break;
        publish_desc(ring, desc_bar, item + DESC_AHEAD, dkv_tile(args, tiles, total, item + DESC_AHEAD));
        mbar_expect_tx(bar(WK_KVFULL0 + kb), 2 * TILE_BYTES);
        load_tile<NSUB, 128>(base + C::OFF_K + kb * TILE_BYTES, &tm_k, bar(WK_KVFULL0 + kb), args.h_first, w.hk, w.pos, w.b);
        load_tile<NSUB, 128>(base + C::OFF_V + kb * TILE_BYTES, &tm_v, bar(WK_KVFULL0 + kb), args.h_first, w.hk, w.pos, w.b);
        int h = w.hk * rep, q0 = w.pos;                // the walk: every query head of the group, each from the diagonal block to the end
        for (int j = 0; j < w.iters; ++j, ++n) {
          const int qs = n % QS, gs = n % GS;
          if (n >= QS && !mbar_wait(bar(WK_QEMPTY0 + qs), ((n / QS) - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          const uint32_t stat_bytes = (uint32_t)min(WB, args.time - q0) * 4u;
          const int64_t idx = ((int64_t)w.b * args.heads + h) * args.time + q0;
          mbar_expect_tx(bar(WK_QFULL0 + qs), TILE_BYTES);
          load_tile<NSUB, 128>(base + C::OFF_Q + qs * TILE_BYTES, &tm_q, bar(WK_QFULL0 + qs), args.h_first, h, q0, w.b);
          if (n >= GS && !mbar_wait(bar(WK_GEMPTY0 + gs), ((n / GS) - 1) & 1, args.fault, abort_flag)) { ok = false; break; }
          mbar_expect_tx(bar(WK_GFULL0 + gs), TILE_BYTES + 2 * stat_bytes);
          bulk_load(base + C::OFF_STAT + gs * 1024, args.lse + idx, stat_bytes, bar(WK_GFULL0 + gs));
          bulk_load(base + C::OFF_STAT + gs * 1024 + 512, args.dr + idx, stat_bytes, bar(WK_GFULL0 + gs));
          load_tile<NSUB, 128>(base + C::OFF_G + gs * TILE_BYTES, &tm_g, bar(WK_GFULL0 + gs), args.h_first, h, q0, w.b);
          q0 += WB;
          if (q0 >= args.time) { q0 = w.pos; ++h; }
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BN, WB, 0, 0), idesc_o = make_idesc(BN, D, 0, 1);
      const uint32_t k_lo = desc_lo(base + C::OFF_K, 0), v_lo = desc_lo(base + C::OFF_V, 0), q_lo = desc_lo(base + C::OFF_Q, 0), g_lo = desc_lo(base + C::OFF_G, 0);
      const uint32_t qm_lo = desc_lo(base + C::OFF_Q, ST128), gm_lo = desc_lo(base + C::OFF_G, ST128);
      using Cur = StepCursor;
      // S^T = K Q^T of the cursor's step
      auto issue_s = [&](const Cur& c) -> bool {
        const uint32_t kv = (uint32_t)(c.item % NKV) * TILE16, qs = (c.n % QS) * TILE16;
        if (c.j == 0 && !mbar_wait(bar(WK_KVFULL0 + c.item % NKV), (c.item / NKV) & 1, args.fault, abort_flag)) return false;
        if (!mbar_wait(bar(WK_QFULL0 + c.n % QS), (c.n / QS) & 1, args.fault, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + C::COL_S + (c.n % NS) * WB, k_lo + kv + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, q_lo + qs + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(WK_SFULL0 + c.n % NS));
        return true;
      };
      // dP^T = V dO^T of the cursor's step; the tile's last one frees its K / V buffer (its S^T went out earlier)
      auto issue_dp = [&](const Cur& c) -> bool {
        const uint32_t kv = (uint32_t)(c.item % NKV) * TILE16, gs = (c.n % GS) * TILE16;
        if (!mbar_wait(bar(WK_GFULL0 + c.n % GS), (c.n / GS) & 1, args.fault, abort_flag)) return false;
        fence_after();
#pragma unroll
        for (uint32_t kk = 0; kk < D / 16; ++kk)
          umma_lh(tmem_base + C::COL_DP, v_lo + kv + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, g_lo + gs + (kk >> 2) * ST128_16 + (kk & 3) * KSTEP, HI, idesc_s, kk > 0);
        umma_commit(bar(WK_DPFULL));
        if (c.last()) umma_commit(bar(WK_KVEMPTY0 + c.item % NKV));
        return true;
      };
      // dV += P^T dO (P^T over the first 32 columns of each half of its S^T buffer), dK += dS^T Q (dS^T likewise over dP^T)
      auto issue_dv = [&](const Cur& c) {
        const uint32_t gs = (c.n % GS) * TILE16, pt = tmem_base + C::COL_S + (c.n % NS) * WB;
#pragma unroll
        for (uint32_t kk = 0; kk < WB / 16; ++kk)
          umma_ts(tmem_base + C::COL_DV, pt + (kk >> 2) * 64 + (kk & 3) * 8, gm_lo + gs + kk * MNSTEP, HI, idesc_o, (c.j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(WK_GEMPTY0 + c.n % GS));
      };
      auto issue_dk = [&](const Cur& c) {
        const uint32_t qs = (c.n % QS) * TILE16, dst = tmem_base + C::COL_DP;
#pragma unroll
        for (uint32_t kk = 0; kk < WB / 16; ++kk)
          umma_ts(tmem_base + C::COL_DK, dst + (kk >> 2) * 64 + (kk & 3) * 8, qm_lo + qs + kk * MNSTEP, HI, idesc_o, (c.j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(WK_QEMPTY0 + c.n % QS));
      };
      auto next = [&](Cur& c) { return c.advance(ring, desc_bar, args.fault, abort_flag); };
      Cur cs, cp, cq;
      bool ok = cs.start(ring, desc_bar, args.fault, abort_flag) && cs.valid;
      cp = cs; cq = cs;
      if (ok) ok = issue_s(cs) && next(cs);
      if (NS == 2 && ok && cs.valid) ok = issue_s(cs) && next(cs);
      if (ok) ok = issue_dp(cp) && next(cp);
      while (ok && cq.valid) {
        if (!mbar_wait(bar(WK_CDONE), cq.n & 1, args.fault, abort_flag)) break;
        // a tile's first accumulating products overwrite dV and dK: the previous tile's rows must hold theirs in registers (they read
        // them right after handing this step over)
        if (cq.j == 0 && cq.item > 0 && !mbar_wait(bar(WK_ACCFREE), (cq.item - 1) & 1, args.fault, abort_flag)) break;
        fence_after();
        const bool last = cq.last();
        if (NS == 2) {
          // dS^T sits over dP^T: dK first, then the next dP^T may overwrite it; P^T sits over S^T: dV, then the S^T two steps ahead
          issue_dk(cq);
          if (cp.valid && !(issue_dp(cp) && next(cp))) break;
          issue_dv(cq);
          if (last) umma_commit(bar(WK_DONE));
          if (!next(cq)) break;
          if (cs.valid && !(issue_s(cs) && next(cs))) break;
        } else {
          // one S^T buffer: dV, then the next S^T at once (the compute threads wait for it), then dK and the next dP^T under its exponentials
          issue_dv(cq);
          if (cs.valid && !(issue_s(cs) && next(cs))) break;
          issue_dk(cq);
          if (last) umma_commit(bar(WK_DONE));
          if (!next(cq)) break;
          if (cp.valid && !(issue_dp(cp) && next(cp))) break;
        }
      }
    }
  } else {
    const int tid = threadIdx.x & 127, half = warp >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl2 = args.scale * LOG2E;
    TileDesc w;
    uint32_t n = 0;
    bool ok = true, fin = false;
    int fin_item = 0, fin_b = 0, fin_hk = 0, fin_key = 0;
    // the finished tile's accumulators: warpgroup 0 takes dV, warpgroup 1 dK (scaled); 32 columns at a time
    auto finalize = [&]() -> bool {
      if (!mbar_wait(bar(WK_DONE), fin_item & 1, args.fault, abort_flag)) return false;
      fence_after();
      bf16* dst = fin_key < args.time ? (half == 0 ? args.g1.row(fin_b, fin_hk, fin_key) : args.g0.row(fin_b, fin_hk, fin_key)) : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t acc[32];
        load_acc<32>(lane_base + (half == 0 ? C::COL_DV : C::COL_DK) + c * 32, acc);
        if (c + 1 == D / 32) { fence_before(); mbar_arrive(bar(WK_ACCFREE)); }
        store_acc_bf16<32>(dst ? dst + c * 32 : nullptr, acc, half == 0 ? 1.0f : args.scale);
      }
      fin = false;
      return true;
    };
    for (int item = 0; ok; ++item) {
      if (!read_desc(ring, desc_bar, item, w, args.fault, abort_flag)) { ok = false; break; }
      if (!w.valid) break;
      const int key = w.pos + tid;
      int q0 = w.pos - WB;
      for (int j = 0; j < w.iters; ++j, ++n) {
        q0 += WB;
        if (q0 >= args.time) q0 = w.pos;              // the next query head of the group, from the diagonal block again
        const int qb = q0 + half * 64;
        const uint32_t s_addr = lane_base + C::COL_S + (n % NS) * WB + half * 64, dp_addr = lane_base + C::COL_DP + half * 64;
        const float* stat = reinterpret_cast<const float*>(base_ptr + C::OFF_STAT + (n % GS) * 1024) + half * 64;
        // the step's statistics arrive with its dO tile; then its S^T
        if (!mbar_wait(bar(WK_GFULL0 + n % GS), (n / GS) & 1, args.fault, abort_flag)) { ok = false; break; }
        if (!mbar_wait(bar(WK_SFULL0 + n % NS), (n / NS) & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        const bool masked = q0 < w.pos + BN || q0 + WB > args.time || w.pos + BN > args.time;
        // visible columns of this half: key <= q, q < time (and the key itself inside the sequence), as a range of column indices
        const int lo = key < args.time ? key - qb : 64, hi = args.time - qb;
        // phase 1: P^T with the columns' (queries') statistics; packed over this half's first 32 S^T columns
        float p[64];
        uint32_t pw[32];
        if (masked) wide_phase1<true, false>(s_addr, sl2, 0.0f, stat, lo, hi, p); else wide_phase1<false, false>(s_addr, sl2, 0.0f, stat, lo, hi, p);
#pragma unroll
        for (int e = 0; e < 32; ++e) pw[e] = pack2_bf16(p[2 * e], p[2 * e + 1]);
        tmem_st_packed(s_addr, pw);
        if (!mbar_wait(bar(WK_DPFULL), n & 1, args.fault, abort_flag)) { ok = false; break; }
        fence_after();
        // phase 2: dS^T over this half's first 32 dP^T columns
        uint32_t dsw[32];
        if (masked) wide_phase2<true, false>(dp_addr, 0.0f, stat + 128, lo, hi, p, dsw); else wide_phase2<false, false>(dp_addr, 0.0f, stat + 128, lo, hi, p, dsw);
        tmem_st_packed(dp_addr, dsw);
        tmem_wait_st();
        fence_before();
        mbar_arrive(bar(WK_CDONE));
        if (fin && !finalize()) { ok = false; break; }   // the previous tile's dV and dK, once this tile's first step has been handed over
      }
      if (!ok) break;
      fin = true; fin_item = item; fin_b = w.b; fin_hk = w.hk; fin_key = key;
    }
    if (ok && fin) finalize();
  }
  if (*abort_flag) __nanosleep(200000);
  fence_before();
  __syncthreads();
  if (warp == 9) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}
