// Tensor-core backward kernels for bf16 / fp16 tensors (reference counterpart: _backward_one_row,
// sb_varlen_bwd.py:297-481, which accumulates dK/dV across blocks under a global spin lock).
//
// Two kernels per call, no atomics, no locks, fixed summation order:
//   dq kernel (tc_bwd_dq2_kernel)   query-stationary, 256 query rows per block.  Walks the keys 0 -> diagonal in
//               64-key sub-tiles; per step S = Q K^T and dP = dO V^T go to TMEM, one thread per query row recomputes
//               A and dz = G - beta * C with the log-space suffix sum (fp64 across tiles, started from the saved
//               log_rem) and the prefix sum C of G carried in registers, writes dz as a 16-bit tile, and
//               dQ += dz K accumulates in TMEM.  It leaves for the second kernel either its A and dz tiles
//               (stored-tiles mode) or, every 32 keys, the two carried values R1 and S2 (small-workspace mode).
//   dK/dV kernel  key-stationary, one 128-key tile per block, query tiles diagonal -> end.
//               tc_bwd_dkv5_kernel: dK += dz^T Q and dV += A^T dO as plain GEMMs over the stored tiles.
//               tc_bwd_dkv4_kernel: repeats the row pass of each tile from the recorded R1/S2 first.
// Head sizes below 128 run the same code: TMA zero-fills the columns past head_dim.  All waits are bounded.
#include "sb_tc_common.cuh"

namespace sb {

// One row, 16 consecutive key columns.  s: raw q.k accumulators, dp: <dO_i, v_j>.
//   x = z log2(e), clamped at 30;  e = 2^x;  t = 1 + e;  1 - beta = 1 / t;  beta = e / t
//   A_j = beta_j * W_j,  W_j = product of (1 - beta) over the allowed keys after j up to the diagonal
//       = e_j * (product of 1 / t over j and the allowed keys after it)
//   G = A (dP - dR);  C = gpre + inclusive prefix of G;  dz = G - beta C
// Three sweeps over the 16 columns, all in registers: (1) e, beta and, per group of four columns, one reciprocal
// and one logarithm of t0 t1 t2 t3, which gives the log-space sum through the end of the chunk; (2) last group to
// first: the product is seeded with 2^(r1 + that sum) -- the largest value it takes in the chunk, so it only
// underflows where A rounds to zero anyway -- shrinks by the group's reciprocal per group, and the four inclusive
// products inside a group come from partial reciprocals sweep 1 already has; (3) first group to last: the prefix
// sum of G, carried per group, and dz.  About 1.6 transcendentals per score (ex2, rcp / 4, lg2 / 4, ex2 / 16).
// kMasked tiles (the diagonal one, or one with rows past the sequence end) zero what is not allowed.
// The chunk is kept to 16 columns so that the unrolled code of all variants stays inside the instruction cache.
// mc0: key index of the first column inside the 128-key tile (for the diagonal mask).
// skip_zero (unmasked chunks only): where the product of (1 - beta) at the END of the chunk -- its largest value in
// the chunk -- has underflowed to exactly 0 and the prefix of G is still exactly 0, for all 32 rows of the warp, every
// A, G and dz of the chunk is exactly 0 (e, the reciprocals and dP - dR are finite): only the log-space sum is formed,
// with the same operations as otherwise, and the rest is not computed.
template <bool kMasked>
__device__ __forceinline__ void bwd_row_chunk_values(const uint32_t (&s)[16], const uint32_t (&dp)[16], int mc0, int r, bool diag,
                                                     int ac, bool row_valid, float scale2, float r1, float gpre, float dr,
                                                     float &gs, float &logsum, float (&pa)[16], float (&pz)[16],
                                                     bool skip_zero = false) {
  // columns (tile-local key indices) below `limit` are allowed: one compare per column, no branches
  const int limit = !row_valid ? -1 : (diag ? r + ac : 0x7fffffff);
  const float2 sc = make_float2(scale2, scale2), one = make_float2(1.f, 1.f);
  float2 e01[4], e23[4], be01[4], be23[4];
  float rpg[4], q23[4], ri1[4], ri3[4];
  float2 tt01[4], tt23[4], ppg[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {   // independent work in packed pairs (two fp32 per instruction)
    const float2 x01 = mul2(make_float2(__uint_as_float(s[4 * g]), __uint_as_float(s[4 * g + 1])), sc);
    const float2 x23 = mul2(make_float2(__uint_as_float(s[4 * g + 2]), __uint_as_float(s[4 * g + 3])), sc);
    e01[g] = make_float2(ex2(fminf(x01.x, 30.f)), ex2(fminf(x01.y, 30.f)));
    e23[g] = make_float2(ex2(fminf(x23.x, 30.f)), ex2(fminf(x23.y, 30.f)));
    float2 t01 = add2(e01[g], one), t23 = add2(e23[g], one);
    if (kMasked) {
      const int col = mc0 + 4 * g;
      if (!(col < limit)) { e01[g].x = 0.f; t01.x = 1.f; }
      if (!(col + 1 < limit)) { e01[g].y = 0.f; t01.y = 1.f; }
      if (!(col + 2 < limit)) { e23[g].x = 0.f; t23.x = 1.f; }
      if (!(col + 3 < limit)) { e23[g].y = 0.f; t23.y = 1.f; }
    }
    const float2 pp = mul2(make_float2(t01.x, t23.x), make_float2(t01.y, t23.y));   // (t0 t1, t2 t3)
    logsum += lg2(pp.x * pp.y);
    tt01[g] = t01;
    tt23[g] = t23;
    ppg[g] = pp;
  }
  if (!kMasked && skip_zero && __all_sync(0xffffffffu, ex2(r1 + logsum) == 0.f && gpre + gs == 0.f)) {
#pragma unroll
    for (int i = 0; i < 16; ++i) { pa[i] = 0.f; pz[i] = 0.f; }
    return;
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const float2 t01 = tt01[g], t23 = tt23[g], pp = ppg[g];
    const float rp = rcp(pp.x * pp.y);
    const float2 ab = mul2(make_float2(rp, rp), make_float2(pp.y, pp.x));           // (1 / t0 t1, 1 / t2 t3)
    const float2 ri01 = mul2(make_float2(ab.x, ab.x), make_float2(t01.y, t01.x));   // (1/t0, 1/t1)
    const float2 ri23 = mul2(make_float2(ab.y, ab.y), make_float2(t23.y, t23.x));   // (1/t2, 1/t3)
    be01[g] = mul2(e01[g], ri01);
    be23[g] = mul2(e23[g], ri23);
    rpg[g] = rp;
    q23[g] = ab.y;
    ri1[g] = ri01.y;
    ri3[g] = ri23.y;
  }
  float wend = ex2(r1 + logsum);   // product of (1 - beta) over everything after the chunk
#pragma unroll
  for (int g = 3; g >= 0; --g) {
    const float2 w32 = mul2(make_float2(wend, wend), make_float2(ri3[g], q23[g]));   // inclusive products at columns 3, 2
    const float w1 = w32.y * ri1[g];                                                  // at column 1
    wend *= rpg[g];                                                                   // at column 0 = after the previous group
    const float2 a01 = mul2(e01[g], make_float2(wend, w1));
    const float2 a23 = mul2(e23[g], make_float2(w32.y, w32.x));
    pa[4 * g] = a01.x;
    pa[4 * g + 1] = a01.y;
    pa[4 * g + 2] = a23.x;
    pa[4 * g + 3] = a23.y;
  }
  const float2 ndr = make_float2(-dr, -dr);
  float cb = gpre + gs, csum = 0.f;   // C before the group; the chunk's own sum of G
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float2 g01 = mul2(make_float2(pa[4 * g], pa[4 * g + 1]),
                      add2(make_float2(__uint_as_float(dp[4 * g]), __uint_as_float(dp[4 * g + 1])), ndr));
    float2 g23 = mul2(make_float2(pa[4 * g + 2], pa[4 * g + 3]),
                      add2(make_float2(__uint_as_float(dp[4 * g + 2]), __uint_as_float(dp[4 * g + 3])), ndr));
    if (kMasked) {   // rows past the sequence end carry arbitrary values: select, do not rely on 0 * x
      const int col = mc0 + 4 * g;
      if (!(col < limit)) { g01.x = 0.f; pa[4 * g] = 0.f; }
      if (!(col + 1 < limit)) { g01.y = 0.f; pa[4 * g + 1] = 0.f; }
      if (!(col + 2 < limit)) { g23.x = 0.f; pa[4 * g + 2] = 0.f; }
      if (!(col + 3 < limit)) { g23.y = 0.f; pa[4 * g + 3] = 0.f; }
    }
    const float t1 = g01.x + g01.y, t23 = g23.x + g23.y;
    const float tg = t1 + t23;
    const float c0v = cb + g01.x, c1v = cb + t1;
    const float c2v = c1v + g23.x;
    cb += tg;
    csum += tg;
    const float2 z01 = fma2(make_float2(-be01[g].x, -be01[g].y), make_float2(c0v, c1v), g01);
    const float2 z23 = fma2(make_float2(-be23[g].x, -be23[g].y), make_float2(c2v, cb), g23);
    pz[4 * g] = z01.x;
    pz[4 * g + 1] = z01.y;
    pz[4 * g + 2] = z23.x;
    pz[4 * g + 3] = z23.y;
    if (kMasked) {
#pragma unroll
      for (int i = 0; i < 4; ++i) pz[4 * g + i] = row_valid ? pz[4 * g + i] : 0.f;
    }
  }
  gs += csum;
}

// The same, written to the 16-bit A (optional) and dz tiles; c0 addresses the output tile.
template <bool kFp16, bool kStoreA, bool kMasked>
__device__ __forceinline__ void bwd_row_chunk(const uint32_t (&s)[16], const uint32_t (&dp)[16], int c0, int mc0, int r, bool diag,
                                              int ac, bool row_valid, float scale2, float r1, float gpre, float dr,
                                              float &gs, float &logsum, uint8_t *tile_a, uint8_t *tile_z,
                                              bool skip_zero = false) {
  float pa[16], pz[16];
  bwd_row_chunk_values<kMasked>(s, dp, mc0, r, diag, ac, row_valid, scale2, r1, gpre, dr, gs, logsum, pa, pz, skip_zero);
  if constexpr (kStoreA) store_row_chunk16<kFp16>(tile_a, r, c0, pa);
  store_row_chunk16<kFp16>(tile_z, r, c0, pz);
}

// One row of a 64-key strip: four 16-column chunks, TMEM read one chunk ahead.  mc0: key index of the strip's first
// column inside its 128-key tile (for the diagonal mask).  empty_bar (optional) is signalled, one arrival per warp,
// once the last S/dP columns are in registers; gate_bar (optional) is waited for before the first store to the
// output tiles, i.e. after the first chunk's arithmetic.  az_a / az_z (optional): this row's 64 values of the stored
// A and dz tiles in global memory (plain row-major, 16-bit), written next to the shared-memory dz tile (the caller may
// instead copy the finished dz tile out of shared memory).
// Returns false if the gate wait gave up.
template <bool kFp16, bool kStoreA, bool kMasked>
__device__ __forceinline__ bool strip_row_pass(uint32_t ts, uint32_t tp, int r, int mc0, bool diag, int ac, bool row_valid,
                                              float scale2, float r1, float gpre, float dr, float &gs, float &logsum,
                                              uint8_t *tile_a, uint8_t *tile_z, float *mid_r1 = nullptr,
                                              float *mid_s2 = nullptr, uint32_t empty_bar = 0, uint32_t gate_bar = 0,
                                              uint32_t gate_parity = 0, unsigned short *az_a = nullptr,
                                              unsigned short *az_z = nullptr, bool skip_zero = false) {
  uint32_t s0[16], d0[16], s1[16], d1[16];
  bool ok = true;
  tmem_ld16(ts, s0);
  tmem_ld16(tp, d0);
#pragma unroll 1
  for (int pair = 0; pair < 2; ++pair) {
    const int c0 = pair * 32;
    tmem_wait_ld_regs(s0, d0);
    tmem_ld16(ts + c0 + 16, s1);
    tmem_ld16(tp + c0 + 16, d1);
    {
      float pa[16], pz[16];
      bwd_row_chunk_values<kMasked>(s0, d0, mc0 + c0, r, diag, ac, row_valid, scale2, r1, gpre, dr, gs, logsum, pa, pz, skip_zero);
      if (pair == 0 && gate_bar != 0) {
        ok = mbar_wait(gate_bar, gate_parity);
        tc_fence_after();
      }
      if constexpr (kStoreA) store_row_chunk16<kFp16>(tile_a, r, c0, pa);
      uint32_t wz[8];
      pack_row_chunk16<kFp16>(pz, wz);
      store_packed_chunk16(tile_z, r, c0, wz);
      if (az_a != nullptr) {
        uint32_t wa[8];
        pack_row_chunk16<kFp16>(pa, wa);
        store_packed_global16(az_a + c0, wa);
        if (az_z != nullptr) store_packed_global16(az_z + c0, wz);
      }
    }
    tmem_wait_ld_regs(s1, d1);
    if (pair == 0) {
      tmem_ld16(ts + 32, s0);
      tmem_ld16(tp + 32, d0);
    } else if (empty_bar != 0) {   // the last columns are in registers: the S/dP slots can be overwritten
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(empty_bar);
    }
    {
      float pa[16], pz[16];
      bwd_row_chunk_values<kMasked>(s1, d1, mc0 + c0 + 16, r, diag, ac, row_valid, scale2, r1, gpre, dr, gs, logsum, pa, pz, skip_zero);
      if constexpr (kStoreA) store_row_chunk16<kFp16>(tile_a, r, c0 + 16, pa);
      uint32_t wz[8];
      pack_row_chunk16<kFp16>(pz, wz);
      store_packed_chunk16(tile_z, r, c0 + 16, wz);
      if (az_a != nullptr) {
        uint32_t wa[8];
        pack_row_chunk16<kFp16>(pa, wa);
        store_packed_global16(az_a + c0 + 16, wa);
        if (az_z != nullptr) store_packed_global16(az_z + c0 + 16, wz);
      }
    }
    if (pair == 0 && mid_r1 != nullptr) {   // the carried values after 32 of the 64 columns
      *mid_r1 = r1 + logsum;
      *mid_s2 = gpre + gs;
    }
  }
  return ok;
}

// =======================================================================================================
// dq kernel for head sizes 72..128: 256 query rows per CTA
// =======================================================================================================
// Two adjacent 128-row query tiles (a, b) share one stream of 64-key K/V sub-tiles, walked from the sequence start
// to tile b's diagonal.  Each tile has its own row-owning warpgroup (warps 0-3 / 4-7), MMA issuer (warps 9 / 10),
// S/dP slots and dQ accumulator in TMEM and dz tile in shared memory.  Per sub-tile and tile: S = Q K^T and
// dP = dO V^T (128 x 64), the row pass (which also records R1/S2 at the sub-tile's first key, i.e. at keys 0 and 64
// of every 128-key tile), then dQ += dz K.
// TMEM columns: S_a 0, dP_a 64, S_b 128, dP_b 192, dQ_a 256, dQ_b 384.
namespace dq2 {
constexpr int kThreads = 352;
constexpr int kBN = 64;
constexpr int kStages = 2;
constexpr int kTileBytes = kBM * 128 * 2;      // Q or dO tile
constexpr int kKvBox = kBN * 64 * 2;           // 64 keys x 64 columns
constexpr int kKvTile = 2 * kKvBox;            // K or V sub-tile
constexpr int kStageBytes = 2 * kKvTile;
constexpr int kZBytes = kBM * kBN * 2;         // dz tile: 128 rows x 64 keys
constexpr int kSmem = 1024 + 4 * kTileBytes + kStages * kStageBytes + 2 * kZBytes + 512;
enum { bQG = 0, bKvFull = 1, bKvEmpty = 3, bSpFull = 5, bZFull = 7, bZEmpty = 9, bFirst = 11, bSpEmpty = 12, bDqFull = 14, bNum = 16 };
}  // namespace dq2

template <bool kFp16>
__global__ void __launch_bounds__(dq2::kThreads, 1)
tc_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                  const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_az, const KParams p) {
  using namespace dq2;
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0) trace_block(p, 0);
  if (p.hdr[0]) return;
  TileCoord c;
  int hh_blk;
  if (!decode_block(p, 2, true, c, hh_blk)) return;   // c.idx: the even tile of the pair (idx, idx + 1)
  const int Ia = c.idx;
  const bool b_active = Ia + 1 < c.n_tiles;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  const uint32_t sQ = base;                     // tile w: Q at sQ + w * 2 * kTileBytes, dO right behind it
  const uint32_t sKV = sQ + 4 * kTileBytes;     // stage: K sub-tile then V sub-tile
  const uint32_t sZ = sKV + kStages * kStageBytes;
  const uint32_t sBar = sZ + 2 * kZBytes;
  Ctl *ctl = reinterpret_cast<Ctl *>(gbase + (sBar - base) + bNum * 8);
  volatile int *abort_flag = &ctl->abort;
  auto bar = [&](int i) { return sBar + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hh = hh_blk, h = p.head0 + hh;
  const int n_sub = (c.len + kBN - 1) / kBN;
  const int steps_a = min(2 * Ia + 2, n_sub);            // sub-tiles 0 .. 2 Ia + 1 reach tile a's diagonal
  const int steps_b = b_active ? min(2 * Ia + 4, n_sub) : 0;
  const int n_steps = b_active ? steps_b : steps_a;
  const int issuers = b_active ? 2 : 1;
  int tr_cur = 0;   // cursor of this thread's event-log lane (diagnostics)

  if (threadIdx.x == 0) {
    mbar_init(bar(bQG), 1);
    mbar_init(bar(bFirst), 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(bar(bKvFull + s), 1); mbar_init(bar(bKvEmpty + s), issuers); }
    for (int w = 0; w < 2; ++w) {
      mbar_init(bar(bSpFull + w), 1);
      mbar_init(bar(bZFull + w), 4);
      mbar_init(bar(bZEmpty + w), 1);
      mbar_init(bar(bSpEmpty + w), 4);
    }
    mbar_init(bar(bDqFull), 1);
    mbar_init(bar(bDqFull + 1), 1);
    ctl->abort = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 8) {
    if (lane == 0) {
      prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v); prefetch_tensormap(&tm_g);
      const int qrow = (int)c.tok0 + Ia * kBM;
      mbar_arrive_expect_tx(bar(bQG), 4 * kTileBytes);
      for (int w = 0; w < 2; ++w)
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_4d(sQ + w * 2 * kTileBytes + kb * kBoxBytes, &tm_q, bar(bQG), kb * 64, qrow + w * kBM, h, (int)c.boff);
          tma_load_4d(sQ + w * 2 * kTileBytes + kTileBytes + kb * kBoxBytes, &tm_g, bar(bQG), kb * 64, qrow + w * kBM, h, (int)c.boff);
        }
      for (int t = 0; t < n_steps; ++t) {
        const int st = t % kStages;
        if (t >= kStages && !wait_or_abort(bar(bKvEmpty + st), ((t / kStages) - 1) & 1, abort_flag, p, 510)) break;
        if (*abort_flag) break;
        const int krow = (int)c.tok0 + t * kBN;
        const uint32_t dst = sKV + st * kStageBytes;
        mbar_arrive_expect_tx(bar(bKvFull + st), kStageBytes);
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_4d(dst + kb * kKvBox, &tm_k, bar(bKvFull + st), kb * 64, krow, h, (int)c.boff);
          tma_load_4d(dst + kKvTile + kb * kKvBox, &tm_v, bar(bKvFull + st), kb * 64, krow, h, (int)c.boff);
        }
      }
    }
  } else if (warp >= 9) {
    // ------------------------------------------------ MMA issuers, one per tile
    const int w = warp - 9;
    if (lane == 0 && w < issuers) {
      constexpr uint32_t idesc_s = idesc_f16(kBM, kBN, kFp16, false, false);
      constexpr uint32_t idesc_dq = idesc_f16(kBM, D, kFp16, false, true);
      const uint32_t qaddr = sQ + w * 2 * kTileBytes, gaddr = qaddr + kTileBytes, zaddr = sZ + w * kZBytes;
      const uint32_t tS = tmem + w * 128, tP = tS + 64, tDQ = tmem + 256 + w * 128;
      const int my_steps = w == 0 ? steps_a : steps_b;
      auto issue_sp = [&](int t) {
        const uint32_t kaddr = sKV + (t % kStages) * kStageBytes;
        mma_kmajor_kmajor<D, kBoxBytes, kKvBox>(tS, qaddr, kaddr, idesc_s, false);            // S = Q K^T
        mma_kmajor_kmajor<D, kBoxBytes, kKvBox>(tP, gaddr, kaddr + kKvTile, idesc_s, false);  // dP = dO V^T
        mma_commit(bar(bSpFull + w));
      };
      bool ok = wait_or_abort(bar(bQG), 0, abort_flag, p, 520) && wait_or_abort(bar(bKvFull), 0, abort_flag, p, 521);
      // tile b starts once tile a's first scores are done, so that one tile's MMAs fall into the other's row pass
      // (bFirst completes exactly once: this waiter does not follow the phases of tile a's own barriers)
      if (ok && w == 1 && steps_a > 0) ok = wait_or_abort(bar(bFirst), 0, abort_flag, p, 525);
      if (ok) {
        tc_fence_after();
        issue_sp(0);
        if (w == 0) mma_commit(bar(bFirst));
      }
      for (int u = 0; ok && u < my_steps; ++u) {
        // the rows of step u have read their S/dP (they are still computing): the next scores go first ...
        if (u + 1 < my_steps) {
          ok = wait_or_abort(bar(bSpEmpty + w), u & 1, abort_flag, p, 526) &&
               wait_or_abort(bar(bKvFull + (u + 1) % kStages), ((u + 1) / kStages) & 1, abort_flag, p, 523);
          if (!ok) break;
          trace_event(p, 1 + 3 * w, tr_cur, 2 + 16 * w, u + 1);
          tc_fence_after();
          issue_sp(u + 1);
          trace_event(p, 1 + 3 * w, tr_cur, 3 + 16 * w, u + 1);
        }
        // ... then, once its dz tile is written, this step's dQ
        ok = wait_or_abort(bar(bZFull + w), u & 1, abort_flag, p, 522);
        if (!ok) break;
        trace_event(p, 1 + 3 * w, tr_cur, 6 + 16 * w, u);
        tc_fence_after();
        // dQ += dz K: dz [128 x 64] K-major, K sub-tile [64 keys x (2 x 64) columns] MN-major
        mma_kmajor_mnmajor<kBN, kKvBox>(tDQ, zaddr, sKV + (u % kStages) * kStageBytes, idesc_dq, u > 0);
        mma_commit(bar(bZEmpty + w));
        mma_commit(bar(bKvEmpty + u % kStages));
      }
      if (ok) mma_commit(bar(bDqFull + w));   // this tile's dQ is complete: its rows store it while the other tile goes on
      // tile a does not read the last sub-tiles: release them on its behalf once they have arrived
      for (int t = my_steps; ok && t < n_steps; ++t) {
        ok = wait_or_abort(bar(bKvFull + t % kStages), (t / kStages) & 1, abort_flag, p, 524);
        if (ok) mbar_arrive(bar(bKvEmpty + t % kStages));
      }
    }
  } else {
    // ------------------------------------------------ rows: warpgroup w owns query tile Ia + w
    using T = typename std::conditional<kFp16, __half, __nv_bfloat16>::type;
    const int w = warp >> 2;
    const int r = threadIdx.x & 127;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float scale2 = p.scale * kLog2e;
    const int I = Ia + w;
    const int my_steps = w == 0 ? steps_a : steps_b;
    const int gi = I * kBM + r;
    const bool valid = gi < c.len;
    const long long idx = (c.boff * p.heads + h) * p.tokens + c.tok0 + gi;
    double r1 = (valid && my_steps > 0) ? p.log_rem[idx] : 0.0;   // sum of log2(1-beta) over the keys from the current one on
    const float dr = (valid && my_steps > 0) ? load_drem<T>(p, idx) : 0.f;
    float gpre = 0.f;
    uint8_t *gZ = gbase + (sZ - base) + w * kZBytes;
    const uint32_t tS = tmem + w * 128 + lane_off, tP = tS + 64;
    // boundary records: [pair (I, J)][half][row]; sub-tile u is half u & 1 of key tile u >> 1
    const long long rec0 = ((long long)hh * p.pairs_cap + c.pair0 + (long long)I * (I + 1) / 2) * (4 * kBM) + r;
    const bool ragged = I * kBM + kBM > c.len;   // the sequence ends inside this tile
    bool ok = true;
    for (int u = 0; u < my_steps && ok; ++u) {
      ok = wait_or_abort(bar(bSpFull + w), u & 1, abort_flag, p, 530);
      if (!ok) break;
      if (threadIdx.x == 0 && u == 0) trace_block(p, 1);
      if (r == 0) trace_event(p, 2 + w, tr_cur, 4 + 16 * w, u);
      tc_fence_after();
      // the dz tile is still being read by the previous step's dQ MMAs: waited for inside the pass, before its first store
      const uint32_t gate = u >= 1 ? bar(bZEmpty + w) : 0u, gate_parity = (u - 1) & 1;
      const float r1f = (float)r1;
      float gs = 0.f, logsum = 0.f;
      bool pass_ok;
      // a tile with rows past the sequence end takes the masking variant throughout: those rows must be zero in the
      // stored tiles (the dK/dV GEMMs sum over all 128 query rows)
      const bool on_diag = u >= 2 * I;
      if (p.az != nullptr) {
        // stored-tiles mode: this row's 64 values of A and dz for key tile u >> 1, half u & 1
        const long long pair = c.pair0 + (long long)I * (I + 1) / 2 + (u >> 1);
        unsigned short *az_a = p.az + ((((long long)hh * 2) * p.pairs_cap + pair) * kBM + r) * kBM + (u & 1) * kBN;
        unsigned short *az_z = nullptr;   // the dz tile leaves by TMA below
        // this warp's copy of the previous step's dz rows has left shared memory before they are rewritten
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        if (on_diag || ragged)
          pass_ok = strip_row_pass<kFp16, false, true>(tS, tP, r, on_diag ? (u - 2 * I) * kBN : 0, on_diag, p.attend_current, valid,
                                                       scale2, r1f, gpre, dr, gs, logsum, nullptr, gZ, nullptr, nullptr,
                                                       bar(bSpEmpty + w), gate, gate_parity, az_a, az_z);
        else
          pass_ok = strip_row_pass<kFp16, false, false>(tS, tP, r, 0, false, 0, true, scale2, r1f, gpre, dr, gs, logsum, nullptr, gZ,
                                                        nullptr, nullptr, bar(bSpEmpty + w), gate, gate_parity, az_a, az_z, !p.dense);
      } else {
        float *rec_r1 = p.bnd_r1 + rec0 + (long long)u * (2 * kBM);   // quarter 2 (u & 1) of key tile u >> 1
        float *rec_s2 = p.bnd_s2 + rec0 + (long long)u * (2 * kBM);
        rec_r1[0] = r1f;
        rec_s2[0] = gpre;
        if (on_diag)
          pass_ok = strip_row_pass<kFp16, false, true>(tS, tP, r, (u - 2 * I) * kBN, true, p.attend_current, true, scale2, r1f, gpre,
                                                       dr, gs, logsum, nullptr, gZ, rec_r1 + kBM, rec_s2 + kBM, bar(bSpEmpty + w),
                                                       gate, gate_parity);
        else
          pass_ok = strip_row_pass<kFp16, false, false>(tS, tP, r, 0, false, 0, true, scale2, r1f, gpre, dr, gs, logsum, nullptr, gZ,
                                                        rec_r1 + kBM, rec_s2 + kBM, bar(bSpEmpty + w), gate, gate_parity, nullptr,
                                                        nullptr, !p.dense);
      }
      if (!pass_ok) {   // the bounded wait inside the pass gave up
        *abort_flag = 1;
        if (p.status != nullptr) { p.status[0] = SB_DEV_WAIT_TIMEOUT; p.status[1] = 531; }
        ok = false;
      }
      r1 += (double)logsum;
      gpre += gs;
      // the sequence ends inside this sub-tile: its dz columns behind the end are exact zeros, the K rows there are
      // not this sequence's (see zero_tile_rows) and are cleared before this step's dz K MMA is released
      if (c.len - u * kBN < kBN)
        zero_tile_rows(gbase + (sKV - base) + (u % kStages) * kStageBytes, c.len - u * kBN, kBN, 2, kKvBox, r, kBM);
      tc_fence_before();          // this step's TMEM reads are done before the slots are handed back
      fence_proxy_async_smem();
      __syncwarp();
      if (r == 0) trace_event(p, 2 + w, tr_cur, 5 + 16 * w, u);
      if (lane == 0) {
        mbar_arrive(bar(bZFull + w));
        if (p.az != nullptr) {   // stored-tiles mode: this warp's 32 rows x 64 keys of dz, out of the shared-memory tile
          const long long pair = c.pair0 + (long long)I * (I + 1) / 2 + (u >> 1);
          tma_store_4d(&tm_az, sZ + w * kZBytes + (warp & 3) * 32 * 128, (u & 1) * kBN, (int)(pair * kBM) + (warp & 3) * 32, 1, hh);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait_read();   // the dz buffer is reused by the epilogue
    __syncwarp();
    if (ok && my_steps > 0) ok = wait_or_abort(bar(bDqFull + w), 0, abort_flag, p, 532);
    if (ok && my_steps > 0) {
      tc_fence_after();
      const uint32_t t_acc = tmem + 256 + w * 128 + lane_off;
      if (I * kBM + kBM <= c.len) {
        // full tile: two 64-column halves through this tile's dz buffer (its last dQ MMA is done), one TMA store per
        // warp and half -- full lines instead of 16 bytes per thread and row
        const uint32_t src = sZ + w * kZBytes + (warp & 3) * 32 * 128;
        const int trow = (int)c.tok0 + I * kBM + (warp & 3) * 32;
#pragma unroll 1
        for (int half = 0; half < (p.head_dim > 64 ? 2 : 1); ++half) {   // columns past head_dim do not exist
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t v[32];
            tmem_ld32(t_acc + half * 64 + ch * 32, v);
            tmem_wait_ld();
            float x[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(v[i]) * p.scale;
            store_row_chunk<kFp16>(gZ, r, ch * 32, x);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&tm_dq, src, half * 64, trow, h, (int)c.boff);
            tma_store_commit();
            tma_store_wait_read();   // the buffer is rewritten by the next half
          }
          __syncwarp();
        }
        if (lane == 0) tma_store_wait_all();
      } else {
        // the sequence ends inside the tile: row by row, rows past the end are left alone
        T *grow = reinterpret_cast<T *>(p.dq.ptr) + c.boff * p.dq.sb + (long long)h * p.dq.sh + (c.tok0 + gi) * p.dq.st;
        store_acc_rows<D, kFp16, T>(t_acc, grow, valid, p.head_dim, p.scale);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace_block(p, 2);
  if (warp == 9) tmem_dealloc(tmem, kTmemCols);
}

// =======================================================================================================
// dkv kernel for head sizes 72..128, pipelined: one CTA per 128-key tile, all eight row warps on one query tile
// =======================================================================================================
// The key tile is handled as two 64-key strips (h = 0, 1) that share every Q/dO tile: a step is one query tile
// against one strip, and the two steps of a query tile use the same Q/dO stage, so Q/dO are loaded once per
// 128 keys.  Within a step, warps 0-3 own key columns 0..31 of the strip and warps 4-7 columns 32..63 for the same
// 128 query rows; each group restarts from its own R1/S2 record (the dq kernel records them every 32 keys), so the
// groups are independent.  S/dP are double-buffered in TMEM and the Q/dO tiles sit in a two-stage ring: the S/dP
// MMAs of step g+1 (issuer warp 9) and the dK^T/dV^T MMAs of step g-1 (issuer warp 10) run while the rows of
// step g are processed.  The A/dz tiles are single-buffered; the rows wait for the previous step's dK^T/dV^T MMAs
// only before their first store, i.e. after a quarter of the step's arithmetic.
// TMEM columns: S[slot] at 128 slot, dP[slot] at 128 slot + 64, dK^T[h] at 256 + 128 h, dV^T[h] at 320 + 128 h.
namespace dkv4 {
constexpr int kThreads = 352;
constexpr int kBN = 64;
constexpr int kTileBytes = kBM * 128 * 2;      // Q, dO, K or V tile: two 128 x 64 boxes
constexpr int kStripOffset = kBN * 128;        // byte offset of strip 1 inside a box (64 rows of 128 bytes)
constexpr int kAzBytes = kBM * kBN * 2;        // A or dz tile, 128 rows x 64 keys
constexpr int kSmem = 1024 + 2 * kTileBytes + 4 * kTileBytes + 2 * kAzBytes + 512;
enum { bKV = 0, bQgFull = 1, bQgEmpty = 3, bSpFull = 5, bSpEmpty = 7, bAzFull = 9, bAzEmpty = 10, bOutFull = 11, bStaged = 12,
       bDrained = 14, bNum = 16 };
}  // namespace dkv4

template <bool kFp16>
__global__ void __launch_bounds__(dkv4::kThreads, 1)
tc_bwd_dkv4_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                   const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv, const KParams p) {
  using namespace dkv4;
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0) trace_block(p, 0);
  if (p.hdr[0]) return;
  TileCoord c;
  int hh_blk;
  if (!decode_block(p, 1, false, c, hh_blk)) return;
  const int J = c.idx;                         // the 128-key tile
  const int n_halves = J * kBM + kBN < c.len ? 2 : 1;   // the sequence may end inside the first strip

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  const uint32_t sK = base;
  const uint32_t sV = sK + kTileBytes;
  const uint32_t sQ = sV + kTileBytes;               // stage b: Q at sQ + b * 2 * kTileBytes, dO right behind it
  const uint32_t sAZ = sQ + 4 * kTileBytes;          // A, then dz
  const uint32_t sBar = sAZ + 2 * kAzBytes;
  Ctl *ctl = reinterpret_cast<Ctl *>(gbase + (sBar - base) + bNum * 8);
  volatile int *abort_flag = &ctl->abort;
  auto bar = [&](int i) { return sBar + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hh = hh_blk, h = p.head0 + hh;
  const int cnt = c.n_tiles - J;               // query tiles J .. n_tiles-1
  const int n_steps = cnt * n_halves;          // step g: query tile J + g / n_halves, strip g % n_halves
  const int hshift = n_halves - 1;
  int tr_cur = 0;   // cursor of this thread's event-log lane (diagnostics)

  if (threadIdx.x == 0) {
    mbar_init(bar(bKV), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(bQgFull + b), 1);
      mbar_init(bar(bQgEmpty + b), 1);
      mbar_init(bar(bSpFull + b), 1);
      mbar_init(bar(bSpEmpty + b), 8);
    }
    mbar_init(bar(bAzFull), 8);
    mbar_init(bar(bAzEmpty), 1);
    mbar_init(bar(bOutFull), 1);
    for (int b = 0; b < 2; ++b) { mbar_init(bar(bStaged + b), 4); mbar_init(bar(bDrained + b), 1); }
    ctl->abort = 0;
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 8) {
    if (lane == 0) {
      prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v); prefetch_tensormap(&tm_g);
      const int krow = (int)c.tok0 + J * kBM;
      mbar_arrive_expect_tx(bar(bKV), 2 * kTileBytes);
      for (int kb = 0; kb < 2; ++kb) {
        tma_load_4d(sK + kb * kBoxBytes, &tm_k, bar(bKV), kb * 64, krow, h, (int)c.boff);
        tma_load_4d(sV + kb * kBoxBytes, &tm_v, bar(bKV), kb * 64, krow, h, (int)c.boff);
      }
      for (int u = 0; u < cnt; ++u) {
        const int b = u & 1;
        if (u >= 2 && !wait_or_abort(bar(bQgEmpty + b), ((u >> 1) - 1) & 1, abort_flag, p, 610)) break;
        if (*abort_flag) break;
        const int qrow = (int)c.tok0 + (J + u) * kBM;
        const uint32_t dst = sQ + b * 2 * kTileBytes;
        trace_event(p, 0, tr_cur, 1, u);
        mbar_arrive_expect_tx(bar(bQgFull + b), 2 * kTileBytes);
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_4d(dst + kb * kBoxBytes, &tm_q, bar(bQgFull + b), kb * 64, qrow, h, (int)c.boff);
          tma_load_4d(dst + kTileBytes + kb * kBoxBytes, &tm_g, bar(bQgFull + b), kb * 64, qrow, h, (int)c.boff);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------ issuer of S = Q K^T and dP = dO V^T (128 x 64)
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_f16(kBM, kBN, kFp16, false, false);
      bool ok = wait_or_abort(bar(bKV), 0, abort_flag, p, 620);
      for (int g = 0; ok && g < n_steps; ++g) {
        const int u = g >> hshift, hf = g & hshift, b = u & 1, slot = g & 1;
        ok = wait_or_abort(bar(bQgFull + b), (u >> 1) & 1, abort_flag, p, 621);
        // the rows of step g-2 have read this S/dP slot
        if (ok && g >= 2) ok = wait_or_abort(bar(bSpEmpty + slot), ((g >> 1) - 1) & 1, abort_flag, p, 622);
        if (!ok) break;
        trace_event(p, 1, tr_cur, 2, g);
        tc_fence_after();
        const uint32_t qaddr = sQ + b * 2 * kTileBytes;
        mma_kmajor_kmajor<D>(tmem + slot * 128, qaddr, sK + hf * kStripOffset, idesc_s, false);
        mma_kmajor_kmajor<D>(tmem + slot * 128 + 64, qaddr + kTileBytes, sV + hf * kStripOffset, idesc_s, false);
        mma_commit(bar(bSpFull + slot));
        trace_event(p, 1, tr_cur, 3, g);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------ issuer of dK^T += Q^T dz and dV^T += dO^T A (128 x 64)
    if (lane == 0) {
      constexpr uint32_t idesc_t = idesc_f16(kBM, kBN, kFp16, true, true);
      const uint64_t a0 = smem_desc_sw128(sAZ, 16, 1024), z0 = smem_desc_sw128(sAZ + kAzBytes, 16, 1024);
      bool ok = true;
      for (int g = 0; ok && g < n_steps; ++g) {
        const int u = g >> hshift, hf = g & hshift, b = u & 1;
        ok = wait_or_abort(bar(bAzFull), g & 1, abort_flag, p, 623);
        if (!ok) break;
        trace_event(p, 4, tr_cur, 6, g);
        tc_fence_after();
        const uint32_t qaddr = sQ + b * 2 * kTileBytes;
        const uint64_t q0 = smem_desc_sw128(qaddr, kBoxBytes, 1024), g0 = smem_desc_sw128(qaddr + kTileBytes, kBoxBytes, 1024);
        const uint32_t t_dk = tmem + 256 + hf * 128, t_dv = t_dk + 64;
#pragma unroll
        for (int ks = 0; ks < kBM / 16; ++ks)
          mma_f16_ss(t_dk, q0 + (uint64_t)(ks * 128), z0 + (uint64_t)(ks * 128), idesc_t, u > 0 || ks > 0);
#pragma unroll
        for (int ks = 0; ks < kBM / 16; ++ks)
          mma_f16_ss(t_dv, g0 + (uint64_t)(ks * 128), a0 + (uint64_t)(ks * 128), idesc_t, u > 0 || ks > 0);
        mma_commit(bar(bAzEmpty));
        if (hf == hshift) mma_commit(bar(bQgEmpty + b));   // the tile's last strip: its Q/dO stage is free
        trace_event(p, 4, tr_cur, 7, g);
      }
      if (ok) mma_commit(bar(bOutFull));
    }
  } else {
    // ------------------------------------------------ rows: warps 0-3 columns 0..31, warps 4-7 columns 32..63
    using T = typename std::conditional<kFp16, __half, __nv_bfloat16>::type;
    const int w = warp >> 2;
    const int r = threadIdx.x & 127;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float scale2 = p.scale * kLog2e;
    bool ok = true;
    // the per-row start values of a step come from global memory: they are fetched one step ahead
    // (the gradient of rem stays a raw 16-bit value until the step that uses it, so that nothing in this step depends
    // on the load)
    auto fetch = [&](int g, float &r1f, float &gpre, unsigned short &dr_raw) {
      const int I = J + (g >> hshift), quarter = 2 * (g & hshift) + w;   // which 32-key quarter of the 128-key tile
      const int gi = I * kBM + r;
      const long long slot = (((long long)hh * p.pairs_cap + c.pair0 + (long long)I * (I + 1) / 2 + J) * 4 + quarter) * kBM + r;
      r1f = p.bnd_r1[slot];
      gpre = p.bnd_s2[slot];
      const long long row = (c.boff * p.heads + h) * p.tokens + c.tok0 + min(gi, c.len - 1);
      dr_raw = reinterpret_cast<const unsigned short *>(p.d_rem)[row];
    };
    uint8_t *gA = gbase + (sAZ - base);
    uint8_t *gZ = gA + kAzBytes;
    float nr1, ngpre;
    unsigned short ndr;
    fetch(0, nr1, ngpre, ndr);
    for (int g = 0; g < n_steps && ok; ++g) {
      const int u = g >> hshift, hf = g & hshift, slot = g & 1;
      const int I = J + u;
      const int quarter = 2 * hf + w;
      const bool valid = I * kBM + r < c.len;
      const float r1f = nr1, gpre = ngpre;
      const float dr = valid ? to_f32<T>(*reinterpret_cast<const T *>(&ndr)) : 0.f;
      if (g + 1 < n_steps) fetch(g + 1, nr1, ngpre, ndr);
      ok = wait_or_abort(bar(bSpFull + slot), (g >> 1) & 1, abort_flag, p, 630);
      if (!ok) break;
      if (threadIdx.x == 0 && g == 0) trace_block(p, 1);
      if (r == 0) trace_event(p, 2 + w, tr_cur, 4 + 16 * w, g);
      tc_fence_after();
      const uint32_t tS = tmem + slot * 128 + w * 32 + lane_off, tP = tS + 64;
      float gs = 0.f, logsum = 0.f;
      const bool diag = (u == 0);
      const bool masked = diag || (I == c.n_tiles - 1 && (c.len & (kBM - 1)) != 0);
      // On the diagonal tile the quarters after this warp's last row are masked for all of its 32 rows, and a warp whose
      // rows all lie past the sequence end has nothing allowed anywhere: A and dz are zero, the scores are not read.
      const bool skip = (diag && quarter * 32 >= (r | 31) + p.attend_current) || I * kBM + (r & ~31) >= c.len;
      if (!skip) {
        uint32_t s0[16], d0[16], s1[16], d1[16];
        tmem_ld16(tS, s0);
        tmem_ld16(tP, d0);
        tmem_wait_ld_regs(s0, d0);
        tmem_ld16(tS + 16, s1);
        tmem_ld16(tP + 16, d1);
        {
          float pa[16], pz[16];
          if (masked)
            bwd_row_chunk_values<true>(s0, d0, quarter * 32, r, diag, p.attend_current, valid, scale2, r1f, gpre, dr, gs, logsum, pa, pz);
          else
            bwd_row_chunk_values<false>(s0, d0, 0, r, false, 0, true, scale2, r1f, gpre, dr, gs, logsum, pa, pz, !p.dense);
          // the A/dz tiles are still being read by the previous step's MMAs
          if (g >= 1) {
            ok = wait_or_abort(bar(bAzEmpty), (g - 1) & 1, abort_flag, p, 631);
            tc_fence_after();
          }
          store_row_chunk16<kFp16>(gA, r, w * 32, pa);
          store_row_chunk16<kFp16>(gZ, r, w * 32, pz);
        }
        tmem_wait_ld_regs(s1, d1);
        tc_fence_before();          // this step's TMEM reads are done: the S/dP slot is handed back
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(bSpEmpty + slot));
        if (masked)
          bwd_row_chunk<kFp16, true, true>(s1, d1, w * 32 + 16, quarter * 32 + 16, r, diag, p.attend_current, valid, scale2, r1f,
                                           gpre, dr, gs, logsum, gA, gZ);
        else
          bwd_row_chunk<kFp16, true, false>(s1, d1, w * 32 + 16, 0, r, false, 0, true, scale2, r1f, gpre, dr, gs, logsum, gA, gZ,
                                            !p.dense);
      } else {
        if (g >= 1) {
          ok = wait_or_abort(bar(bAzEmpty), (g - 1) & 1, abort_flag, p, 631);
          tc_fence_after();
        }
        const uint32_t zero[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          store_packed_chunk16(gA, r, w * 32 + 16 * q, zero);
          store_packed_chunk16(gZ, r, w * 32 + 16 * q, zero);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(bSpEmpty + slot));
      }
      // the sequence ends inside this query tile: the A and dz rows behind the end are exact zeros, the Q and dO rows
      // there are not this sequence's (see zero_tile_rows) and are cleared before this step's MMAs are released
      if (c.len - I * kBM < kBM)
        zero_tile_rows(gbase + (sQ - base) + (u & 1) * 2 * kTileBytes, c.len - I * kBM, kBM, 4, kBoxBytes, threadIdx.x, 2 * kBM);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(bAzFull));
      if (r == 0) trace_event(p, 2 + w, tr_cur, 5 + 16 * w, g);
    }
    // ---- epilogue: dK^T (warps 0-3) and dV^T (warps 4-7), lanes = head dimension, columns = keys.  A full strip is
    // transposed into this warpgroup's buffer (A for dK, dz for dV: all their MMAs are done) and leaves by TMA;
    // a strip the sequence ends in is written element by element.
    if (ok) ok = wait_or_abort(bar(bOutFull), 0, abort_flag, p, 632);
    if (ok) {
      tc_fence_after();
      const TensorRef &out = w == 0 ? p.dk : p.dv;
      const CUtensorMap *omap = w == 0 ? &tm_dk : &tm_dv;
      const float mul = w == 0 ? p.scale : 1.f;
      uint8_t *stage = w == 0 ? gA : gZ;
      const uint32_t stage_addr = sAZ + w * kAzBytes;
      T *obase = reinterpret_cast<T *>(out.ptr) + c.boff * out.sb + (long long)h * out.sh + (c.tok0 + J * kBM) * out.st + r;
      int round = 0;
#pragma unroll 1
      for (int hf = 0; hf < n_halves && ok; ++hf) {
        // the same for all row warps; columns at and beyond head_dim lie outside the tensor map and are not written
        const bool full = J * kBM + hf * kBN + kBN <= c.len;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t va[16];
          tmem_ld16(tmem + 256 + hf * 128 + w * 64 + ch * 16 + lane_off, va);
          tmem_wait_ld();
          if (full) {
            // element (key, r) of a [64 keys x 128] tile: two 64-column blocks, 128-byte swizzle
            const uint32_t col_off = (r >> 6) * (kBN * 128) + (r & 7) * 2;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const int key = ch * 16 + k;
              const uint32_t off = col_off + (key >> 3) * 1024 + (key & 7) * 128 + ((((r & 63) >> 3) ^ (key & 7)) << 4);
              *reinterpret_cast<T *>(stage + off) = from_f32<T>(__uint_as_float(va[k]) * mul);
            }
          } else if (r < p.head_dim) {
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const int key = J * kBM + hf * kBN + ch * 16 + k;
              if (key < c.len) obase[(long long)(hf * kBN + ch * 16 + k) * out.st] = from_f32<T>(__uint_as_float(va[k]) * mul);
            }
          }
        }
        if (full) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(bStaged + w));
          if (r == 0 && (ok = wait_or_abort(bar(bStaged + w), round & 1, abort_flag, p, 633))) {
            const int krow = (int)c.tok0 + J * kBM + hf * kBN;
            tma_store_4d(omap, stage_addr, 0, krow, h, (int)c.boff);
            if (p.head_dim > 64) tma_store_4d(omap, stage_addr + kBN * 128, 64, krow, h, (int)c.boff);
            tma_store_commit();
            tma_store_wait_read();
            mbar_arrive(bar(bDrained + w));
          }
          // the buffer is rewritten for the next strip
          if (ok && hf + 1 < n_halves) ok = wait_or_abort(bar(bDrained + w), round & 1, abort_flag, p, 634);
          ++round;
        }
      }
      if (r == 0) tma_store_wait_all();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace_block(p, 2);
  if (warp == 9) tmem_dealloc(tmem, kTmemCols);
}

// =======================================================================================================
// dK/dV from stored tiles (head sizes 72..128): two GEMMs per 128-key tile, no row passes
// =======================================================================================================
// In stored-tiles mode the dq kernel leaves the 16-bit A and dz tiles of every (query tile, key tile) pair in the
// workspace.  This kernel owns one 128-key tile and walks its query tiles diagonal -> end, 32 query rows per stage:
//   dK[keys x d] += dz^T Q,   dV[keys x d] += A^T dO      (M = 128 keys, N = 128 columns, K = 32 query rows)
// with all four operands read row-major as "MN-major" tiles (rows = query rows = the contraction).  Accumulators sit
// in TMEM with lanes = keys, so the epilogue writes plain rows.  Fixed summation order, no atomics.
//   warp 4    TMA producer: per stage A, dz (from the workspace), Q, dO -- 32 KiB, three stages
//   warp 5    MMA issuer
//   warps 0-3 epilogue: dK, dV rows -> shared memory -> TMA stores
// The kernel is bound by reading the stored tiles (64 KiB per 128x128 pair) from HBM.  A block has a fixed cost of
// several microseconds (first loads, and at the end accumulators -> shared memory -> TMA stores) next to ~17 stages
// on average, so the stages are kept small enough for TWO blocks per SM (100 KB of shared memory, 256 TMEM columns
// each): one block's prologue and epilogue run under the other's stages.
namespace dkv5 {
constexpr int kThreads = 192;
constexpr int kStages = 3;
constexpr int kRows = 32;                    // query rows per stage
constexpr int kSub = kBM / kRows;            // stages per query tile
constexpr int kBox = kRows * 64 * 2;         // kRows rows x 64 columns, 16-bit
constexpr int kStageBytes = 8 * kBox;        // A, dz, Q, dO: two 64-column blocks each; also one 128 x 128 output tile
constexpr int kSmem = 1024 + kStages * kStageBytes + 512;
constexpr uint32_t kCols = 256;              // dK 0..127, dV 128..255
enum { bFull = 0, bEmpty = 3, bOut = 6, bClean = 7, bLanded = 8, bNum = 9 };
}  // namespace dkv5

template <bool kFp16>
__global__ void __launch_bounds__(dkv5::kThreads, 2)
tc_bwd_dkv5_kernel(const __grid_constant__ CUtensorMap tm_az, const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_dk,
                   const __grid_constant__ CUtensorMap tm_dv, const KParams p) {
  using namespace dkv5;
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  if (p.hdr[0]) return;
  TileCoord c;
  int hh;
  if (!decode_block(p, 1, false, c, hh)) return;
  const int h = p.head0 + hh;
  const int J = c.idx;                        // the 128-key tile
  const int n_stages = kSub * (c.n_tiles - J);   // stage t: query tile J + t / kSub, rows (t % kSub) * kRows .. + kRows
  // The sequence may end inside the last query tile.  The A and dz rows behind the end are zeros in the workspace; the
  // Q and dO rows there are not this sequence's (see zero_tile_rows).  Stages from t_clean on hold such rows: the
  // issuer tells the epilogue warps, idle until the end, that such a stage has landed (bLanded; a barrier of its own,
  // because a parity wait on bFull only works for a waiter that follows every phase), they clear the rows and hand
  // the stage back through bClean.
  const int last_rows = c.len - (c.n_tiles - 1) * kBM;          // 1 .. 128 rows of the last query tile exist
  const int t_clean = last_rows >= kBM ? n_stages : n_stages - (kSub - last_rows / kRows);

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  const uint32_t sBar = base + kStages * kStageBytes;
  Ctl *ctl = reinterpret_cast<Ctl *>(gbase + (sBar - base) + bNum * 8);
  volatile int *abort_flag = &ctl->abort;
  auto bar = [&](int i) { return sBar + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(bar(bFull + s), 1); mbar_init(bar(bEmpty + s), 1); }
    mbar_init(bar(bOut), 1);
    mbar_init(bar(bClean), 4);
    mbar_init(bar(bLanded), 1);
    ctl->abort = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tensormap(&tm_az); prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_g);
      for (int t = 0; t < n_stages; ++t) {
        const int st = t % kStages;
        if (t >= kStages && !wait_or_abort(bar(bEmpty + st), ((t / kStages) - 1) & 1, abort_flag, p, 640)) break;
        if (*abort_flag) break;
        const int I = J + t / kSub, hq = t % kSub;
        const long long pair = c.pair0 + (long long)I * (I + 1) / 2 + J;
        const int az_row = (int)(pair * kBM) + hq * kRows;
        const int qrow = (int)c.tok0 + I * kBM + hq * kRows;
        const uint32_t dst = base + st * kStageBytes;
        mbar_arrive_expect_tx(bar(bFull + st), kStageBytes);
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_4d(dst + (0 + kb) * kBox, &tm_az, bar(bFull + st), kb * 64, az_row, 0, hh);   // A
          tma_load_4d(dst + (2 + kb) * kBox, &tm_az, bar(bFull + st), kb * 64, az_row, 1, hh);   // dz
          tma_load_4d(dst + (4 + kb) * kBox, &tm_q, bar(bFull + st), kb * 64, qrow, h, (int)c.boff);
          tma_load_4d(dst + (6 + kb) * kBox, &tm_g, bar(bFull + st), kb * 64, qrow, h, (int)c.boff);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // all operands MN-major: rows = query rows (the contraction), two 64-column blocks kBox apart
      constexpr uint32_t idesc = idesc_f16(kBM, D, kFp16, true, true);
      bool ok = true;
      for (int t = 0; ok && t < n_stages; ++t) {
        const int st = t % kStages;
        ok = wait_or_abort(bar(bFull + st), (t / kStages) & 1, abort_flag, p, 641);
        if (ok && t >= t_clean) {
          mbar_arrive(bar(bLanded));
          ok = wait_or_abort(bar(bClean), (t - t_clean) & 1, abort_flag, p, 643);
        }
        if (!ok) break;
        tc_fence_after();
        const uint32_t a = base + st * kStageBytes;
        const uint64_t dA = smem_desc_sw128(a, kBox, 1024), dZ = smem_desc_sw128(a + 2 * kBox, kBox, 1024);
        const uint64_t dQ = smem_desc_sw128(a + 4 * kBox, kBox, 1024), dG = smem_desc_sw128(a + 6 * kBox, kBox, 1024);
#pragma unroll
        for (int ks = 0; ks < kRows / 16; ++ks)   // 16 query rows = 2048 bytes per step
          mma_f16_ss(tmem, dZ + (uint64_t)(ks * 128), dQ + (uint64_t)(ks * 128), idesc, t > 0 || ks > 0);
#pragma unroll
        for (int ks = 0; ks < kRows / 16; ++ks)
          mma_f16_ss(tmem + 128, dA + (uint64_t)(ks * 128), dG + (uint64_t)(ks * 128), idesc, t > 0 || ks > 0);
        mma_commit(bar(bEmpty + st));
      }
      if (ok) mma_commit(bar(bOut));
    }
  } else {
    // ------------------------------------------------ epilogue: one thread per key row
    using T = typename std::conditional<kFp16, __half, __nv_bfloat16>::type;
    const int r = threadIdx.x;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int t = t_clean; ok && t < n_stages; ++t) {
      const int st = t % kStages;
      ok = wait_or_abort(bar(bLanded), (t - t_clean) & 1, abort_flag, p, 644);
      if (!ok) break;
      int keep = last_rows - (t % kSub) * kRows;   // rows of this stage that belong to the sequence
      keep = keep < 0 ? 0 : keep;
      zero_tile_rows(gbase + st * kStageBytes + 4 * kBox, keep, kRows, 4, kBox, r, kBM);   // Q and dO: boxes 4..7 of the stage
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(bClean));
    }
    if (ok && wait_or_abort(bar(bOut), 0, abort_flag, p, 642)) {
      tc_fence_after();
      const int key = J * kBM + r;
      const bool valid = key < c.len;
      // out = o + rem * v was requested: dV gains rem * d_out on its own row (rem = 2^log_rem)
      const T *grow = nullptr;
      float rem_f = 0.f;
      if (p.fuse_rem_v && valid) {
        grow = reinterpret_cast<const T *>(p.d_o.ptr) + c.boff * p.d_o.sb + (long long)h * p.d_o.sh + (c.tok0 + key) * p.d_o.st;
        rem_f = exp2f((float)p.log_rem[(c.boff * p.heads + h) * p.tokens + c.tok0 + key]);
      }
      if (J * kBM + kBM <= c.len) {
        // full tile: through the first two stages' memory (all MMAs are done), one TMA store per warp and half
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          uint8_t *stage = gbase + which * kStageBytes;                // [128 x 128] as two blocks of 128-byte rows
          stage_acc_rows<D, kFp16>(tmem + which * 128 + lane_off, stage, r, which == 0 ? p.scale : 1.f,
                                   which == 1 ? grow : nullptr, rem_f, p.head_dim);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const uint32_t src = base + which * kStageBytes + warp * 32 * 128;
            const int trow = (int)c.tok0 + J * kBM + warp * 32;
            const CUtensorMap *omap = which == 0 ? &tm_dk : &tm_dv;
            tma_store_4d(omap, src, 0, trow, h, (int)c.boff);
            if (p.head_dim > 64) tma_store_4d(omap, src + kBoxBytes, 64, trow, h, (int)c.boff);
            tma_store_commit();
          }
        }
        if (lane == 0) tma_store_wait_all();
      } else {
        // the sequence ends inside the tile: row by row, rows past the end are left alone
        T *krow = reinterpret_cast<T *>(p.dk.ptr) + c.boff * p.dk.sb + (long long)h * p.dk.sh + (c.tok0 + key) * p.dk.st;
        T *vrow = reinterpret_cast<T *>(p.dv.ptr) + c.boff * p.dv.sb + (long long)h * p.dv.sh + (c.tok0 + key) * p.dv.st;
        store_acc_rows<D, kFp16, T>(tmem + lane_off, krow, valid, p.head_dim, p.scale);
        store_acc_rows<D, kFp16, T>(tmem + 128 + lane_off, vrow, valid, p.head_dim, 1.f, grow, rem_f);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, kCols);
}

// -------------------------------------------------------------------------------------------------------
template <bool kFp16>
static cudaError_t launch_bwd_t(const KParams &p, int dtype, cudaStream_t s) {
  CUtensorMap mq, mk, mv, mg;
  cudaError_t e;
  if ((e = make_tile_map(&mq, p.q, p, dtype)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mk, p.k, p, dtype)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mv, p.v, p, dtype)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mg, p.d_o, p, dtype)) != cudaSuccess) return e;
  const dim3 grid((unsigned)item_blocks(p, 1)), grid_pairs((unsigned)item_blocks(p, 2));
  if (!p.skip_dq) {
    auto kernel = tc_bwd_dq2_kernel<kFp16>;
    e = allow_dynamic_smem(reinterpret_cast<const void *>(kernel), dq2::kSmem);
    if (e != cudaSuccess) return e;
    CUtensorMap mk64, mv64;   // 64-row boxes: the kernel streams 64-key sub-tiles
    if ((e = make_tile_map(&mk64, p.k, p, dtype, 64)) != cudaSuccess) return e;
    if ((e = make_tile_map(&mv64, p.v, p, dtype, 64)) != cudaSuccess) return e;
    CUtensorMap mdq, maz32;   // stores: 32 rows per warp
    if ((e = make_tile_map(&mdq, p.dq, p, dtype, 32)) != cudaSuccess) return e;
    if (p.az != nullptr) { if ((e = make_az_map(&maz32, p, dtype, 32)) != cudaSuccess) return e; }
    else maz32 = mdq;         // not used
    kernel<<<grid_pairs, dq2::kThreads, dq2::kSmem, s>>>(mq, mk64, mv64, mg, mdq, maz32, p);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  if (!p.skip_dkv && p.az != nullptr) {
    auto kernel = tc_bwd_dkv5_kernel<kFp16>;
    e = allow_dynamic_smem(reinterpret_cast<const void *>(kernel), dkv5::kSmem);
    if (e != cudaSuccess) return e;
    CUtensorMap maz, mq64, mg64, mdk, mdv;
    if ((e = make_az_map(&maz, p, dtype, dkv5::kRows)) != cudaSuccess) return e;
    if ((e = make_tile_map(&mq64, p.q, p, dtype, dkv5::kRows)) != cudaSuccess) return e;
    if ((e = make_tile_map(&mg64, p.d_o, p, dtype, dkv5::kRows)) != cudaSuccess) return e;
    if ((e = make_tile_map(&mdk, p.dk, p, dtype, 32)) != cudaSuccess) return e;   // stores: 32 rows per warp
    if ((e = make_tile_map(&mdv, p.dv, p, dtype, 32)) != cudaSuccess) return e;
    kernel<<<grid, dkv5::kThreads, dkv5::kSmem, s>>>(maz, mq64, mg64, mdk, mdv, p);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  } else if (!p.skip_dkv) {
    auto kernel = tc_bwd_dkv4_kernel<kFp16>;
    e = allow_dynamic_smem(reinterpret_cast<const void *>(kernel), dkv4::kSmem);
    if (e != cudaSuccess) return e;
    CUtensorMap mdk, mdv;   // stores: one 64-key strip at a time
    if ((e = make_tile_map(&mdk, p.dk, p, dtype, 64)) != cudaSuccess) return e;
    if ((e = make_tile_map(&mdv, p.dv, p, dtype, 64)) != cudaSuccess) return e;
    kernel<<<grid, dkv4::kThreads, dkv4::kSmem, s>>>(mq, mk, mv, mg, mdk, mdv, p);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// Every head size up to 128 runs the same 128-column kernels: TMA fills the columns past head_dim with zeros, and the
// row passes, which bound these kernels, do not depend on the head size.
cudaError_t launch_tc_bwd(const KParams &p, int dtype, cudaStream_t s, int *launches) {
  *launches += (p.skip_dq ? 0 : 1) + (p.skip_dkv ? 0 : 1);
  return dtype == SB_DTYPE_F16 ? launch_bwd_t<true>(p, dtype, s) : launch_bwd_t<false>(p, dtype, s);
}

}  // namespace sb
