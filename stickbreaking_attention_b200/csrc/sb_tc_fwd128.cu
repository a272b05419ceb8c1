// Tensor-core forward kernel for head sizes up to 64 and short sequences: two independent 128-row tiles per block.
//
// Reference counterpart: _forward_one_row, sb_varlen_fwd.py:81-215.  The 256-row kernel (sb_tc_fwd256.cu) lets two
// adjacent tiles share one stream of K/V sub-tiles; with sequences of a few hundred tokens that coupling costs more
// than it saves: the earlier tile of a pair has no work in the first two steps of every item (half of a four-step
// item), a sequence's last item often has no second tile at all, and both tiles stand still together at every item
// boundary.  Here a block holds two WORKERS that share nothing but the SM: each has its own list of 128-row tiles
// (weight-ordered, boustrophedon over all workers of the grid), its own TMA producer and MMA issuer, its own
// three-stage K/V ring, two Q buffers, S slots and O accumulator.  At 64 columns all of that fits twice.
//   warps 0-3 / 4-7   rows of worker 0 / 1: one thread per query row (the row arithmetic of sb_tc_fwd_rows.cuh)
//   warps 8 / 11      TMA producers of worker 0 / 1
//   warps 9 / 10      MMA issuers of worker 0 / 1: S = Q K^T (128x64x64) into a double-buffered TMEM slot,
//                     O += P V (128x64x64) with P read from tensor memory
// TMEM columns of worker w: S[2] at 192 w + {0, 64}, O at 192 w + 128.  All waits are bounded.
//
// Row warp j of either worker runs on scheduler j of the SM, and the later rows of a tile have more allowed keys in the
// diagonal band (and are the ones missing when the sequence ends inside the tile).  Worker 1 therefore holds its tile
// with the four 32-row blocks in reverse order (Q is loaded as four 32-row boxes, tensor-memory lanes 0..31 are query
// rows 96..127 of the tile): every scheduler then serves one warp with much and one with little work.
#include "sb_tc_fwd_rows.cuh"

namespace sb {

namespace fwd128 {
constexpr int kThreads = 384;
constexpr int D = 64;                         // columns (head sizes below 64: TMA fills the rest with zeros)
constexpr int kBN = 64;                       // keys per sub-tile
constexpr int kQBytes = kBM * D * 2;          // one 128-row Q tile = one 128 x 64 box
constexpr int kKvTileBytes = kBN * D * 2;     // K or V sub-tile: one 64 x 64 box
constexpr int kStageBytes = 2 * kKvTileBytes;
constexpr int kStages = 3;                    // (a fourth stage fits and was measured: no gain)
constexpr int kQBufs = 2;
constexpr int kOBytes = kBM * D * 2;          // staging tile of the O epilogue
constexpr int kWorkerBytes = kQBufs * kQBytes + kStages * kStageBytes + kOBytes;
constexpr int kBarBytes = 512;
constexpr int kSmem = 1024 + 2 * kWorkerBytes + kBarBytes;
constexpr uint32_t kWorkerCols = 192;
// barriers of one worker
enum { bQ = 0, bQFree = 2, bKvFull = 4, bKvEmpty = 4 + kStages, bSFull = 4 + 2 * kStages, bPFull = bSFull + 2, bOFull = bSFull + 4,
       bOFree = bSFull + 5, bPerWorker = bSFull + 6 };
}  // namespace fwd128

struct Fwd128Item {
  TileCoord c;
  int h;          // head
  int row0;       // first row of the tile inside the sequence
  int s_top;      // sub-tile of step 0; step t handles sub-tile s_top - t
  int n_steps;
};

// Item number `it` of worker v out of V: the workers walk the weight-ordered tile list in a boustrophedon.
__device__ __forceinline__ long long fwd128_lin(int it, int v, int V) {
  return (long long)it * V + ((it & 1) ? V - 1 - v : v);
}
__device__ __forceinline__ void fwd128_finish(const KParams &p, long long lin, long long item, Fwd128Item &w) {
  w.h = p.head0 + (int)(lin - item * p.head_cnt);
  const int n_sub = (w.c.len + fwd128::kBN - 1) / fwd128::kBN;
  w.row0 = w.c.idx * kBM;
  w.s_top = min(2 * w.c.idx + 1, n_sub - 1);
  w.n_steps = w.s_top + 1;
}
__device__ __forceinline__ bool fwd128_item(const KParams &p, int it, int v, int V, Fwd128Item &w) {
  const long long lin = fwd128_lin(it, v, V);
  const long long item = lin / p.head_cnt;
  if (item > 0x7fffffffLL || !decode_item(p, (int)item, 1, true, w.c)) return false;
  fwd128_finish(p, lin, item, w);
  return true;
}

template <bool kFp16>
__global__ void __launch_bounds__(fwd128::kThreads, 1)
tc_fwd128x2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const KParams p) {
  using namespace fwd128;
  extern __shared__ uint8_t smem_raw[];
  if (p.hdr[0]) return;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  const uint32_t sBar = base + 2 * kWorkerBytes;
  Ctl *ctl = reinterpret_cast<Ctl *>(gbase + (sBar - base) + 2 * bPerWorker * 8);
  volatile int *abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // which worker this warp serves
  const int wk = warp < 8 ? warp >> 2 : (warp == 8 || warp == 9 ? 0 : 1);
  const int v = 2 * blockIdx.x + wk, V = 2 * gridDim.x;
  auto bar = [&](int i) { return sBar + 8u * (wk * bPerWorker + i); };
  const uint32_t sQ = base + wk * kWorkerBytes;            // two Q buffers
  const uint32_t sKV = sQ + kQBufs * kQBytes;              // stages: K sub-tile then V sub-tile
  const uint32_t sO = sKV + kStages * kStageBytes;         // staging tile of the epilogue

  if (threadIdx.x == 0) {
    for (int w = 0; w < 2; ++w) {
      auto b = [&](int i) { return sBar + 8u * (w * bPerWorker + i); };
      for (int i = 0; i < kQBufs; ++i) { mbar_init(b(bQ + i), 1); mbar_init(b(bQFree + i), 1); }
      for (int s = 0; s < kStages; ++s) { mbar_init(b(bKvFull + s), 1); mbar_init(b(bKvEmpty + s), 1); }
      for (int s = 0; s < 2; ++s) { mbar_init(b(bSFull + s), 1); mbar_init(b(bPFull + s), 4); }
      mbar_init(b(bOFull), 1);
      mbar_init(b(bOFree), 4);
    }
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
  const uint32_t tmem = ctl->tmem_base + wk * kWorkerCols;

  Fwd128Item w;
  if (warp == 8 || warp == 11) {
    // ------------------------------------------------ TMA producer of this worker
    if (lane == 0) {
      prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
      int T = 0;   // K/V stages filled so far
      for (int it = 0; fwd128_item(p, it, v, V, w); ++it) {
        const int qb = it % kQBufs, qn = it / kQBufs;
        // the buffer's previous tile is no longer read once its last S MMA has finished
        if (qn >= 1 && !wait_or_abort(bar(bQFree + qb), (qn - 1) & 1, abort_flag, p, 711)) break;
        mbar_arrive_expect_tx(bar(bQ + qb), kQBytes);
        for (int b = 0; b < 4; ++b)   // block b of the shared-memory tile (= TMEM lanes 32 b ..) holds row block wk ? 3 - b : b
          tma_load_4d(sQ + qb * kQBytes + b * (kQBytes / 4), &tm_q, bar(bQ + qb), 0,
                      (int)w.c.tok0 + w.row0 + (wk ? 3 - b : b) * 32, w.h, (int)w.c.boff);
        bool ok = true;
        for (int t = 0; t < w.n_steps; ++t) {
          const int g = T + t, st = g % kStages;
          if (g >= kStages && !wait_or_abort(bar(bKvEmpty + st), ((g / kStages) - 1) & 1, abort_flag, p, 710)) { ok = false; break; }
          if (*abort_flag) { ok = false; break; }
          const int krow = (int)w.c.tok0 + (w.s_top - t) * kBN;
          const uint32_t dst = sKV + st * kStageBytes;
          mbar_arrive_expect_tx(bar(bKvFull + st), kStageBytes);
          tma_load_4d(dst, &tm_k, bar(bKvFull + st), 0, krow, w.h, (int)w.c.boff);
          tma_load_4d(dst + kKvTileBytes, &tm_v, bar(bKvFull + st), 0, krow, w.h, (int)w.c.boff);
        }
        if (!ok) break;
        T += w.n_steps;
      }
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------------------------ MMA issuer of this worker
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_f16(kBM, kBN, kFp16, false, false);
      constexpr uint32_t idesc_pv = idesc_f16(kBM, D, kFp16, false, true);
      int T = 0, U = 0;   // K/V stages and steps of the earlier tiles
      bool ok = true;
      for (int it = 0; ok && fwd128_item(p, it, v, V, w); ++it) {
        const int qb = it % kQBufs, qn = it / kQBufs;
        ok = wait_or_abort(bar(bQ + qb), qn & 1, abort_flag, p, 720);
        const uint32_t qaddr = sQ + qb * kQBytes;
        // Iteration u issues S(u) and then P V of step u-1, so that the next scores are being computed while the
        // rows of the current step are processed.  S(u) reuses the TMEM slot of step u-2, whose P the P V MMA of
        // that step (issued earlier by this thread) has read.
        for (int u = 0; ok && u <= w.n_steps; ++u) {
          if (u < w.n_steps) {
            const int g = T + u, st = g % kStages, gu = U + u;
            ok = wait_or_abort(bar(bKvFull + st), (g / kStages) & 1, abort_flag, p, 721);
            if (!ok) break;
            tc_fence_after();
            mma_kmajor_kmajor<D, kQBytes, kKvTileBytes>(tmem + (gu & 1) * 64, qaddr, sKV + st * kStageBytes, idesc_s, false);
            mma_commit(bar(bSFull + (gu & 1)));
            if (u == w.n_steps - 1) mma_commit(bar(bQFree + qb));   // the tile's last read of Q
          }
          if (u >= 1) {
            const int up = u - 1, g = T + up, st = g % kStages, gu = U + up;
            ok = wait_or_abort(bar(bPFull + (gu & 1)), (gu >> 1) & 1, abort_flag, p, 723);
            // the accumulator still holds the previous tile's O until its rows have read it
            if (ok && up == 0 && it >= 1) ok = wait_or_abort(bar(bOFree), (it - 1) & 1, abort_flag, p, 725);
            if (!ok) break;
            tc_fence_after();
            mma_tmem_mnmajor<kBN, kKvTileBytes>(tmem + 128, tmem + (gu & 1) * 64 + kPCol,
                                                sKV + st * kStageBytes + kKvTileBytes, idesc_pv, up > 0);
            mma_commit(bar(bKvEmpty + st));
          }
        }
        if (!ok) break;
        mma_commit(bar(bOFull));   // this tile's O is complete
        T += w.n_steps;
        U += w.n_steps;
      }
    }
  } else {
    // ------------------------------------------------ one thread per query row
    using T = typename std::conditional<kFp16, __half, __nv_bfloat16>::type;
    const int r = threadIdx.x & 127;                 // TMEM lane == row of the shared-memory tiles
    const int blk = wk ? 3 - (warp & 3) : (warp & 3); // which 32-row block of the query tile this warp's lanes hold
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float scale2 = p.scale * kLog2e;
    const int ac = p.attend_current;
    int U = 0, S = 0;   // steps and K/V stages of the earlier tiles
    bool ok = true;
    Fwd128Item w_next;
    bool have = fwd128_item(p, 0, v, V, w);
    uint8_t *stage = gbase + (sO - base);
    for (int it = 0; ok && have; ++it) {
      const int row = w.row0 + blk * 32 + lane;      // row index inside the sequence
      const int s_diag0 = 2 * w.c.idx;               // first sub-tile that reaches this tile's diagonal band
      const bool warp_live = (row & ~31) < w.c.len;  // a warp whose 32 rows all lie past the sequence end computes nothing
      double run = 0.0;
      if (lane == 0) tma_store_wait_read();          // the previous tile's O has left the staging tile
      __syncwarp();
      for (int u = 0; u < w.n_steps && ok; ++u) {
        const int s = w.s_top - u;
        const int gu = U + u, buf = gu & 1;
        ok = wait_or_abort(bar(bSFull + buf), (gu >> 1) & 1, abort_flag, p, 730);
        if (!ok) break;
        tc_fence_after();
        const uint32_t ts = tmem + buf * 64 + lane_off;
        // the sequence ends inside this sub-tile: the V rows behind its end are not this sequence's (see
        // zero_tile_rows); their P columns are exact zeros, so the rows are cleared before this step's P V MMA
        const int tail_rows = w.c.len - s * kBN;
        if (tail_rows < kBN) {
          zero_tile_rows(gbase + (sKV - base) + ((S + u) % kStages) * kStageBytes + kKvTileBytes, tail_rows, kBN, 1, kKvTileBytes, r, kBM);
          fence_proxy_async_smem();
        }
        float R = ex2(-(float)run);
        float logsum = 0.f;
        // (the P rows of such a warp keep whatever the slot held: they only reach accumulator rows that are never stored)
        if (!warp_live) {
        } else if (s >= s_diag0) fwd256_row_pass<kFp16, true>(ts, s * kBN, row, ac, scale2, R, logsum, nullptr, r, ts + kPCol);
        else fwd256_row_pass<kFp16, false>(ts, 0, 0, ac, scale2, R, logsum, nullptr, r, ts + kPCol, !p.dense);
        run += (double)logsum;
        tmem_wait_st();
        tc_fence_before();          // this step's TMEM reads and its writes of P are done before the slot is handed back
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(bPFull + buf));
      }
      // ---- epilogue: O (TMEM) -> global, rem, log_rem
      // While the last P V MMA finishes: rem and log_rem leave, and the next tile's table entries are fetched.
      const bool valid = row < w.c.len;
      const float rem_f = ex2(-(float)run);
      if (ok && valid) {
        const long long idx = (w.c.boff * p.heads + w.h) * p.tokens + w.c.tok0 + row;
        reinterpret_cast<T *>(p.rem)[idx] = from_f32<T>(rem_f);
        p.log_rem[idx] = -run;
      }
      const bool have_next = fwd128_item(p, it + 1, v, V, w_next);
      if (ok) ok = wait_or_abort(bar(bOFull), it & 1, abort_flag, p, 732);
      if (ok) {
        tc_fence_after();
        // out = o + rem * v on request: this row of V comes straight from global memory
        const T *vrow = (p.fuse_rem_v && valid) ? reinterpret_cast<const T *>(p.v.ptr) + w.c.boff * p.v.sb +
                                                      (long long)w.h * p.v.sh + (w.c.tok0 + row) * p.v.st
                                                : nullptr;
        if (w.row0 + kBM <= w.c.len) {
          // full tile: through the staging tile, one TMA store per warp (full 128-byte lines)
          stage_acc_rows<D, kFp16>(tmem + 128 + lane_off, stage, r, 1.f, vrow, rem_f, p.head_dim);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&tm_o, sO + (warp & 3) * 32 * 128, 0, (int)w.c.tok0 + w.row0 + blk * 32, w.h, (int)w.c.boff);
            tma_store_commit();
          }
        } else {
          // the sequence ends inside the tile: row by row, rows past the end are left alone
          T *orow = reinterpret_cast<T *>(p.o.ptr) + w.c.boff * p.o.sb + (long long)w.h * p.o.sh + (w.c.tok0 + row) * p.o.st;
          store_acc_rows<D, kFp16, T>(tmem + 128 + lane_off, orow, valid, p.head_dim, 1.f, vrow, rem_f);
        }
      }
      tc_fence_before();            // the accumulator has been read: the next tile may overwrite it
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(bOFree));
      U += w.n_steps;
      S += w.n_steps;
      w = w_next;
      have = have_next;
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(ctl->tmem_base, kTmemCols);
}

template <bool kFp16>
static cudaError_t launch128_t(const KParams &p, int dtype, cudaStream_t s) {
  CUtensorMap mq, mk, mv, mo;
  cudaError_t e;
  if ((e = make_tile_map(&mq, p.q, p, dtype, 32)) != cudaSuccess) return e;   // loads and stores: 32-row blocks
  if ((e = make_tile_map(&mo, p.o, p, dtype, 32)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mk, p.k, p, dtype, fwd128::kBN)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mv, p.v, p, dtype, fwd128::kBN)) != cudaSuccess) return e;
  int sms = 0;
  if ((e = sm_count(&sms)) != cudaSuccess) return e;
  const long long blocks = (item_blocks(p, 1) + 1) / 2;       // two workers per block
  const dim3 grid((unsigned)(blocks < sms ? blocks : sms));   // one resident block per SM
  auto kernel = tc_fwd128x2_kernel<kFp16>;
  if ((e = allow_dynamic_smem(reinterpret_cast<const void *>(kernel), fwd128::kSmem)) != cudaSuccess) return e;
  kernel<<<grid, fwd128::kThreads, fwd128::kSmem, s>>>(mq, mk, mv, mo, p);
  return cudaGetLastError();
}

cudaError_t launch_tc_fwd128(const KParams &p, int dtype, cudaStream_t s) {
  return dtype == SB_DTYPE_F16 ? launch128_t<true>(p, dtype, s) : launch128_t<false>(p, dtype, s);
}

}  // namespace sb
