// Tensor-core forward kernel for bf16 / fp16 tensors: 256 query rows per work item, persistent blocks.
//
// Reference counterpart: _forward_one_row, sb_varlen_fwd.py:81-215.  A CTA owns two adjacent 128-row query tiles
// (a: rows 0..127, b: rows 128..255 of its 256-row block) of one (sequence, head) and streams 64-key K/V
// sub-tiles from its last needed key back to the sequence start.  Both tiles consume the same K/V stage, so K/V
// is read once per 256 rows, and the two row-owning warpgroups (warps 0-3: tile a, warps 4-7: tile b) keep two
// warps resident per scheduler so that one hides the other's dependent-issue and TMEM latency.
//   warp 8    TMA producer: Q_a, Q_b once, then K/V sub-tiles into a 3-stage ring
//   warps 9,10 MMA issuers, one per tile: S_x = Q_x K^T (128x64) into a double-buffered TMEM slot, O_x += P_x V
//   warps 0-7 one thread per query row: p = beta * R with the running product R of (1 - beta) over later keys,
//             P written as a 16-bit [128 x 64] swizzled tile (double-buffered) for the second MMA
// TMEM columns: S_a[2] 0..127, S_b[2] 128..255, O_a 256..383, O_b 384..511.  All waits are bounded.
#include "sb_tc_fwd_rows.cuh"

namespace sb {

namespace fwd256 {
constexpr int kThreads = 352;
constexpr int kMaxStages = 6;
constexpr int kKvBoxBytes = kBN * 64 * 2;     // one 64-row x 64-column box
constexpr int kBarBytes = 512;
template <int D>                              // D: head size rounded up to 64 or 128
struct Cfg {
  static constexpr int kBoxes = D / 64;                        // 64-column blocks per row
  static constexpr int kQBytes = kBM * D * 2;                  // one 128-row Q tile
  static constexpr int kKvTileBytes = kBoxes * kKvBoxBytes;    // K or V sub-tile: 64 keys x D columns
  static constexpr int kStageBytes = 2 * kKvTileBytes;         // K and V
  // K/V ring: three stages at 128 columns fill the shared memory; at 64 columns six fit, and short sequences need
  // them: a stage is reloaded only after both tiles' P V MMAs of its step, so with three stages the load for step
  // s + 3 starts one row pass before its scores are wanted, which the ~2000 clk load latency does not always meet
  static constexpr int kStages = D == 64 ? 6 : 3;
  // Q tiles of two items at 64 columns (there is room): the next item's Q is loaded while the current item still
  // reads its own, so a short item does not wait a load latency for its first scores
  static constexpr int kQBufs = D == 64 ? 2 : 1;
  static constexpr int kSmem = 1024 + kQBufs * 2 * kQBytes + kStages * kStageBytes + 4 * kPBytes + kBarBytes;
};
enum { bQ = 0, bKvFull = 1, bKvEmpty = 7, bSFull = 13, bQFree = 17, bOFree = 18, bPFull = 20, bPEmpty = 24, bOFull = 28, bQ2 = 30,
       bQFree2 = 31, bNum = 32 };   // bQ2 / bQFree2: the second Q buffer
static_assert(bKvEmpty - bKvFull == kMaxStages && bSFull - bKvEmpty == kMaxStages, "barrier slots per stage");
// per-warpgroup barrier index: base + wg * 2 + buf
}  // namespace fwd256

// What one work item (a 256-row block of one sequence and head) looks like to every role.
struct Fwd256Item {
  TileCoord c;
  int h;          // head
  int blk_row0;   // first row of the block inside the sequence
  bool b_active;  // the block has a second tile
  int s_top;      // sub-tile of step 0; step t handles sub-tile s_top - t
  int n_steps;
  int t0_a;       // first step in which tile a takes part
};

// Item number `it` of this block: the launch holds one block per SM; blocks walk the weight-ordered item list in a
// boustrophedon (even rounds left to right, odd rounds right to left), which evens out the sums of the weights.
__device__ __forceinline__ bool fwd256_item(const KParams &p, int it, Fwd256Item &w) {
  const long long G = gridDim.x;
  const long long lin = (long long)it * G + ((it & 1) ? G - 1 - blockIdx.x : blockIdx.x);
  const long long item = lin / p.head_cnt;
  if (item > 0x7fffffffLL || !decode_item(p, (int)item, 1, true, w.c)) return false;
  w.h = p.head0 + (int)(lin - item * p.head_cnt);
  const int m = w.c.idx;
  const int n_sub = (w.c.len + fwd256::kBN - 1) / fwd256::kBN;   // 64-key sub-tiles of the sequence
  w.blk_row0 = m * 256;
  w.b_active = w.blk_row0 + kBM < w.c.len;
  const int s_hi_a = min(4 * m + 1, n_sub - 1);                 // last sub-tile tile a needs
  const int s_hi_b = min(4 * m + 3, n_sub - 1);
  w.s_top = w.b_active ? s_hi_b : s_hi_a;
  w.n_steps = w.s_top + 1;
  w.t0_a = w.s_top - s_hi_a;
  return true;
}

// Persistent: every block works through several items; all barrier phases run on across items (the counters T, U
// below), so the loads and first MMAs of the next item overlap the last row pass and the epilogue of the current one.
// Per item and role the barriers advance by fixed amounts whether or not tile b exists: an idle issuer still commits
// and releases the K/V stages (after they were filled, so that it cannot run ahead of a phase).
template <int D, bool kFp16>
__global__ void __launch_bounds__(fwd256::kThreads, 1)
tc_fwd256_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, const KParams p) {
  using namespace fwd256;
  using C = Cfg<D>;
  constexpr int kQBytes = C::kQBytes, kKvTileBytes = C::kKvTileBytes, kStageBytes = C::kStageBytes, kBoxes = C::kBoxes;
  constexpr int kStages = C::kStages, kQBufs = C::kQBufs;
  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0) trace_block(p, 0);
  if (p.hdr[0]) return;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  const uint32_t sQ = base;                             // per buffer: Q_a, Q_b
  const uint32_t sKV = sQ + kQBufs * 2 * kQBytes;       // stages: K sub-tile then V sub-tile
  const uint32_t sP = sKV + kStages * kStageBytes;      // P[wg][buf]
  const uint32_t sBar = sP + 4 * kPBytes;
  uint8_t *gP = gbase + (sP - base);
  Ctl *ctl = reinterpret_cast<Ctl *>(gbase + (sBar - base) + bNum * 8);
  volatile int *abort_flag = &ctl->abort;
  auto bar = [&](int i) { return sBar + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int tr_cur = 0;   // cursor of this thread's event-log lane (experiments only)

  if (threadIdx.x == 0) {
    mbar_init(bar(bQ), 1);
    mbar_init(bar(bQFree), 2);
    mbar_init(bar(bQ2), 1);
    mbar_init(bar(bQFree2), 2);
    for (int s = 0; s < kStages; ++s) { mbar_init(bar(bKvFull + s), 1); mbar_init(bar(bKvEmpty + s), 2); }
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar(bSFull + s), 1);
      mbar_init(bar(bPFull + s), 4);
      mbar_init(bar(bPEmpty + s), 1);
    }
    mbar_init(bar(bOFull), 1);
    mbar_init(bar(bOFull + 1), 1);
    mbar_init(bar(bOFree), 4);
    mbar_init(bar(bOFree + 1), 4);
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

  Fwd256Item w;
  if (warp == 8) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
      int T = 0;   // K/V stages filled so far
      for (int it = 0; fwd256_item(p, it, w); ++it) {
        // the Q buffer's previous item (kQBufs items back) is no longer read once both issuers have finished its last S MMAs
        const int qb = it % kQBufs, qn = it / kQBufs;     // buffer and how many items it has held before
        const uint32_t bar_q = bar(qb ? bQ2 : bQ), bar_qfree = bar(qb ? bQFree2 : bQFree);
        if (qn >= 1 && !wait_or_abort(bar_qfree, (qn - 1) & 1, abort_flag, p, 311)) break;
        const int qrow = (int)w.c.tok0 + w.blk_row0;
        mbar_arrive_expect_tx(bar_q, 2 * kQBytes);
        for (int t = 0; t < 2; ++t)
          for (int kb = 0; kb < kBoxes; ++kb)
            tma_load_4d(sQ + (qb * 2 + t) * kQBytes + kb * kBoxBytes, &tm_q, bar_q, kb * 64, qrow + t * kBM, w.h, (int)w.c.boff);
        bool ok = true;
        for (int t = 0; t < w.n_steps; ++t) {
          const int g = T + t, st = g % kStages;
          if (g >= kStages && !wait_or_abort(bar(bKvEmpty + st), ((g / kStages) - 1) & 1, abort_flag, p, 310)) { ok = false; break; }
          if (*abort_flag) { ok = false; break; }
          const int krow = (int)w.c.tok0 + (w.s_top - t) * kBN;
          const uint32_t dst = sKV + st * kStageBytes;
          trace_event(p, 0, tr_cur, 1, t);
          mbar_arrive_expect_tx(bar(bKvFull + st), kStageBytes);
          for (int kb = 0; kb < kBoxes; ++kb) {
            tma_load_4d(dst + kb * kKvBoxBytes, &tm_k, bar(bKvFull + st), kb * 64, krow, w.h, (int)w.c.boff);
            tma_load_4d(dst + kKvTileBytes + kb * kKvBoxBytes, &tm_v, bar(bKvFull + st), kb * 64, krow, w.h, (int)w.c.boff);
          }
        }
        if (!ok) break;
        T += w.n_steps;
      }
    }
  } else if (warp >= 9) {
    // ------------------------------------------------ MMA issuers: warp 9 for tile a, warp 10 for tile b
    const int wg = warp - 9;
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_f16(kBM, kBN, kFp16, false, false);
      constexpr uint32_t idesc_pv = idesc_f16(kBM, D, kFp16, false, true);
      int T = 0, U = 0;   // K/V stages and this tile's steps of the earlier items
      bool ok = true;
      for (int it = 0; ok && fwd256_item(p, it, w); ++it) {
        const bool active = wg == 0 || w.b_active;
        const int t0 = active ? (wg == 0 ? w.t0_a : 0) : w.n_steps;   // stages this tile does not read
        const int my_steps = w.n_steps - t0;
        // release the unread stages on this tile's behalf, each once it has been filled
        for (int t = 0; ok && t < t0; ++t) {
          const int g = T + t;
          ok = wait_or_abort(bar(bKvFull + g % kStages), (g / kStages) & 1, abort_flag, p, 324);
          if (ok) mbar_arrive(bar(bKvEmpty + g % kStages));
        }
        const int qb = it % kQBufs, qn = it / kQBufs;
        const uint32_t qaddr = sQ + (qb * 2 + wg) * kQBytes, bar_qfree = bar(qb ? bQFree2 : bQFree);
        // (an idle issuer waits too: a parity wait is only meaningful for a waiter that follows every phase)
        if (ok) ok = wait_or_abort(bar(qb ? bQ2 : bQ), qn & 1, abort_flag, p, 320);
        // Iteration u issues S(u) and then P V of step u-1, so that the next scores are being computed while the
        // rows of the current step are processed.  S(u) reuses the TMEM slot of step u-2, whose rows were finished
        // before p_full(u-2) was signalled, and that was waited for in iteration u-1.
        for (int u = 0; ok && active && u <= my_steps; ++u) {
          if (u < my_steps) {
            const int g = T + t0 + u, st = g % kStages, gu = U + u;
            ok = wait_or_abort(bar(bKvFull + st), (g / kStages) & 1, abort_flag, p, 321);
            if (!ok) break;
            trace_event(p, 1 + 3 * wg, tr_cur, 2 + 16 * wg, t0 + u);
            tc_fence_after();
            mma_kmajor_kmajor<D, kBoxBytes, kKvBoxBytes>(tmem + wg * 128 + (gu & 1) * 64, qaddr, sKV + st * kStageBytes, idesc_s,
                                                         false);
            mma_commit(bar(bSFull + wg * 2 + (gu & 1)));
            if (u == my_steps - 1) mma_commit(bar_qfree);   // the item's last read of Q
            trace_event(p, 1 + 3 * wg, tr_cur, 3 + 16 * wg, t0 + u);
          }
          if (u >= 1) {
            const int up = u - 1, g = T + t0 + up, st = g % kStages, gu = U + up;
            ok = wait_or_abort(bar(bPFull + wg * 2 + (gu & 1)), (gu >> 1) & 1, abort_flag, p, 323);
            // the accumulator still holds the previous item's O until its rows have read it
            if (ok && up == 0 && it >= 1) ok = wait_or_abort(bar(bOFree + wg), (it - 1) & 1, abort_flag, p, 325);
            if (!ok) break;
            trace_event(p, 1 + 3 * wg, tr_cur, 6 + 16 * wg, t0 + up);
            tc_fence_after();
            // 16 keys per MMA; V: 64 rows x (2 x 64) columns, MN-major
            if constexpr (kPTmem) {
              mma_tmem_mnmajor<kBN, kKvBoxBytes>(tmem + 256 + wg * 128, tmem + wg * 128 + (gu & 1) * 64 + kPCol,
                                                 sKV + st * kStageBytes + kKvTileBytes, idesc_pv, up > 0);
            } else {
              mma_kmajor_mnmajor<kBN, kKvBoxBytes>(tmem + 256 + wg * 128, sP + (wg * 2 + (gu & 1)) * kPBytes,
                                                   sKV + st * kStageBytes + kKvTileBytes, idesc_pv, up > 0);
              mma_commit(bar(bPEmpty + wg * 2 + (gu & 1)));
            }
            mma_commit(bar(bKvEmpty + st));
            trace_event(p, 1 + 3 * wg, tr_cur, 7 + 16 * wg, t0 + up);
          }
        }
        if (!ok) break;
        if (!active) mma_commit(bar_qfree);   // after this thread's earlier MMAs, like every arrival on these two
        mma_commit(bar(bOFull + wg));   // this tile's O is complete (an idle tile: behind its earlier MMAs)
        T += w.n_steps;
        U += my_steps;
      }
    }
  } else {
    // ------------------------------------------------ one thread per query row, one warpgroup per 128-row tile
    using T = typename std::conditional<kFp16, __half, __nv_bfloat16>::type;
    const int wg = warp >> 2;
    const int r = threadIdx.x & 127;                 // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float scale2 = p.scale * kLog2e;
    const int ac = p.attend_current;
    int U = 0, S = 0;   // this tile's steps and the K/V stages of the earlier items
    bool ok = true;
    Fwd256Item w_next;
    bool have = fwd256_item(p, 0, w);
    for (int it = 0; ok && have; ++it) {
      const bool active = wg == 0 || w.b_active;
      const int t0 = wg == 0 ? w.t0_a : 0;
      const int my_steps = active ? w.n_steps - t0 : 0;
      const int row = w.blk_row0 + wg * kBM + r;       // row index inside the sequence
      const int s_diag0 = 4 * w.c.idx + 2 * wg;        // first sub-tile that reaches this tile's diagonal band
      const bool warp_live = (row & ~31) < w.c.len;    // a warp whose 32 rows all lie past the sequence end computes nothing
      double run = 0.0;
      if (lane == 0) tma_store_wait_read();   // the previous item's O has left the P buffers
      __syncwarp();
      if ((threadIdx.x & 127) == 0) trace_event(p, 2 + wg, tr_cur, 40 + wg, it);
      for (int u = 0; u < my_steps && ok; ++u) {
        const int s = w.s_top - (t0 + u);
        const int gu = U + u, buf = gu & 1;
        ok = wait_or_abort(bar(bSFull + wg * 2 + buf), (gu >> 1) & 1, abort_flag, p, 330);
        // a shared-memory P buffer is free once the P V MMA of two steps ago has read it; P in tensor memory needs no
        // such wait: it overwrites scores of this very step, which the same thread has already loaded
        if (!kPTmem && ok && gu >= 2) ok = wait_or_abort(bar(bPEmpty + wg * 2 + buf), ((gu >> 1) - 1) & 1, abort_flag, p, 331);
        if (!ok) break;
        if (threadIdx.x == 128 && u == 0 && it == 0) trace_block(p, 1);
        if ((threadIdx.x & 127) == 0) trace_event(p, 2 + wg, tr_cur, 4 + 16 * wg, t0 + u);
        tc_fence_after();
        const uint32_t ts = tmem + wg * 128 + buf * 64 + lane_off;
        uint8_t *tile_p = gP + (wg * 2 + buf) * kPBytes;
        // the sequence ends inside this sub-tile: the V rows behind its end are not this sequence's (see zero_tile_rows);
        // their P columns are exact zeros, so the rows are cleared before this step's P V MMA is released
        const int tail_rows = w.c.len - s * kBN;
        if (tail_rows < kBN) {
          uint8_t *v_tile = gbase + (sKV - base) + ((S + t0 + u) % kStages) * kStageBytes + kKvTileBytes;
          zero_tile_rows(v_tile, tail_rows, kBN, kBoxes, kKvBoxBytes, r, kBM);
          fence_proxy_async_smem();
        }
        float R = ex2(-(float)run);
        float logsum = 0.f;
        // 64 columns in chunks of 16, last chunk first; TMEM is read one chunk ahead of the arithmetic
        // (the P rows of such a warp keep whatever their buffer held: they only reach accumulator rows that are never stored)
        if (!warp_live) {
        } else if (s >= s_diag0) fwd256_row_pass<kFp16, true>(ts, s * kBN, row, ac, scale2, R, logsum, tile_p, r, ts + kPCol);
        else fwd256_row_pass<kFp16, false>(ts, 0, 0, ac, scale2, R, logsum, tile_p, r, ts + kPCol, !p.dense);
        run += (double)logsum;
        if constexpr (kPTmem) tmem_wait_st();
        tc_fence_before();          // this step's TMEM reads (and writes of P) are done before the slot is handed back
        if constexpr (!kPTmem) fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(bPFull + wg * 2 + buf));
        if ((threadIdx.x & 127) == 0) trace_event(p, 2 + wg, tr_cur, 5 + 16 * wg, t0 + u);
      }
      // ---- epilogue: O (TMEM) -> global, rem, log_rem
      if ((threadIdx.x & 127) == 0) trace_event(p, 2 + wg, tr_cur, 42 + wg, it);
      // While the last P V MMA finishes: rem and log_rem leave, and the next item's table entries are fetched.
      const bool valid = row < w.c.len;
      const float rem_f = ex2(-(float)run);
      if (ok && my_steps > 0 && valid) {
        const long long idx = (w.c.boff * p.heads + w.h) * p.tokens + w.c.tok0 + row;
        reinterpret_cast<T *>(p.rem)[idx] = from_f32<T>(rem_f);
        p.log_rem[idx] = -run;
      }
      const bool have_next = fwd256_item(p, it + 1, w_next);
      if (ok) ok = wait_or_abort(bar(bOFull + wg), it & 1, abort_flag, p, 332);
      if ((threadIdx.x & 127) == 0) trace_event(p, 2 + wg, tr_cur, 44 + wg, it);
      if (ok && my_steps > 0) {
        tc_fence_after();
        const int tile_row0 = w.blk_row0 + wg * kBM;
        // out = o + rem * v on request: this row of V comes straight from global memory
        const T *vrow = (p.fuse_rem_v && valid) ? reinterpret_cast<const T *>(p.v.ptr) + w.c.boff * p.v.sb +
                                                      (long long)w.h * p.v.sh + (w.c.tok0 + row) * p.v.st
                                                : nullptr;
        if (tile_row0 + kBM <= w.c.len) {
          // full tile: through this tile's two P buffers (all P V MMAs are done), one TMA store per warp and half
          uint8_t *stage = gP + wg * 2 * kPBytes;
          stage_acc_rows<D, kFp16>(tmem + 256 + wg * 128 + lane_off, stage, r, 1.f, vrow, rem_f, p.head_dim);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const uint32_t src = sP + wg * 2 * kPBytes + (warp & 3) * 32 * 128;
            const int trow = (int)w.c.tok0 + tile_row0 + (warp & 3) * 32;
            for (int kb = 0; kb < kBoxes; ++kb) tma_store_4d(&tm_o, src + kb * kPBytes, kb * 64, trow, w.h, (int)w.c.boff);
            tma_store_commit();
          }
        } else {
          // the sequence ends inside the tile: row by row, rows past the end are left alone
          T *orow = reinterpret_cast<T *>(p.o.ptr) + w.c.boff * p.o.sb + (long long)w.h * p.o.sh + (w.c.tok0 + row) * p.o.st;
          store_acc_rows<D, kFp16, T>(tmem + 256 + wg * 128 + lane_off, orow, valid, p.head_dim, 1.f, vrow, rem_f);
        }
      }
      tc_fence_before();            // the accumulator has been read: the next item may overwrite it
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(bOFree + wg));
      if ((threadIdx.x & 127) == 0) trace_event(p, 2 + wg, tr_cur, 46 + wg, it);
      U += my_steps;
      S += w.n_steps;
      w = w_next;
      have = have_next;
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace_block(p, 2);
  if (warp == 9) tmem_dealloc(tmem, kTmemCols);
}

template <int D, bool kFp16>
static cudaError_t launch_t(const KParams &p, int dtype, cudaStream_t s) {
  CUtensorMap mq, mk, mv, mo;
  cudaError_t e;
  if ((e = make_tile_map(&mq, p.q, p, dtype, kBM)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mo, p.o, p, dtype, 32)) != cudaSuccess) return e;   // stores: 32 rows per warp
  if ((e = make_tile_map(&mk, p.k, p, dtype, fwd256::kBN)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mv, p.v, p, dtype, fwd256::kBN)) != cudaSuccess) return e;
  int sms = 0;
  if ((e = sm_count(&sms)) != cudaSuccess) return e;
  const long long blocks = item_blocks(p, 1);
  const dim3 grid((unsigned)(blocks < sms ? blocks : sms));   // one resident block per SM
  auto kernel = tc_fwd256_kernel<D, kFp16>;
  constexpr int smem = fwd256::Cfg<D>::kSmem;
  if ((e = allow_dynamic_smem(reinterpret_cast<const void *>(kernel), smem)) != cudaSuccess) return e;
  kernel<<<grid, fwd256::kThreads, smem, s>>>(mq, mk, mv, mo, p);
  return cudaGetLastError();
}

cudaError_t launch_tc_fwd256(const KParams &p, int dtype, cudaStream_t s) {
  const bool f16 = dtype == SB_DTYPE_F16;
  if (p.head_dim <= 64) return f16 ? launch_t<64, true>(p, dtype, s) : launch_t<64, false>(p, dtype, s);
  return f16 ? launch_t<128, true>(p, dtype, s) : launch_t<128, false>(p, dtype, s);
}

}  // namespace sb
