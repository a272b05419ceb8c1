// The forward's row arithmetic, shared by the forward kernels: one query row per thread, scores read from tensor
// memory in chunks of 16 columns, P written back to tensor memory as the A operand of O += P V.
#pragma once

#include "sb_tc_common.cuh"

namespace sb {

namespace fwd256 {
constexpr int kBN = 64;                       // keys per sub-tile
constexpr int kPBytes = kBM * kBN * 2;        // a 128 x 64 16-bit tile (the staging unit of the O epilogue)
// P, the 16-bit A operand of O += P V, goes to the second MMA through tensor memory: the row threads write their
// packed row into columns 32..63 of the very S slot they have just read (key k of the step in column 32 + k / 2;
// the chunks are read last column first, so every column written has been read before), and the MMA takes its A
// operand from there.  The next S MMA into that slot is issued by the same thread after this P V MMA, and MMAs of
// one thread execute in order.  With SB_FWD_P_SMEM the earlier hand-over through a swizzled shared-memory tile is built.
#ifdef SB_FWD_P_SMEM
constexpr bool kPTmem = false;
#else
constexpr bool kPTmem = true;
#endif
constexpr uint32_t kPCol = 32;
}  // namespace fwd256

using fwd256::kPCol;
using fwd256::kPTmem;

// One row, 16 consecutive key columns of a 64-key sub-tile, last column first.  key0: index inside the sequence of
// the chunk's first column; row: index of this query row.
//   x = z log2(e), clamped at 30;  e = 2^x;  t = 1 + e;  1 - beta = 1 / t;  beta = e / t
//   p_j = beta_j * (product of (1 - beta) over the allowed keys after j) = e_j * (product of 1 / t over j and after)
// R carries that product over everything after the current column.  Four columns share one reciprocal and one
// logarithm of t0 t1 t2 t3; the four inclusive products follow from R, that reciprocal and partial products with
// five multiplications, and beta itself is never formed.
template <bool kFp16, bool kMasked>
__device__ __forceinline__ void fwd256_row_chunk(const uint32_t (&v)[16], int c0, int key0, int row, int ac,
                                                 float scale2, float &R, float &logsum, uint8_t *tile_p, int r,
                                                 uint32_t tmem_p) {
  float pr[16];
  const float2 sc = make_float2(scale2, scale2), one = make_float2(1.f, 1.f);
#pragma unroll
  for (int g = 3; g >= 0; --g) {   // four columns at a time, last group first; independent work in packed pairs
    const float2 x01 = mul2(make_float2(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1])), sc);
    const float2 x23 = mul2(make_float2(__uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3])), sc);
    float2 e01 = make_float2(ex2(fminf(x01.x, 30.f)), ex2(fminf(x01.y, 30.f)));
    float2 e23 = make_float2(ex2(fminf(x23.x, 30.f)), ex2(fminf(x23.y, 30.f)));
    float2 t01 = add2(e01, one), t23 = add2(e23, one);
    if (kMasked) {
      const int key = key0 + 4 * g, lim = row + ac;
      if (!(key < lim)) { e01.x = 0.f; t01.x = 1.f; }
      if (!(key + 1 < lim)) { e01.y = 0.f; t01.y = 1.f; }
      if (!(key + 2 < lim)) { e23.x = 0.f; t23.x = 1.f; }
      if (!(key + 3 < lim)) { e23.y = 0.f; t23.y = 1.f; }
    }
    const float p01 = t01.x * t01.y, p23 = t23.x * t23.y;
    const float prod = p01 * p23;
    const float rp = rcp(prod);
    logsum += lg2(prod);
    const float rb = R * (rp * p01);          // R / (t2 t3): inclusive product at column 2
    const float r3 = rb * t23.x;              // R / t3
    R *= rp;                                  // R / (t0 t1 t2 t3): at column 0, and the carry into the next group
    const float r1 = R * t01.x;               // R / (t1 t2 t3)
    const float2 q01 = mul2(e01, make_float2(R, r1));
    const float2 q23 = mul2(e23, make_float2(rb, r3));
    pr[4 * g] = q01.x;
    pr[4 * g + 1] = q01.y;
    pr[4 * g + 2] = q23.x;
    pr[4 * g + 3] = q23.y;
  }
  if constexpr (kPTmem) {   // 16 keys = 8 packed columns of this row's lane
    uint32_t w[8];
    pack_row_chunk16<kFp16>(pr, w);
    tmem_st8(tmem_p + (c0 >> 1), w);
  } else {
    store_row_chunk16<kFp16>(tile_p, r, c0, pr);
  }
}

// P of 32 key columns (from column c0 of the sub-tile on) set to zero without looking at the scores.
template <bool kFp16>
__device__ __forceinline__ void fwd256_zero_pair(int c0, uint8_t *tile_p, int r, uint32_t tmem_p) {
  if constexpr (kPTmem) {
    const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    tmem_st8(tmem_p + (c0 >> 1), z);
    tmem_st8(tmem_p + (c0 >> 1) + 8, z);
  } else {
    const float z[16] = {};
    store_row_chunk16<kFp16>(tile_p, r, c0, z);
    store_row_chunk16<kFp16>(tile_p, r, c0 + 16, z);
  }
}

// One row of a 64-key sub-tile whose P is known to be exactly zero: only the log-space sum is formed, with the same
// operations in the same order as fwd256_row_chunk, so that it is the same number bit for bit.
__device__ __forceinline__ void fwd256_logsum_chunk(const uint32_t (&v)[16], float scale2, float &logsum) {
  const float2 sc = make_float2(scale2, scale2), one = make_float2(1.f, 1.f);
#pragma unroll
  for (int g = 3; g >= 0; --g) {
    const float2 x01 = mul2(make_float2(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1])), sc);
    const float2 x23 = mul2(make_float2(__uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3])), sc);
    const float2 e01 = make_float2(ex2(fminf(x01.x, 30.f)), ex2(fminf(x01.y, 30.f)));
    const float2 e23 = make_float2(ex2(fminf(x23.x, 30.f)), ex2(fminf(x23.y, 30.f)));
    const float2 t01 = add2(e01, one), t23 = add2(e23, one);
    const float p01 = t01.x * t01.y, p23 = t23.x * t23.y;
    logsum += lg2(p01 * p23);
  }
}
template <bool kFp16>
__device__ __forceinline__ void fwd256_logsum_pass(uint32_t ts, float scale2, float &logsum, uint8_t *tile_p, int r,
                                                   uint32_t tmem_p) {
  uint32_t va[16], vb[16];
  tmem_ld16(ts + 48, va);
#pragma unroll 1
  for (int pair = 1; pair >= 0; --pair) {
    tmem_wait_ld_regs(va);
    tmem_ld16(ts + pair * 32, vb);
    fwd256_logsum_chunk(va, scale2, logsum);
    tmem_wait_ld_regs(vb);
    if (pair == 1) tmem_ld16(ts + 16, va);
    fwd256_logsum_chunk(vb, scale2, logsum);
  }
  // P is written last: its columns alias scores that have all been read by now
  fwd256_zero_pair<kFp16>(32, tile_p, r, tmem_p);
  fwd256_zero_pair<kFp16>(0, tile_p, r, tmem_p);
}

// One row of a 64-key sub-tile.  In a masked sub-tile the columns from (last row of this warp) + ac on are masked for
// every row of the warp (its 32 rows are consecutive and 32-aligned): such 32-column halves are not computed at all,
// their P is zero and R and logsum stay as they are -- 6 of the 16 (warp, half) pairs of a diagonal 128 x 128 tile.
// skip_zero: an unmasked sub-tile whose P is exactly zero for the whole warp (R has underflowed) only sums its logs.
template <bool kFp16, bool kMasked>
__device__ __forceinline__ void fwd256_row_pass(uint32_t ts, int key0, int row, int ac, float scale2, float &R,
                                                float &logsum, uint8_t *tile_p, int r, uint32_t tmem_p,
                                                bool skip_zero = false) {
  if (!kMasked && skip_zero && __all_sync(0xffffffffu, R == 0.f)) {
    // The product over the keys after this sub-tile has underflowed to exactly 0 for all 32 rows of the warp: every
    // p of the sub-tile is e * 0 = 0 (e is finite: its exponent is clamped) and R stays 0.
    fwd256_logsum_pass<kFp16>(ts, scale2, logsum, tile_p, r, tmem_p);
    return;
  }
  int hi = 1;   // last 32-column half with an allowed key
  if (kMasked) {
    const int span = (row | 31) + ac - key0;   // the warp's rows may attend to columns [0, span) of this sub-tile
    hi = span > 32 ? 1 : (span > 0 ? 0 : -1);
    if (hi < 1) fwd256_zero_pair<kFp16>(32, tile_p, r, tmem_p);
    if (hi < 0) {
      fwd256_zero_pair<kFp16>(0, tile_p, r, tmem_p);
      return;
    }
  }
  uint32_t va[16], vb[16];
  tmem_ld16(ts + hi * 32 + 16, va);
#pragma unroll 1
  for (int pair = hi; pair >= 0; --pair) {
    tmem_wait_ld_regs(va);
    tmem_ld16(ts + pair * 32, vb);
    fwd256_row_chunk<kFp16, kMasked>(va, pair * 32 + 16, key0 + pair * 32 + 16, row, ac, scale2, R, logsum, tile_p, r, tmem_p);
    tmem_wait_ld_regs(vb);
    if (pair == 1) tmem_ld16(ts + 16, va);
    fwd256_row_chunk<kFp16, kMasked>(vb, pair * 32, key0 + pair * 32, row, ac, scale2, R, logsum, tile_p, r, tmem_p);
  }
}

}  // namespace sb
