// Pieces shared by the tensor-core forward and backward kernels.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "sb_common.cuh"
#include "sb_ptx.cuh"

namespace sb {

using namespace ptx;

constexpr int kBM = kTcTile;  // 128 query rows per CTA, 128 keys per tile
constexpr int kTcThreads = 192;  // warps 0-3: one thread per tile row; warp 4: TMA; warp 5: MMA issue
constexpr uint32_t kTmemCols = 512;
constexpr int kBoxBytes = kBM * 64 * 2;  // one TMA box: 128 rows x 64 16-bit elements, 128-byte swizzled

struct Ctl {  // lives behind the barriers in shared memory
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag, const KParams &p,
                                              int which) {
  if (mbar_wait(bar, parity)) return true;
  *abort_flag = 1;
  if (p.status != nullptr) { p.status[0] = SB_DEV_WAIT_TIMEOUT; p.status[1] = which; }
  return false;
}

// Zero-fills rows [row0, box_rows) of `boxes` consecutive [box_rows x 64] 16-bit boxes in shared memory (128-byte
// rows; the 128-byte swizzle only permutes the 16-byte chunks inside a row, so whole rows are plain byte ranges).
// The tensor maps cover the whole tokens axis, so a box that reaches past the end of its sequence holds the next
// sequence's rows or whatever lies behind the last one.  Wherever such rows are an MMA operand whose partner is an
// exact zero (V under P = 0, K under dz = 0, Q and dO under zero rows of dz and A) they are cleared first: 0 x NaN and
// 0 x Inf are NaN.  Called by `nthreads` threads with indices `tid`; the caller fences (generic -> async proxy)
// before it signals the MMA issuer.
// (Not inlined: it runs once per sequence end, and the row loops it is called from are register-bound.)
static __device__ __noinline__ void zero_tile_rows(uint8_t *tile, int row0, int box_rows, int boxes, int box_bytes, int tid,
                                            int nthreads) {
  const int chunks = (box_rows - row0) * 8;   // 16-byte chunks per box
  for (int i = tid; i < chunks * boxes; i += nthreads) {
    const int b = i / chunks, c = i - b * chunks;
    *reinterpret_cast<uint4 *>(tile + b * box_bytes + row0 * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <bool kFp16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kFp16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
}

// Byte offset of the 16-byte chunk holding columns [c0, c0+8) of row r in a [128 x 128] 16-bit tile stored as
// two [128 x 64] blocks of 128-byte rows with the 128-byte swizzle (chunk index XOR row mod 8).  Read by the
// MMA either as a K-major operand (rows = M, columns = K) or as an MN-major one (rows = K, columns = M).
__device__ __forceinline__ uint32_t sw128_chunk_offset(int r, int c0) {
  const int kb = c0 >> 6, chunk = (c0 & 63) >> 3;
  return kb * kBoxBytes + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4);
}

// Stores 32 consecutive columns (first column c0, a multiple of 32) of row r of such a tile.
template <bool kFp16>
__device__ __forceinline__ void store_row_chunk(uint8_t *tile, int r, int c0, const float (&x)[32]) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 w;
    w.x = pack2<kFp16>(x[g * 8 + 0], x[g * 8 + 1]);
    w.y = pack2<kFp16>(x[g * 8 + 2], x[g * 8 + 3]);
    w.z = pack2<kFp16>(x[g * 8 + 4], x[g * 8 + 5]);
    w.w = pack2<kFp16>(x[g * 8 + 6], x[g * 8 + 7]);
    *reinterpret_cast<uint4 *>(tile + sw128_chunk_offset(r, c0 + g * 8)) = w;
  }
}

// Stores 16 consecutive columns (first column c0, a multiple of 16) of row r of such a tile.
template <bool kFp16>
__device__ __forceinline__ void store_row_chunk16(uint8_t *tile, int r, int c0, const float (&x)[16]) {
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    uint4 w;
    w.x = pack2<kFp16>(x[g * 8 + 0], x[g * 8 + 1]);
    w.y = pack2<kFp16>(x[g * 8 + 2], x[g * 8 + 3]);
    w.z = pack2<kFp16>(x[g * 8 + 4], x[g * 8 + 5]);
    w.w = pack2<kFp16>(x[g * 8 + 6], x[g * 8 + 7]);
    *reinterpret_cast<uint4 *>(tile + sw128_chunk_offset(r, c0 + g * 8)) = w;
  }
}

// The same in two steps: 16 values packed into eight 32-bit registers, which can go to several places.
template <bool kFp16>
__device__ __forceinline__ void pack_row_chunk16(const float (&x)[16], uint32_t (&w)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = pack2<kFp16>(x[2 * i], x[2 * i + 1]);
}
__device__ __forceinline__ void store_packed_chunk16(uint8_t *tile, int r, int c0, const uint32_t (&w)[8]) {
  *reinterpret_cast<uint4 *>(tile + sw128_chunk_offset(r, c0)) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4 *>(tile + sw128_chunk_offset(r, c0 + 8)) = make_uint4(w[4], w[5], w[6], w[7]);
}
// 16 consecutive 16-bit values of a plain row-major global row (32 bytes, 32-byte aligned)
__device__ __forceinline__ void store_packed_global16(unsigned short *dst, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]),
               "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");   // one full 32-byte sector per thread
}

// Eight consecutive 16-bit values of a global row (16 bytes, aligned) as floats.
template <bool kFp16>
__device__ __forceinline__ void load_row8(const void *src, float (&x)[8]) {
  const uint4 w = *reinterpret_cast<const uint4 *>(src);
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kFp16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
      x[2 * i] = f.x; x[2 * i + 1] = f.y;
    } else {
      x[2 * i] = __uint_as_float(u[i] << 16); x[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
}

// TMEM accumulator rows (one per thread) -> 16-bit global rows, `mul` applied, columns >= head_dim dropped.
// With `add_row` (a 16-bit global row of head_dim values) the stored value is acc * mul + add_mul * add_row.
template <int D, bool kFp16, typename T>
__device__ __forceinline__ void store_acc_rows(uint32_t tmem_addr, T *grow, bool valid, int head_dim, float mul,
                                               const T *add_row = nullptr, float add_mul = 0.f) {
#pragma unroll 1
  for (int ch = 0; ch < D / 32; ++ch) {
    uint32_t v[32];
    tmem_ld32(tmem_addr + ch * 32, v);
    tmem_wait_ld();
    if (valid) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const int x0 = ch * 32 + g * 8;
        if (x0 < head_dim) {
          float x[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = __uint_as_float(v[g * 8 + i]) * mul;
          if (add_row != nullptr) {
            float a[8];
            load_row8<kFp16>(add_row + x0, a);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = fmaf(add_mul, a[i], x[i]);
          }
          uint4 w;
          w.x = pack2<kFp16>(x[0], x[1]);
          w.y = pack2<kFp16>(x[2], x[3]);
          w.z = pack2<kFp16>(x[4], x[5]);
          w.w = pack2<kFp16>(x[6], x[7]);
          *reinterpret_cast<uint4 *>(grow + x0) = w;
        }
      }
    }
  }
}

// TMEM accumulator rows (one per thread) -> a 16-bit [128 x D] tile in shared memory (D / 64 blocks of 128-byte
// rows, 128-byte swizzle), from where TMA stores it with full lines instead of 16 bytes per thread and row.
// `add_row` / `add_mul` as above (the row must exist: callers use this for full tiles only).
template <int D, bool kFp16>
__device__ __forceinline__ void stage_acc_rows(uint32_t tmem_addr, uint8_t *tile, int r, float mul,
                                               const void *add_row = nullptr, float add_mul = 0.f, int head_dim = D) {
#pragma unroll 1
  for (int ch = 0; ch < D / 32; ++ch) {
    uint32_t v[32];
    tmem_ld32(tmem_addr + ch * 32, v);
    tmem_wait_ld();
    float x[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(v[i]) * mul;
    if (add_row != nullptr) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (ch * 32 + g * 8 < head_dim) {
          float a[8];
          load_row8<kFp16>(reinterpret_cast<const uint16_t *>(add_row) + ch * 32 + g * 8, a);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[g * 8 + i] = fmaf(add_mul, a[i], x[g * 8 + i]);
        }
      }
    }
    store_row_chunk<kFp16>(tile, r, ch * 32, x);
  }
}

// MMA issue helpers (called by one thread).  The issuing thread is a scalar instruction stream, so descriptors are
// built once per tile and only their 14-bit start-address field (bytes >> 4) is advanced per instruction:
// a K-major operand moves 32 bytes per 16-element K step inside a 64-element block and one box per block; an
// MN-major one moves 16 rows (2048 bytes) per K step.
__device__ __forceinline__ constexpr uint64_t kstep_kmajor(int k, int box_bytes) {
  return (uint64_t)(((k >> 2) * box_bytes + (k & 3) * 32) >> 4);
}
template <int KDIM, int A_BOX = kBoxBytes, int B_BOX = kBoxBytes>
__device__ __forceinline__ void mma_kmajor_kmajor(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc,
                                                  bool accumulate) {
  const uint64_t a0 = smem_desc_sw128(a_addr, 16, 1024), b0 = smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
  for (int k = 0; k < KDIM / 16; ++k)
    mma_f16_ss(d_tmem, a0 + kstep_kmajor(k, A_BOX), b0 + kstep_kmajor(k, B_BOX), idesc, accumulate || k > 0);
}
// A: K-major [128 x KDIM];  B: rows = K (KDIM), columns = N in blocks of 64 that are B_BOX bytes apart, MN-major.
template <int KDIM = kBM, int B_BOX = kBoxBytes>
__device__ __forceinline__ void mma_kmajor_mnmajor(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc,
                                                   bool accumulate) {
  const uint64_t a0 = smem_desc_sw128(a_addr, 16, 1024), b0 = smem_desc_sw128(b_addr, B_BOX, 1024);
#pragma unroll
  for (int ks = 0; ks < KDIM / 16; ++ks)
    mma_f16_ss(d_tmem, a0 + kstep_kmajor(ks, kBoxBytes), b0 + (uint64_t)(ks * 128), idesc, accumulate || ks > 0);
}
// A: [128 x KDIM] 16-bit rows in tensor memory (KDIM / 2 columns starting at a_tmem, two K elements per column);
// B as in mma_kmajor_mnmajor.
template <int KDIM, int B_BOX = kBoxBytes>
__device__ __forceinline__ void mma_tmem_mnmajor(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, uint32_t idesc,
                                                 bool accumulate) {
  const uint64_t b0 = smem_desc_sw128(b_addr, B_BOX, 1024);
#pragma unroll
  for (int ks = 0; ks < KDIM / 16; ++ks)
    mma_f16_ts(d_tmem, a_tmem + ks * 8, b0 + (uint64_t)(ks * 128), idesc, accumulate || ks > 0);
}
// A and B both stored with rows = K (128): A^T B.
__device__ __forceinline__ void mma_mnmajor_mnmajor(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc,
                                                    bool accumulate) {
  const uint64_t a0 = smem_desc_sw128(a_addr, kBoxBytes, 1024), b0 = smem_desc_sw128(b_addr, kBoxBytes, 1024);
#pragma unroll
  for (int ks = 0; ks < kBM / 16; ++ks)
    mma_f16_ss(d_tmem, a0 + (uint64_t)(ks * 128), b0 + (uint64_t)(ks * 128), idesc, accumulate || ks > 0);
}

// host: 4-D TMA map (head_dim, tokens, heads, batch), [64 x 128 x 1 x 1] box, 128-byte swizzle, zero fill
cudaError_t make_tile_map(CUtensorMap *map, const TensorRef &t, const KParams &p, int dtype, int box_rows = kBM);
// host: cudaFuncSetAttribute(MaxDynamicSharedMemorySize), issued once per kernel and device
cudaError_t allow_dynamic_smem(const void *kernel, int bytes);
// host: 4-D TMA map of the stored A / dz tiles, (keys 128, pairs * 128 query rows, {A, dz}, heads), [64 x 64 x 1 x 1] box
cudaError_t make_az_map(CUtensorMap *map, const KParams &p, int dtype, int box_rows = 64);

}  // namespace sb
