// Tensor-core forward kernel for bf16 / fp16 tensors: tcgen05 MMAs with TMEM accumulators, K/V tiles staged by TMA.
//
// Reference counterpart: _forward_one_row, sb_varlen_fwd.py:81-215.  One CTA owns a 128-row query tile of one
// (sequence, head) and walks the key tiles from the diagonal back to the sequence start:
//   warp 4    TMA producer: Q once, then K and V tiles into a ring of shared-memory stages
//   warp 5    MMA issuer:   S = Q K^T into one of two TMEM buffers, O += P V into a third
//   warps 0-3 one thread per query row: reads its row of S from TMEM (32 columns at a time, last column
//             first), turns z into p = 2^(z + suffix sum of log2(1-beta)) with a running fp32 sum carried in
//             registers, writes P as bf16 into the swizzled shared-memory layout the MMA reads
// Every wait on an mbarrier is bounded; a wait that gives up records SB_DEV_WAIT_TIMEOUT and all roles
// leave through the common exit, which frees the tensor memory.
#include "sb_tc_common.cuh"

namespace sb {

template <int D>
struct FwdCfg {
  static constexpr int kStages = D == 128 ? 2 : 3;
  static constexpr int kTileBytes = kBM * D * 2;
  static constexpr int kPBytes = kBM * kBM * 2;
  static constexpr int kBarBytes = 256;
  static constexpr int kSmem = 1024 + kTileBytes * (1 + 2 * kStages) + 2 * kPBytes + kBarBytes;
};

// barrier slots (8 bytes each) inside the barrier block
enum { kBarQ = 0, kBarKvFull = 1, kBarKvEmpty = 5, kBarSFull = 9, kBarSEmpty = 11, kBarPFull = 13, kBarPEmpty = 15,
       kBarOFull = 17, kNumBars = 18 };

// One row, 32 consecutive key columns starting at c0, visited from the last column to the first.
//   x = z log2(e), clamped at 30 (sigmoid is 1 to 1e-9 there);  e = 2^x;  1 - beta = 1 / (1 + e)
//   p = beta * R with R the product of (1 - beta) over the later keys (kept in registers, may underflow to 0,
//   which is also what p rounds to then);  R *= (1 - beta)
// Four columns share one reciprocal and one logarithm (of the product of their (1 + e)): 1.5 transcendentals per
// score.  The logarithms give the tile's contribution to log2 of the product exactly enough for 131072-token rows.
template <bool kFp16, bool kDiag>
__device__ __forceinline__ void fwd_row_chunk(const uint32_t (&v)[32], int c0, int r, int ac, float scale2, float &R,
                                              float &logsum, uint8_t *tile_p) {
  float pr[32];
#pragma unroll
  for (int g = 7; g >= 0; --g) {   // four columns at a time, last group first
    float e[4], t[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      e[i] = ex2(fminf(__uint_as_float(v[4 * g + i]) * scale2, 30.f));
      t[i] = 1.f + e[i];
      if (kDiag) {
        const bool allowed = c0 + 4 * g + i < r + ac;
        e[i] = allowed ? e[i] : 0.f;
        t[i] = allowed ? t[i] : 1.f;
      }
    }
    // one reciprocal and one logarithm for the four factors (1 + e): 1/t_i = (1 / t0 t1 t2 t3) * (product of the others)
    const float p01 = t[0] * t[1], p23 = t[2] * t[3];
    const float prod = p01 * p23;
    const float rp = rcp(prod);
    logsum += lg2(prod);
    const float a = rp * p23, b = rp * p01;
    const float ri3 = b * t[2], ri2 = b * t[3], ri1 = a * t[0], ri0 = a * t[1];
    pr[4 * g + 3] = (e[3] * ri3) * R; R *= ri3;
    pr[4 * g + 2] = (e[2] * ri2) * R; R *= ri2;
    pr[4 * g + 1] = (e[1] * ri1) * R; R *= ri1;
    pr[4 * g + 0] = (e[0] * ri0) * R; R *= ri0;
  }
  store_row_chunk<kFp16>(tile_p, r, c0, pr);
}

template <int D, bool kFp16>
__global__ void __launch_bounds__(kTcThreads, 1)
tc_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const KParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int NS = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  if (p.hdr[0]) return;
  TileCoord c;
  int hh_blk;
  if (!decode_block(p, 1, true, c, hh_blk)) return;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gbase = smem_raw + (base - raw);
  const uint32_t sQ = base;
  const uint32_t sK = sQ + Cfg::kTileBytes;
  const uint32_t sV = sK + NS * Cfg::kTileBytes;
  const uint32_t sP = sV + NS * Cfg::kTileBytes;
  const uint32_t sBar = sP + 2 * Cfg::kPBytes;
  uint8_t *gP0 = gbase + (sP - base);
  Ctl *ctl = reinterpret_cast<Ctl *>(gbase + (sBar - base) + kNumBars * 8);
  volatile int *abort_flag = &ctl->abort;
  auto bar = [&](int i) { return sBar + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = p.head0 + hh_blk;
  const int I = c.idx;
  const int n_tiles = I + 1;
  const int row0 = (int)c.tok0 + I * kBM;

  if (threadIdx.x == 0) {
    mbar_init(bar(kBarQ), 1);
    for (int s = 0; s < NS; ++s) { mbar_init(bar(kBarKvFull + s), 1); mbar_init(bar(kBarKvEmpty + s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar(kBarSFull + s), 1); mbar_init(bar(kBarSEmpty + s), 4); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar(kBarPFull + s), 4); mbar_init(bar(kBarPEmpty + s), 1); }
    mbar_init(bar(kBarOFull), 1);
    ctl->abort = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tO = tmem + 256;

  if (warp == 4) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q); prefetch_tensormap(&tm_k); prefetch_tensormap(&tm_v);
      mbar_arrive_expect_tx(bar(kBarQ), Cfg::kTileBytes);
      for (int kb = 0; kb < D / 64; ++kb)
        tma_load_4d(sQ + kb * kBoxBytes, &tm_q, bar(kBarQ), kb * 64, row0, h, (int)c.boff);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % NS;
        if (j >= NS && !wait_or_abort(bar(kBarKvEmpty + st), ((j / NS) - 1) & 1, abort_flag, p, 10)) break;
        if (*abort_flag) break;
        const int krow = (int)c.tok0 + (I - j) * kBM;
        mbar_arrive_expect_tx(bar(kBarKvFull + st), 2 * Cfg::kTileBytes);
        for (int kb = 0; kb < D / 64; ++kb) {
          tma_load_4d(sK + st * Cfg::kTileBytes + kb * kBoxBytes, &tm_k, bar(kBarKvFull + st), kb * 64, krow, h, (int)c.boff);
          tma_load_4d(sV + st * Cfg::kTileBytes + kb * kBoxBytes, &tm_v, bar(kBarKvFull + st), kb * 64, krow, h, (int)c.boff);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_f16(kBM, kBM, kFp16, false, false);
      constexpr uint32_t idesc_pv = idesc_f16(kBM, D, kFp16, false, true);
      auto issue_s = [&](int j) {  // S[j & 1] = Q K_j^T
        mma_kmajor_kmajor<D>(tS[j & 1], sQ, sK + (j % NS) * Cfg::kTileBytes, idesc_s, false);
        mma_commit(bar(kBarSFull + (j & 1)));
      };
      bool ok = wait_or_abort(bar(kBarQ), 0, abort_flag, p, 20) && wait_or_abort(bar(kBarKvFull), 0, abort_flag, p, 21);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles) {
          const int jn = j + 1;
          ok = wait_or_abort(bar(kBarKvFull + jn % NS), (jn / NS) & 1, abort_flag, p, 22);
          if (ok && jn >= 2) ok = wait_or_abort(bar(kBarSEmpty + (jn & 1)), ((jn >> 1) - 1) & 1, abort_flag, p, 23);
          if (!ok) break;
          tc_fence_after();
          issue_s(jn);
        }
        ok = wait_or_abort(bar(kBarPFull + (j & 1)), (j >> 1) & 1, abort_flag, p, 24);
        if (!ok) break;
        tc_fence_after();
        mma_kmajor_mnmajor(tO, sP + (j & 1) * Cfg::kPBytes, sV + (j % NS) * Cfg::kTileBytes, idesc_pv, j > 0);   // O += P V_j
        mma_commit(bar(kBarKvEmpty + j % NS));
        mma_commit(bar(kBarPEmpty + (j & 1)));
      }
      if (ok) mma_commit(bar(kBarOFull));
    }
  } else {
    // ------------------------------------------------ one thread per query row
    const int r = threadIdx.x;                       // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const float scale2 = p.scale * kLog2e;
    const int ac = p.attend_current;
    double run = 0.0;                                // sum of log2(1+2^x) over the key tiles already visited
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      ok = wait_or_abort(bar(kBarSFull + (j & 1)), (j >> 1) & 1, abort_flag, p, 30);
      if (ok && j >= 2) ok = wait_or_abort(bar(kBarPEmpty + (j & 1)), ((j >> 1) - 1) & 1, abort_flag, p, 31);
      uint8_t *gP = gP0 + (j & 1) * Cfg::kPBytes;
      if (!ok) break;
      tc_fence_after();
      const uint32_t ts = tS[j & 1] + lane_off;
      float R = ex2(-(float)run);   // product of (1 - beta) over the keys after this tile
      float logsum = 0.f;           // sum of log2(1 + 2^x) over this tile's allowed keys
      if (j == 0) {                 // diagonal tile: masked, one rolled loop
#pragma unroll 1
        for (int ch = 3; ch >= 0; --ch) {
          uint32_t v[32];
          tmem_ld32(ts + ch * 32, v);
          tmem_wait_ld_regs(v);
          if (ch == 0) {            // the whole row of S is in registers or consumed: the buffer may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarSEmpty + (j & 1)));
          }
          fwd_row_chunk<kFp16, true>(v, ch * 32, r, ac, scale2, R, logsum, gP);
        }
      } else {                      // the row is read 32 columns at a time, one load ahead of the arithmetic
        uint32_t va[32], vb[32];
        tmem_ld32(ts + 96, va);
#pragma unroll 1
        for (int pair = 1; pair >= 0; --pair) {
          const int c0 = pair * 64;
          tmem_wait_ld_regs(va);
          tmem_ld32(ts + c0, vb);
          fwd_row_chunk<kFp16, false>(va, c0 + 32, r, ac, scale2, R, logsum, gP);
          tmem_wait_ld_regs(vb);
          if (pair == 1) {
            tmem_ld32(ts + 32, va);
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarSEmpty + (j & 1)));
          }
          fwd_row_chunk<kFp16, false>(vb, c0, r, ac, scale2, R, logsum, gP);
        }
      }
      run += (double)logsum;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull + (j & 1)));
    }
    // ---- epilogue: O (TMEM) -> global, rem, log_rem
    if (ok) ok = wait_or_abort(bar(kBarOFull), 0, abort_flag, p, 32);
    if (ok) {
      tc_fence_after();
      const int gi = I * kBM + r;
      const bool valid = gi < c.len;
      using T = typename std::conditional<kFp16, __half, __nv_bfloat16>::type;
      T *orow = reinterpret_cast<T *>(p.o.ptr) + c.boff * p.o.sb + (long long)h * p.o.sh + (c.tok0 + gi) * p.o.st;
      store_acc_rows<D, kFp16, T>(tO + lane_off, orow, valid, p.head_dim, 1.f);
      if (valid) {
        const long long idx = (c.boff * p.heads + h) * p.tokens + c.tok0 + gi;
        reinterpret_cast<T *>(p.rem)[idx] = from_f32<T>(ex2(-(float)run));
        p.log_rem[idx] = -run;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

cudaError_t make_tile_map(CUtensorMap *map, const TensorRef &t, const KParams &p, int dtype, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return cudaErrorNotSupported;
  const cuuint64_t esz = 2;
  long long sb_el = t.sb > 0 ? t.sb : (t.sh > 0 ? t.sh * p.heads : (long long)p.tokens * p.head_dim);
  long long sh_el = t.sh > 0 ? t.sh : (long long)p.tokens * p.head_dim;
  cuuint64_t dims[4] = {(cuuint64_t)p.head_dim, (cuuint64_t)p.tokens, (cuuint64_t)p.heads, (cuuint64_t)p.batch};
  cuuint64_t strides[3] = {(cuuint64_t)t.st * esz, (cuuint64_t)sh_el * esz, (cuuint64_t)sb_el * esz};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dtype == SB_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// The forward for head sizes above 64 works on 256 query rows per CTA (two 128-row tiles sharing the K/V stream).
int tc_tile(int head_dim, bool backward) { return (!backward && head_dim > 64) ? 256 : kBM; }

cudaError_t sm_count(int *out) {
  static int cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (cached[dev] == 0) {
    int n = 0;
    if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    cached[dev] = n;
  }
  *out = cached[dev];
  return cudaSuccess;
}

bool tc_supported(int dtype, int head_dim, bool backward) {
  (void)backward;
  return (dtype == SB_DTYPE_BF16 || dtype == SB_DTYPE_F16) && head_dim % 8 == 0 && head_dim <= 128;
}

template <int D, bool kFp16>
static cudaError_t launch_fwd_t(const KParams &p, int dtype, cudaStream_t s) {
  CUtensorMap mq, mk, mv;
  cudaError_t e;
  if ((e = make_tile_map(&mq, p.q, p, dtype)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mk, p.k, p, dtype)) != cudaSuccess) return e;
  if ((e = make_tile_map(&mv, p.v, p, dtype)) != cudaSuccess) return e;
  auto kernel = tc_fwd_kernel<D, kFp16>;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<D>::kSmem);
  if (e != cudaSuccess) return e;
  const dim3 grid((unsigned)item_blocks(p, 1));
  kernel<<<grid, kTcThreads, FwdCfg<D>::kSmem, s>>>(mq, mk, mv, p);
  return cudaGetLastError();
}

cudaError_t launch_tc_fwd(const KParams &p, int dtype, cudaStream_t s, int *launches) {
  *launches += 1;
  const bool f16 = dtype == SB_DTYPE_F16;
  if (p.head_dim <= 64) return f16 ? launch_fwd_t<64, true>(p, dtype, s) : launch_fwd_t<64, false>(p, dtype, s);
  return launch_tc_fwd256(p, dtype, s);
}

}  // namespace sb
