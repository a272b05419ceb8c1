// CUDA-core (fp32 FMA) kernels: the exact path for fp32 tensors and for head sizes the tensor-core
// kernels do not take.  Also holds the two helper kernels every path uses: the sequence-table
// builder and the tail zero-fill.
//
// Structure (shared with the tensor-core path):
//   forward      one block per (sequence, 32-row query tile, head); key tiles are walked from the
//                diagonal back to the sequence start while every row carries sum softplus(z), so the
//                log-space suffix sum needs no second pass              (reference: _forward_one_row,
//                sb_varlen_fwd.py:81-215)
//   backward A   query-stationary, key tiles 0 -> diagonal: dQ, plus the per-(row, key tile)
//                boundary values R1 (suffix sum of log(1-beta) from this key tile on) and S2 (prefix sum
//                of G before this key tile)                             (reference: _backward_one_row,
//                sb_varlen_bwd.py:297-481, which adds dK/dV under a spin lock instead)
//   backward B   key-stationary: recomputes each tile from R1/S2 and accumulates dK, dV in registers;
//                no atomics, no locks, fixed summation order.
#include "sb_common.cuh"

namespace sb {

// ------------------------------------------------------------------------------------------------
// Sequence table: exclusive prefix of tiles per sequence and of (query tile, key tile) pairs.
// ------------------------------------------------------------------------------------------------
// Work items by descending weight (see decode_item): a counting sort over classes of `order_span` consecutive tiles
// (counted in units of `group`), the heaviest class first.  The tiles of one sequence inside a class stay neighbours
// (they read the same keys or queries at about the same time and share them through L2); the order of the
// sequences inside a class is whatever the shared-memory atomics give, which does not matter.
constexpr int kMaxClasses = 8192;
__device__ __forceinline__ int seq_tiles(const KParams &p, int s) {
  const long long start = s == 0 ? 0 : load_cu(p, s - 1);
  const long long len = load_cu(p, s) - start;
  if (len < 0 || len > p.max_seqlen) return 0;
  return (int)((len + p.tile - 1) / p.tile);
}
__device__ void build_order(const KParams &p, int group, int2 *out, int hdr_slot, int *s_cls) {
  const int t = threadIdx.x;
  const int span = p.order_span;                         // entries of one sequence that stay neighbours
  const int m_max = (p.n_max + group - 1) / group;       // entries of the longest sequence
  const int c_max = (m_max + span - 1) / span;           // classes
  if (c_max > kMaxClasses) {   // sequences beyond millions of tokens: sequence by sequence, serially
    if (t == 0) {
      int pos = 0;
      for (int s = 0; s < p.num_seq; ++s)
        for (int j = (seq_tiles(p, s) + group - 1) / group - 1; j >= 0; --j) out[pos++] = make_int2(s, j * group);
      p.hdr[hdr_slot] = pos;
    }
    __syncthreads();
    return;
  }
  for (int j = t; j < c_max; j += blockDim.x) s_cls[j] = 0;
  __syncthreads();
  for (int s = t; s < p.num_seq; s += blockDim.x) {   // entries per class
    const int m = (seq_tiles(p, s) + group - 1) / group;
    for (int cl = 0; cl * span < m; ++cl) atomicAdd(&s_cls[cl], min(span, m - cl * span));
  }
  __syncthreads();
  if (t == 0) {   // -> first position of every class, the heaviest class first
    int pos = 0;
    for (int cl = c_max - 1; cl >= 0; --cl) {
      const int n = s_cls[cl];
      s_cls[cl] = pos;
      pos += n;
    }
    p.hdr[hdr_slot] = pos;
  }
  __syncthreads();
  for (int s = t; s < p.num_seq; s += blockDim.x) {
    const int m = (seq_tiles(p, s) + group - 1) / group;
    for (int cl = 0; cl * span < m; ++cl) {
      const int n = min(span, m - cl * span);
      const int pos = atomicAdd(&s_cls[cl], n);
      for (int i = 0; i < n; ++i) out[pos + i] = make_int2(s, (cl * span + n - 1 - i) * group);   // heaviest first
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(256) prep_kernel(KParams p) {
  __shared__ int s_cls[kMaxClasses];
  __shared__ long long s_tiles[256];
  __shared__ long long s_pairs[256];
  const int t = threadIdx.x;
  if (t < 8) p.hdr[t] = 0;   // the header is this kernel's to initialise (a fixed-length batch uses clear_hdr_kernel)
  __syncthreads();
  const int per = (p.num_seq + 255) / 256;
  const int s0 = t * per, s1 = min(p.num_seq, s0 + per);
  const int busy = (p.num_seq + per - 1) / per;   // threads that own sequences
  long long tiles = 0, pairs = 0;
  int bad = -1;
  for (int s = s0; s < s1; ++s) {
    const long long start = s == 0 ? 0 : load_cu(p, s - 1);
    const long long end = load_cu(p, s);
    const long long len = end - start;
    if (len < 0 || end > p.tokens || start < 0 || len > p.max_seqlen) { if (bad < 0) bad = s; continue; }
    const long long n = (len + p.tile - 1) / p.tile;
    tiles += n;
    pairs += n * (n + 1) / 2;
  }
  s_tiles[t] = tiles;
  s_pairs[t] = pairs;
  if (bad >= 0) {
    p.hdr[0] = 1;
    if (p.status != nullptr) { p.status[0] = SB_DEV_BAD_CU_SEQLENS; p.status[1] = bad; }
  }
  __syncthreads();
  if (t == 0) {
    if (p.check_leading_zero && load_cu(p, -1) != 0) {
      p.hdr[0] = 1;
      if (p.status != nullptr) { p.status[0] = SB_DEV_BAD_CU_SEQLENS; p.status[1] = -1; }
    }
    long long a = 0, b = 0;
    for (int i = 0; i < busy; ++i) {
      const long long x = s_tiles[i], y = s_pairs[i];
      s_tiles[i] = a; s_pairs[i] = b;
      a += x; b += y;
    }
    p.tile_prefix[p.num_seq] = (int)a;
    p.pair_prefix[p.num_seq] = b;
    p.hdr[1] = p.num_seq > 0 ? (int)load_cu(p, p.num_seq - 1) : 0;
    if (a > p.tiles_cap || b > p.pairs_cap) p.hdr[0] = 1;  // cannot happen for valid cu_seqlens
  }
  __syncthreads();
  tiles = s_tiles[t];
  pairs = s_pairs[t];
  for (int s = s0; s < s1; ++s) {
    p.tile_prefix[s] = (int)tiles;
    p.pair_prefix[s] = pairs;
    const long long start = s == 0 ? 0 : load_cu(p, s - 1);
    const long long len = load_cu(p, s) - start;
    if (len < 0 || len > p.max_seqlen) continue;
    const long long n = (len + p.tile - 1) / p.tile;
    tiles += n;
    pairs += n * (n + 1) / 2;
  }
  __syncthreads();
  if (p.hdr[0]) return;   // bad cu_seqlens: no kernel will look at the order
  build_order(p, 1, const_cast<int2 *>(p.order), 2, s_cls);
  if (p.order2 != nullptr) build_order(p, 2, const_cast<int2 *>(p.order2), 3, s_cls);
}

__global__ void clear_hdr_kernel(int *hdr, unsigned long long *trace) {
  if (threadIdx.x < 8) hdr[threadIdx.x] = 0;
  if (trace != nullptr)
    for (int i = threadIdx.x; i < (int)(kTraceBytes / 8); i += blockDim.x) trace[i] = 0;
}

cudaError_t launch_prep(const KParams &p, cudaStream_t s) {
  if (p.cu == nullptr || p.trace != nullptr) clear_hdr_kernel<<<1, 32, 0, s>>>(p.hdr, p.trace);
  if (p.cu != nullptr) prep_kernel<<<1, 256, 0, s>>>(p);
  return cudaGetLastError();
}

// Rows past the end of the last packed sequence belong to no sequence: write zeros there.  When the sequence table
// was refused (bad cu_seqlens: every other kernel of the call has returned at once), every row of the outputs is
// filled with NaN instead, so that a caller who does not look at the status word cannot mistake uninitialised memory
// for results.
template <typename T>
__global__ void zero_tail_kernel(KParams p, bool backward) {
  const bool refused = p.hdr[0] != 0;
  const long long first = refused ? 0 : p.hdr[1];
  const float fill = refused ? __int_as_float(0x7fc00000) : 0.f;
  const int h = p.head0 + blockIdx.y;
  const int d = p.head_dim;
  for (long long row = first + blockIdx.x; row < p.tokens; row += gridDim.x) {
    if (!backward) {
      T *o = reinterpret_cast<T *>(p.o.ptr) + h * p.o.sh + row * p.o.st;
      for (int x = threadIdx.x; x < d; x += blockDim.x) o[x] = from_f32<T>(fill);
      if (threadIdx.x == 0) {
        reinterpret_cast<T *>(p.rem)[(long long)h * p.tokens + row] = from_f32<T>(fill);
        p.log_rem[(long long)h * p.tokens + row] = (double)fill;
      }
    } else {
      T *a = reinterpret_cast<T *>(p.dq.ptr) + h * p.dq.sh + row * p.dq.st;
      T *b = reinterpret_cast<T *>(p.dk.ptr) + h * p.dk.sh + row * p.dk.st;
      T *c = reinterpret_cast<T *>(p.dv.ptr) + h * p.dv.sh + row * p.dv.st;
      for (int x = threadIdx.x; x < d; x += blockDim.x) { a[x] = b[x] = c[x] = from_f32<T>(fill); }
    }
  }
}

// Backward with out = o + rem * v: the upstream gradient of rem gains <d_out, v> per row, and dv gains rem * d_out
// (rem = 2^log_rem, from the saved fp64 value) on the rows that belong to a sequence.  Two elementwise kernels over
// the (batch, heads, tokens) rows: grid (token blocks, heads, batch); `group` consecutive lanes share a row, each
// lane holding `kVec` consecutive elements (16 bytes when the rows allow it, else one element).
template <typename T, int kVec>
struct alignas(16) RowVec {
  T e[kVec];
};
template <typename T, int kVec>
__device__ __forceinline__ RowVec<T, kVec> load_vec(const T *src) {
  RowVec<T, kVec> r;
  if (kVec == 1) r.e[0] = *src;
  else *reinterpret_cast<uint4 *>(&r) = *reinterpret_cast<const uint4 *>(src);
  return r;
}

template <typename T, int kVec>
__global__ void __launch_bounds__(256) fused_drem_kernel(KParams p, int group) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rows_per_warp = 32 / group;
  const long long tok = ((long long)blockIdx.x * 8 + warp) * rows_per_warp + lane / group;
  const int x0 = (lane % group) * kVec;
  const long long h = blockIdx.y, b = blockIdx.z;
  float s = 0.f;
  if (tok < p.tokens) {
    const T *g = reinterpret_cast<const T *>(p.d_o.ptr) + b * p.d_o.sb + h * p.d_o.sh + tok * p.d_o.st;
    const T *v = reinterpret_cast<const T *>(p.v.ptr) + b * p.v.sb + h * p.v.sh + tok * p.v.st;
    for (int x = x0; x < p.head_dim; x += group * kVec) {
      const RowVec<T, kVec> gv = load_vec<T, kVec>(g + x), vv = load_vec<T, kVec>(v + x);
#pragma unroll
      for (int i = 0; i < kVec; ++i) s = fmaf(to_f32<T>(gv.e[i]), to_f32<T>(vv.e[i]), s);
    }
  }
  for (int o = group >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (tok < p.tokens && x0 == 0) {
    const long long row = (b * p.heads + h) * p.tokens + tok;
    reinterpret_cast<T *>(p.d_rem_fused)[row] =
        from_f32<T>(s + (p.d_rem != nullptr ? to_f32<T>(reinterpret_cast<const T *>(p.d_rem)[row]) : 0.f));
  }
}

template <typename T, int kVec>
__global__ void __launch_bounds__(256) fused_dv_kernel(KParams p, int group) {
  if (p.hdr[0]) return;
  const long long covered = p.cu != nullptr ? (long long)p.hdr[1] : p.tokens;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rows_per_warp = 32 / group;
  const long long tok = ((long long)blockIdx.x * 8 + warp) * rows_per_warp + lane / group;
  if (tok >= covered) return;
  const int x0 = (lane % group) * kVec;
  const long long h = blockIdx.y, b = blockIdx.z;
  const T *g = reinterpret_cast<const T *>(p.d_o.ptr) + b * p.d_o.sb + h * p.d_o.sh + tok * p.d_o.st;
  T *dv = reinterpret_cast<T *>(p.dv.ptr) + b * p.dv.sb + h * p.dv.sh + tok * p.dv.st;
  const float rem = exp2f((float)p.log_rem[(b * p.heads + h) * p.tokens + tok]);
  for (int x = x0; x < p.head_dim; x += group * kVec) {
    const RowVec<T, kVec> gv = load_vec<T, kVec>(g + x);
    RowVec<T, kVec> dvv = load_vec<T, kVec>(dv + x);
#pragma unroll
    for (int i = 0; i < kVec; ++i) dvv.e[i] = from_f32<T>(fmaf(rem, to_f32<T>(gv.e[i]), to_f32<T>(dvv.e[i])));
    if (kVec == 1) dv[x] = dvv.e[0];
    else *reinterpret_cast<uint4 *>(dv + x) = *reinterpret_cast<const uint4 *>(&dvv);
  }
}

// 16-byte accesses need rows that start on 16-byte boundaries and hold a whole number of them.
static bool rows_vectorizable(const TensorRef &t, int head_dim, int esize) {
  const long long m = 16 / esize;
  return reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0 && head_dim % m == 0 && t.sb % m == 0 && t.sh % m == 0 && t.st % m == 0;
}

template <typename T, bool kDv>
static cudaError_t launch_fused_t(const KParams &p, cudaStream_t s) {
  constexpr int kVec = 16 / (int)sizeof(T);
  const bool vec = rows_vectorizable(p.d_o, p.head_dim, sizeof(T)) &&
                   rows_vectorizable(kDv ? p.dv : p.v, p.head_dim, sizeof(T));
  const int per_lane = vec ? kVec : 1;
  int group = 1;
  while (group < 32 && group * per_lane < p.head_dim) group <<= 1;
  const long long rows_per_block = 8 * (32 / group);
  const dim3 grid((unsigned)((p.tokens + rows_per_block - 1) / rows_per_block), p.heads, p.batch);
  if (kDv) {
    if (vec) fused_dv_kernel<T, kVec><<<grid, 256, 0, s>>>(p, group);
    else fused_dv_kernel<T, 1><<<grid, 256, 0, s>>>(p, group);
  } else {
    if (vec) fused_drem_kernel<T, kVec><<<grid, 256, 0, s>>>(p, group);
    else fused_drem_kernel<T, 1><<<grid, 256, 0, s>>>(p, group);
  }
  return cudaGetLastError();
}

cudaError_t launch_fused_drem(const KParams &p, int dtype, cudaStream_t s) {
  if (dtype == SB_DTYPE_F32) return launch_fused_t<float, false>(p, s);
  if (dtype == SB_DTYPE_BF16) return launch_fused_t<__nv_bfloat16, false>(p, s);
  return launch_fused_t<__half, false>(p, s);
}

cudaError_t launch_fused_dv(const KParams &p, int dtype, cudaStream_t s) {
  if (dtype == SB_DTYPE_F32) return launch_fused_t<float, true>(p, s);
  if (dtype == SB_DTYPE_BF16) return launch_fused_t<__nv_bfloat16, true>(p, s);
  return launch_fused_t<__half, true>(p, s);
}

cudaError_t launch_zero_tail(const KParams &p, int dtype, bool backward, cudaStream_t s) {
  if (p.cu == nullptr) return cudaSuccess;
  dim3 grid(32, p.head_cnt);
  if (dtype == SB_DTYPE_F32) zero_tail_kernel<float><<<grid, 128, 0, s>>>(p, backward);
  else if (dtype == SB_DTYPE_BF16) zero_tail_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(p, backward);
  else zero_tail_kernel<__half><<<grid, 128, 0, s>>>(p, backward);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// SIMT kernels.  256 threads; thread t owns output row t/8 and columns (t%8) + 8u.
// ------------------------------------------------------------------------------------------------
constexpr int kT = kSimtTile;   // 32
constexpr int kLdS = kT + 1;

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

template <typename T>
__device__ __forceinline__ void load_rows(float *dst, int ld, const TensorRef &t, const TileCoord &c, int h,
                                          int tile_idx, int d) {
  const T *base = reinterpret_cast<const T *>(t.ptr) + c.boff * t.sb + (long long)h * t.sh;
  for (int e = threadIdx.x; e < kT * d; e += blockDim.x) {
    const int r = e / d, x = e - r * d;
    const int li = tile_idx * kT + r;
    dst[r * ld + x] = li < c.len ? to_f32<T>(base[(c.tok0 + li) * t.st + x]) : 0.f;
  }
}

// S[r][c] = scale * <A_r, B_c> for the 4 columns of this thread.
__device__ __forceinline__ void tile_dot(float *S, const float *A, const float *B, int ld, int d, float scale) {
  const int r = threadIdx.x >> 3, cg = threadIdx.x & 7;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  const float *a = A + r * ld;
  const float *b0 = B + cg * ld, *b1 = b0 + 8 * ld, *b2 = b0 + 16 * ld, *b3 = b0 + 24 * ld;
  for (int x = 0; x < d; ++x) {
    const float av = a[x];
    s0 = fmaf(av, b0[x], s0); s1 = fmaf(av, b1[x], s1); s2 = fmaf(av, b2[x], s2); s3 = fmaf(av, b3[x], s3);
  }
  S[r * kLdS + cg] = s0 * scale; S[r * kLdS + cg + 8] = s1 * scale;
  S[r * kLdS + cg + 16] = s2 * scale; S[r * kLdS + cg + 24] = s3 * scale;
}

template <typename T, int U>
__global__ void __launch_bounds__(256) simt_fwd_kernel(KParams p) {
  extern __shared__ float smem[];
  if (p.hdr[0]) return;
  TileCoord c;
  if (!decode_tile(p, blockIdx.x, true, c)) return;
  const int d = p.head_dim, ld = d + 1;
  float *Qs = smem, *Ks = Qs + kT * ld, *Vs = Ks + kT * ld, *Ss = Vs + kT * ld;
  const int h = p.head0 + blockIdx.y;
  const int t = threadIdx.x, r = t >> 3, cg = t & 7;
  const int I = c.idx;

  load_rows<T>(Qs, ld, p.q, c, h, I, d);
  float acc[U];
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = 0.f;
  float run_sp = 0.f;  // sum of softplus(z) over the key tiles already visited (rows of warp 0)

  for (int J = I; J >= 0; --J) {
    load_rows<T>(Ks, ld, p.k, c, h, J, d);
    load_rows<T>(Vs, ld, p.v, c, h, J, d);
    __syncthreads();
    tile_dot(Ss, Qs, Ks, ld, d, p.scale);
    __syncthreads();
    if (t < kT) {
      const int gi = I * kT + t;
      float suffix = 0.f;
      for (int j = kT - 1; j >= 0; --j) {
        const int gj = J * kT + j;
        const bool allowed = gi < c.len && (p.attend_current ? gj <= gi : gj < gi);
        const float z = Ss[t * kLdS + j];
        float a = 0.f;
        if (allowed) {
          suffix += softplus_f(z);
          a = expf(z - run_sp - suffix);
        }
        Ss[t * kLdS + j] = a;
      }
      run_sp += suffix;
    }
    __syncthreads();
    if (p.attn != nullptr) {   // debugging aid: the attention weights of this tile, keys indexed inside the sequence
      for (int e = t; e < kT * kT; e += blockDim.x) {
        const int rr = e / kT, j = e - rr * kT;
        const int gi = I * kT + rr, gj = J * kT + j;
        if (gi < c.len && gj < c.len && gj < p.attn_cols)
          p.attn[((c.boff * p.heads + h) * p.tokens + c.tok0 + gi) * p.attn_cols + gj] = Ss[rr * kLdS + j];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = cg + 8 * u;
      if (x < d) {
        float s = acc[u];
        for (int j = 0; j < kT; ++j) s = fmaf(Ss[r * kLdS + j], Vs[j * ld + x], s);
        acc[u] = s;
      }
    }
    __syncthreads();
  }

  const int gi = I * kT + r;
  if (p.fuse_rem_v) {   // out = o + rem * v: the row owners publish rem through the free score tile
    if (t < kT) Ss[t * kLdS] = expf(-run_sp);
    __syncthreads();
  }
  if (gi < c.len) {
    T *o = reinterpret_cast<T *>(p.o.ptr) + c.boff * p.o.sb + (long long)h * p.o.sh + (c.tok0 + gi) * p.o.st;
    const T *vrow = reinterpret_cast<const T *>(p.v.ptr) + c.boff * p.v.sb + (long long)h * p.v.sh + (c.tok0 + gi) * p.v.st;
    const float rem_r = p.fuse_rem_v ? Ss[r * kLdS] : 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = cg + 8 * u;
      if (x < d) o[x] = from_f32<T>(p.fuse_rem_v ? fmaf(rem_r, to_f32<T>(vrow[x]), acc[u]) : acc[u]);
    }
  }
  if (t < kT && I * kT + t < c.len) {
    const long long idx = (c.boff * p.heads + h) * p.tokens + c.tok0 + I * kT + t;
    reinterpret_cast<T *>(p.rem)[idx] = from_f32<T>(expf(-run_sp));
    p.log_rem[idx] = -(double)run_sp * kLog2eD;
  }
}

// Row pass of the backward: on entry Z holds z, P holds dP; on exit Z holds dz and P holds A.
// r1 = sum of log(1-beta) over the allowed keys from this tile's first key on (<= 0).
__device__ __forceinline__ void bwd_row_pass(float *Z, float *P, int row, int gi, int J, int len, int ac,
                                             float r1, float gpre, float dr, float &sp_sum, float &g_sum) {
  float spl = 0.f, gs = 0.f;
  for (int j = 0; j < kT; ++j) {
    const int gj = J * kT + j;
    const bool allowed = gi < len && (ac ? gj <= gi : gj < gi);
    const float z = Z[row * kLdS + j];
    float a = 0.f, dz = 0.f;
    if (allowed) {
      a = expf(z + r1 + spl);
      spl += softplus_f(z);
      const float g = a * (P[row * kLdS + j] - dr);
      gs += g;
      const float beta = 1.f / (1.f + expf(-z));
      dz = g - beta * (gpre + gs);
    }
    Z[row * kLdS + j] = dz;
    P[row * kLdS + j] = a;
  }
  sp_sum = spl;
  g_sum = gs;
}

template <typename T, int U>
__global__ void __launch_bounds__(256) simt_bwd_dq_kernel(KParams p) {
  extern __shared__ float smem[];
  if (p.hdr[0]) return;
  TileCoord c;
  if (!decode_tile(p, blockIdx.x, true, c)) return;
  const int d = p.head_dim, ld = d + 1;
  float *Qs = smem, *Gs = Qs + kT * ld, *Ks = Gs + kT * ld, *Vs = Ks + kT * ld;
  float *Zs = Vs + kT * ld, *Ps = Zs + kT * kLdS;
  const int hh = blockIdx.y, h = p.head0 + hh;
  const int t = threadIdx.x, r = t >> 3, cg = t & 7;
  const int I = c.idx;

  load_rows<T>(Qs, ld, p.q, c, h, I, d);
  load_rows<T>(Gs, ld, p.d_o, c, h, I, d);
  float acc[U];
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = 0.f;
  double r1 = 0.0;
  float gpre = 0.f, dr = 0.f;
  const int my_row = I * kT + t;
  if (t < kT && my_row < c.len) {
    const long long idx = (c.boff * p.heads + h) * p.tokens + c.tok0 + my_row;
    r1 = p.log_rem[idx] * kLn2D;
    dr = load_drem<T>(p, idx);
  }

  for (int J = 0; J <= I; ++J) {
    load_rows<T>(Ks, ld, p.k, c, h, J, d);
    load_rows<T>(Vs, ld, p.v, c, h, J, d);
    __syncthreads();
    tile_dot(Zs, Qs, Ks, ld, d, p.scale);
    tile_dot(Ps, Gs, Vs, ld, d, 1.f);
    __syncthreads();
    if (t < kT) {
      const long long slot = ((long long)hh * p.pairs_cap + c.pair0 + (long long)I * (I + 1) / 2 + J) * kT + t;
      p.bnd_r1[slot] = (float)r1;
      p.bnd_s2[slot] = gpre;
      float sp_sum, g_sum;
      bwd_row_pass(Zs, Ps, t, my_row, J, c.len, p.attend_current, (float)r1, gpre, dr, sp_sum, g_sum);
      r1 += (double)sp_sum;
      gpre += g_sum;
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = cg + 8 * u;
      if (x < d) {
        float s = acc[u];
        for (int j = 0; j < kT; ++j) s = fmaf(Zs[r * kLdS + j], Ks[j * ld + x], s);
        acc[u] = s;
      }
    }
    __syncthreads();
  }

  const int gi = I * kT + r;
  if (gi < c.len) {
    T *o = reinterpret_cast<T *>(p.dq.ptr) + c.boff * p.dq.sb + (long long)h * p.dq.sh + (c.tok0 + gi) * p.dq.st;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = cg + 8 * u;
      if (x < d) o[x] = from_f32<T>(acc[u] * p.scale);
    }
  }
}

template <typename T, int U>
__global__ void __launch_bounds__(256) simt_bwd_dkv_kernel(KParams p) {
  extern __shared__ float smem[];
  if (p.hdr[0]) return;
  TileCoord c;
  if (!decode_tile(p, blockIdx.x, false, c)) return;
  const int d = p.head_dim, ld = d + 1;
  float *Qs = smem, *Gs = Qs + kT * ld, *Ks = Gs + kT * ld, *Vs = Ks + kT * ld;
  float *Zs = Vs + kT * ld, *Ps = Zs + kT * kLdS;
  const int hh = blockIdx.y, h = p.head0 + hh;
  const int t = threadIdx.x, r = t >> 3, cg = t & 7;
  const int J = c.idx;

  load_rows<T>(Ks, ld, p.k, c, h, J, d);
  load_rows<T>(Vs, ld, p.v, c, h, J, d);
  float dk[U], dv[U];
#pragma unroll
  for (int u = 0; u < U; ++u) { dk[u] = 0.f; dv[u] = 0.f; }

  for (int I = J; I < c.n_tiles; ++I) {
    load_rows<T>(Qs, ld, p.q, c, h, I, d);
    load_rows<T>(Gs, ld, p.d_o, c, h, I, d);
    __syncthreads();
    tile_dot(Zs, Qs, Ks, ld, d, p.scale);
    tile_dot(Ps, Gs, Vs, ld, d, 1.f);
    __syncthreads();
    if (t < kT) {
      const int gi = I * kT + t;
      float dr = 0.f;
      if (gi < c.len)
        dr = load_drem<T>(p, (c.boff * p.heads + h) * p.tokens + c.tok0 + gi);
      const long long slot = ((long long)hh * p.pairs_cap + c.pair0 + (long long)I * (I + 1) / 2 + J) * kT + t;
      float sp_sum, g_sum;
      bwd_row_pass(Zs, Ps, t, gi, J, c.len, p.attend_current, p.bnd_r1[slot], p.bnd_s2[slot], dr, sp_sum, g_sum);
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = cg + 8 * u;
      if (x < d) {
        float a = dk[u], b = dv[u];
        for (int i = 0; i < kT; ++i) {
          a = fmaf(Zs[i * kLdS + r], Qs[i * ld + x], a);
          b = fmaf(Ps[i * kLdS + r], Gs[i * ld + x], b);
        }
        dk[u] = a; dv[u] = b;
      }
    }
    __syncthreads();
  }

  const int gj = J * kT + r;
  if (gj < c.len) {
    T *ok = reinterpret_cast<T *>(p.dk.ptr) + c.boff * p.dk.sb + (long long)h * p.dk.sh + (c.tok0 + gj) * p.dk.st;
    T *ov = reinterpret_cast<T *>(p.dv.ptr) + c.boff * p.dv.sb + (long long)h * p.dv.sh + (c.tok0 + gj) * p.dv.st;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int x = cg + 8 * u;
      if (x < d) { ok[x] = from_f32<T>(dk[u] * p.scale); ov[x] = from_f32<T>(dv[u]); }
    }
  }
}

template <typename K>
static cudaError_t launch_one(K kernel, const KParams &p, size_t smem, cudaStream_t s) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(p.tiles_cap, p.head_cnt);
  kernel<<<grid, 256, smem, s>>>(p);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t simt_fwd_t(const KParams &p, cudaStream_t s) {
  const size_t smem = (size_t)(3 * kT * (p.head_dim + 1) + kT * kLdS) * sizeof(float);
  if (p.head_dim <= 64) return launch_one(simt_fwd_kernel<T, 8>, p, smem, s);
  if (p.head_dim <= 128) return launch_one(simt_fwd_kernel<T, 16>, p, smem, s);
  return launch_one(simt_fwd_kernel<T, 32>, p, smem, s);
}

template <typename T>
static cudaError_t simt_bwd_t(const KParams &p, cudaStream_t s) {
  const size_t smem = (size_t)(4 * kT * (p.head_dim + 1) + 2 * kT * kLdS) * sizeof(float);
  cudaError_t e = cudaSuccess;
  if (p.head_dim <= 64) {
    if (!p.skip_dq) e = launch_one(simt_bwd_dq_kernel<T, 8>, p, smem, s);
    if (e == cudaSuccess && !p.skip_dkv) e = launch_one(simt_bwd_dkv_kernel<T, 8>, p, smem, s);
  } else if (p.head_dim <= 128) {
    if (!p.skip_dq) e = launch_one(simt_bwd_dq_kernel<T, 16>, p, smem, s);
    if (e == cudaSuccess && !p.skip_dkv) e = launch_one(simt_bwd_dkv_kernel<T, 16>, p, smem, s);
  } else {
    if (!p.skip_dq) e = launch_one(simt_bwd_dq_kernel<T, 32>, p, smem, s);
    if (e == cudaSuccess && !p.skip_dkv) e = launch_one(simt_bwd_dkv_kernel<T, 32>, p, smem, s);
  }
  return e;
}

cudaError_t launch_simt_fwd(const KParams &p, int dtype, cudaStream_t s, int *launches) {
  *launches += 1;
  if (dtype == SB_DTYPE_F32) return simt_fwd_t<float>(p, s);
  if (dtype == SB_DTYPE_BF16) return simt_fwd_t<__nv_bfloat16>(p, s);
  return simt_fwd_t<__half>(p, s);
}

cudaError_t launch_simt_bwd(const KParams &p, int dtype, cudaStream_t s, int *launches) {
  *launches += (p.skip_dq ? 0 : 1) + (p.skip_dkv ? 0 : 1);
  if (dtype == SB_DTYPE_F32) return simt_bwd_t<float>(p, s);
  if (dtype == SB_DTYPE_BF16) return simt_bwd_t<__nv_bfloat16>(p, s);
  return simt_bwd_t<__half>(p, s);
}

}  // namespace sb
