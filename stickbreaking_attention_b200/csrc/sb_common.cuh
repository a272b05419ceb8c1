// Shared host/device definitions of the stick-breaking attention kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sb_b200.h"

namespace sb {

constexpr float kLog2e = 1.4426950408889634f;
constexpr double kLog2eD = 1.4426950408889634074;
constexpr double kLn2D = 0.69314718055994530942;

struct TensorRef {
  char *ptr;
  long long sb, sh, st;  // element strides of batch, head, token
};

// Everything a kernel needs; passed by value.
struct KParams {
  TensorRef q, k, v, o, d_o, dq, dk, dv;
  char *rem;
  const char *d_rem;
  double *log_rem;
  const void *cu;      // sequence end offsets, or nullptr for a fixed-length batch
  int cu64;
  int batch, heads, head_dim, num_seq;
  long long tokens;
  int attend_current;
  float scale;         // logit scale (natural units)
  int head0, head_cnt; // heads [head0, head0 + head_cnt) are processed by this launch
  int tile;            // rows per query tile == keys per key tile of the launch
  int tiles_cap;       // upper bound on the number of query tiles over all sequences
  int n_max;           // upper bound on tiles per sequence
  int max_seqlen;
  int check_leading_zero;  // the element before cu[0] must be 0
  int skip_dq, skip_dkv;   // timing aids: leave one of the two backward kernels out
  int dense;               // measuring aid: do the per-score arithmetic even where it is known to give exact zeros
  const int2 *order;       // packed batches: work items by descending weight, see decode_item
  const int2 *order2;      // the same for every second tile (backward only)
  int order_span;          // entries of one sequence that stay neighbours in order / order2 (>= 1)
  int trace_mode;          // diagnostics builds: bit 1 = log every block's SM, start, first row work and end time
  int dbg;                 // experiments only (SbParams.reserved): 0 = normal arithmetic
  unsigned long long *trace;  // experiments only: event log of block (0,0) in the workspace tail, or nullptr
  // workspace views
  int *hdr;            // [0] abort flag, [1] end of the last sequence (varlen), [2] / [3] entries of order / order2
  int *tile_prefix;    // [num_seq + 1]  exclusive prefix of tiles per sequence (varlen)
  long long *pair_prefix;  // [num_seq + 1] exclusive prefix of n(n+1)/2 (varlen)
  float *bnd_r1;       // [head_cnt][pairs_cap][tile]  suffix sums of log(1-beta) at tile starts
  float *bnd_s2;       // [head_cnt][pairs_cap][tile]  prefix sums of G before each key tile
  unsigned short *az;  // stored-tiles mode: [head_cnt][pairs_cap][A, dz][128 query rows][128 keys], 16-bit; else null
  long long pairs_cap;
  float *attn;         // forward, CUDA-core kernels only: [batch][heads][tokens][attn_cols] attention weights, or null
  long long attn_cols;
  int fuse_rem_v;      // forward writes o + rem * v; backward folds the two extra gradient terms in
  char *d_rem_fused;   // backward with fuse_rem_v: [batch][heads][tokens] d_rem + <d_out, v> in the tensors' dtype,
                       // written by the first kernel of the call; `d_rem` then points here for the other kernels
  int *status;
};

// One (sequence, query-or-key tile) work item.
struct TileCoord {
  int seq;         // sequence (varlen) or batch element (fixed)
  int idx;         // tile index inside the sequence
  int n_tiles;     // tiles of this sequence
  int len;         // sequence length
  long long tok0;  // first token of the sequence on the tokens axis
  long long boff;  // batch element (fixed) else 0
  long long pair0; // first (query tile, key tile) pair slot of this sequence
};

__device__ __forceinline__ long long load_cu(const KParams &p, int i) {
  return p.cu64 ? reinterpret_cast<const long long *>(p.cu)[i]
                : (long long)reinterpret_cast<const int *>(p.cu)[i];
}

// Maps a work-item number to its sequence and tile.  Items are ordered by weight across ALL sequences: the tile with
// the most key (or query) tiles to visit comes first, so that the blocks that run longest start earliest and the
// last blocks of a launch are the short ones.  For a packed batch the order is a table the prep kernel writes
// (entries (sequence, k), k = tile index counted so that larger means heavier; `group` > 1 lists every group-th
// tile only); for a fixed-length batch it is arithmetic.  `reverse`: the heavy tiles are the late ones (a query
// tile sees all earlier keys); otherwise the early ones (a key tile is seen by all later queries).
__device__ __forceinline__ bool decode_item(const KParams &p, int item, int group, bool reverse, TileCoord &c) {
  int s, k;
  if (p.cu == nullptr) {
    const int n = (int)((p.tokens + p.tile - 1) / p.tile);
    const int m = (n + group - 1) / group;
    if (item >= m * p.batch) return false;
    const int j = item / p.batch;
    s = item - j * p.batch;
    k = (m - 1 - j) * group;
    c.n_tiles = n;
    c.len = (int)p.tokens;
    c.tok0 = 0;
    c.boff = s;
    c.pair0 = (long long)s * ((long long)n * (n + 1) / 2);
  } else {
    if (item >= p.hdr[group == 1 ? 2 : 3]) return false;
    const int2 e = (group == 1 ? p.order : p.order2)[item];
    s = e.x;
    k = e.y;
    c.n_tiles = p.tile_prefix[s + 1] - p.tile_prefix[s];
    c.tok0 = s == 0 ? 0 : load_cu(p, s - 1);
    c.len = (int)(load_cu(p, s) - c.tok0);
    c.boff = 0;
    c.pair0 = p.pair_prefix[s];
  }
  c.seq = s;
  c.idx = reverse ? k : c.n_tiles - 1 - k;
  return true;
}
__device__ __forceinline__ bool decode_tile(const KParams &p, int item, bool reverse, TileCoord &c) {
  return decode_item(p, item, 1, reverse, c);
}
// One-dimensional grids: block = item * head_cnt + head, so that equal-weight items of all heads are neighbours.
__device__ __forceinline__ bool decode_block(const KParams &p, int group, bool reverse, TileCoord &c, int &hh) {
  const int item = blockIdx.x / p.head_cnt;
  hh = blockIdx.x - item * p.head_cnt;
  return decode_item(p, item, group, reverse, c);
}
// Blocks to launch for such a grid (an upper bound for packed batches: surplus blocks leave at once).
inline long long item_blocks(const KParams &p, int group) {
  long long items;
  if (p.cu == nullptr) {
    const long long n = (p.tokens + p.tile - 1) / p.tile;
    items = ((n + group - 1) / group) * p.batch;
  } else {
    items = group == 1 ? p.tiles_cap : (p.tiles_cap + p.num_seq + 1) / 2;
  }
  return items * p.head_cnt;
}

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Upstream gradient of rem for row `idx` of the (batch, heads, tokens) array.
template <typename T>
__device__ __forceinline__ float load_drem(const KParams &p, long long idx) {
  return to_f32<T>(reinterpret_cast<const T *>(p.d_rem)[idx]);
}

// Host-side launch helpers implemented in the .cu files; all return cudaError_t of the launch.
cudaError_t launch_fused_drem(const KParams &p, int dtype, cudaStream_t s);   // fills d_rem_fused (all heads)
cudaError_t launch_fused_dv(const KParams &p, int dtype, cudaStream_t s);     // dv += rem * d_out (all heads)
cudaError_t launch_prep(const KParams &p, cudaStream_t s);
cudaError_t launch_zero_tail(const KParams &p, int dtype, bool backward, cudaStream_t s);
cudaError_t launch_simt_fwd(const KParams &p, int dtype, cudaStream_t s, int *launches);
cudaError_t launch_simt_bwd(const KParams &p, int dtype, cudaStream_t s, int *launches);
cudaError_t launch_tc_fwd(const KParams &p, int dtype, cudaStream_t s, int *launches);
cudaError_t launch_tc_bwd(const KParams &p, int dtype, cudaStream_t s, int *launches);
bool tc_supported(int dtype, int head_dim, bool backward);
int tc_tile(int head_dim, bool backward, int max_seqlen);   // rows per work item of the tensor-core kernels
cudaError_t launch_tc_fwd256(const KParams &p, int dtype, cudaStream_t s);
cudaError_t launch_tc_fwd128(const KParams &p, int dtype, cudaStream_t s);
cudaError_t sm_count(int *out);              // SMs of the current device (cached)

constexpr size_t kTraceBytes = 8 * 1024 * 16;   // workspace tail reserved for the event log

// Event log of block (0,0): each logging thread owns a lane of 1024 entries [tag << 32 | step][SM clock]
// and keeps its own cursor, so that logging costs two stores and no round trip.
#ifdef SB_TRACE
__device__ __forceinline__ void trace_event(const KParams &p, int lane_id, int &cursor, unsigned tag, unsigned step) {
  if (p.trace == nullptr || (p.trace_mode & 2) || blockIdx.x != 0 || blockIdx.y != 0 || cursor >= 1023) return;
  const unsigned long long t = (unsigned long long)clock64();   // SM clock: all logging threads share one SM
  unsigned long long *slot = p.trace + ((size_t)lane_id * 1024 + cursor) * 2;
  slot[0] = ((unsigned long long)tag << 32) | step;
  slot[1] = t;
  ++cursor;
}
// Block schedule log: [linear block id][3] = (globaltimer ns << 10 | SM id) at entry, first row work and exit.
__device__ __forceinline__ void trace_block(const KParams &p, int which) {
  if (p.trace == nullptr || !(p.trace_mode & 2)) return;
  const unsigned lin = blockIdx.y * gridDim.x + blockIdx.x;
  if (lin >= 5400) return;
  unsigned long long t;
  unsigned smid;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  p.trace[lin * 3 + which] = (t << 10) | smid;
}
#else   // the event log is compiled in only for diagnostic builds (nvcc -DSB_TRACE)
__device__ __forceinline__ void trace_block(const KParams &, int) {}
__device__ __forceinline__ void trace_event(const KParams &, int, int &, unsigned, unsigned) {}
#endif

constexpr int kSimtTile = 32;
constexpr int kTcTile = 128;

}  // namespace sb
