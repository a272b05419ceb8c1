// C ABI of the library: argument checks, workspace layout, kernel selection, launches.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "sb_common.cuh"

namespace sb {

static thread_local char g_err[512] = "";
static thread_local int g_launches = 0;

static int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Workspace layout, a pure function of the shapes:
//   [hdr 256 B][tile_prefix int32 x (num_seq+1)][pair_prefix int64 x (num_seq+1)]
//   packed batches: [order int2 x tiles][order2 (backward) int2 x tiles]
//   backward, either: [A | dz tiles, 16-bit x chunk_heads x pairs_cap x 2 x 128 x 128]   (stored-tiles mode)
//             or:     [R1 fp32 x chunk_heads x pairs_cap x halves x tile][S2 same]       (recompute mode)
//   backward with SB_FLAG_FUSE_REM_V: [d_rem + <d_out, v>, one value of the tensors' dtype in a 4-byte slot budget x batch x heads x tokens]
struct Plan {
  int path;
  int tile;
  int tiles_cap;
  int n_max;
  int max_seqlen;
  long long pairs_cap;
  size_t off_tile_prefix, off_pair_prefix, off_order, off_order2, off_bnd, off_drem;
  int bnd_halves;             // boundary records per (query tile, key tile) pair
  size_t bnd_bytes_per_head;  // one of the two arrays
  int chunk_heads;
  bool store_az;              // backward: the dq kernel stores its A and dz tiles for the dK/dV kernel
  size_t az_bytes_per_head;
  size_t total_fwd, total_bwd;
};

// Upper bound on the backward's per-chunk scratch (stored tiles, or R1 + S2): heads are processed in chunks that fit
// it, and a call whose single head does not fit the stored tiles takes the recomputing dK/dV kernel.  Process-wide,
// set through sb_set_backward_scratch_budget.
static std::atomic<size_t> g_scratch_budget{(size_t)8 << 30};

static int check_tensor(const SbTensor &t, const char *name, bool required) {
  if (t.ptr == nullptr) return required ? fail(SB_ERR_ARGUMENT, "%s.ptr is NULL", name) : SB_OK;
  if (t.stride_t < 0 || t.stride_h < 0 || t.stride_b < 0) return fail(SB_ERR_ARGUMENT, "%s has a negative stride", name);
  return SB_OK;
}

static bool tma_friendly(const SbTensor &t, int esize) {
  if (reinterpret_cast<uintptr_t>(t.ptr) % 16) return false;
  const long long m = 16 / esize;
  return t.stride_t % m == 0 && t.stride_h % m == 0 && t.stride_b % m == 0 && t.stride_t > 0;
}

static int make_plan(const SbParams *p, Plan &pl, bool backward) {
  if (p == nullptr) return fail(SB_ERR_ARGUMENT, "params is NULL");
  if (p->struct_bytes != (int)sizeof(SbParams))
    return fail(SB_ERR_ARGUMENT, "struct_bytes %d != sizeof(SbParams) %d", p->struct_bytes, (int)sizeof(SbParams));
  if (p->dtype < SB_DTYPE_F32 || p->dtype > SB_DTYPE_F16) return fail(SB_ERR_ARGUMENT, "unknown dtype %d", p->dtype);
  if (p->batch < 1 || p->batch > 65535 || p->heads < 1 || p->heads > 65535)
    return fail(SB_ERR_ARGUMENT, "batch/heads out of range (1..65535)");
  if (p->head_dim < 1 || p->head_dim > 256) return fail(SB_ERR_ARGUMENT, "head_dim %d outside 1..256", p->head_dim);
  if (p->tokens < 0 || p->tokens > 0x7fffff00LL) return fail(SB_ERR_ARGUMENT, "tokens out of range");
  if (p->cu_seqlens != nullptr) {
    if (p->batch != 1) return fail(SB_ERR_ARGUMENT, "a packed batch (cu_seqlens given) needs batch == 1");
    if (p->num_seq < 1) return fail(SB_ERR_ARGUMENT, "num_seq must be >= 1 with cu_seqlens");
  } else if (p->num_seq != 0) {
    return fail(SB_ERR_ARGUMENT, "num_seq must be 0 without cu_seqlens");
  }
  if (p->max_seqlen < 0) return fail(SB_ERR_ARGUMENT, "max_seqlen is negative");

  const int esize = p->dtype == SB_DTYPE_F32 ? 4 : 2;
  bool tc = !(p->flags & SB_FLAG_FORCE_SIMT) && !(p->attn_weights != nullptr && !backward) &&
            tc_supported(p->dtype, p->head_dim, backward) &&
            tma_friendly(p->q, esize) && tma_friendly(p->k, esize) && tma_friendly(p->v, esize);
  // outputs and gradients are stored with 16-byte vectors on the tensor-core path
  const SbTensor *others[] = {&p->o, &p->d_o, &p->dq, &p->dk, &p->dv};
  for (const SbTensor *t : others)
    if (t->ptr != nullptr && !tma_friendly(*t, esize)) tc = false;
  pl.path = tc ? SB_PATH_TCGEN05 : SB_PATH_SIMT;
  const long long T = p->tokens;
  pl.max_seqlen = (p->max_seqlen == 0 || p->max_seqlen > T) ? (int)T : p->max_seqlen;
  if (p->cu_seqlens == nullptr) pl.max_seqlen = (int)T;
  pl.tile = tc ? tc_tile(p->head_dim, backward, pl.max_seqlen) : kSimtTile;
  const long long n_all = (T + pl.tile - 1) / pl.tile;
  pl.n_max = (int)((pl.max_seqlen + pl.tile - 1) / pl.tile);
  if (p->cu_seqlens == nullptr) {
    pl.tiles_cap = (int)(n_all * p->batch);
    pl.pairs_cap = (long long)p->batch * (n_all * (n_all + 1) / 2);
  } else {
    pl.tiles_cap = (int)(n_all + p->num_seq);
    pl.pairs_cap = ((long long)pl.tiles_cap * (pl.n_max + 1) + 1) / 2;
  }
  if (pl.tiles_cap < 1) pl.tiles_cap = 1;
  pl.off_tile_prefix = 256;
  pl.off_pair_prefix = align_up(pl.off_tile_prefix + sizeof(int) * (size_t)(p->num_seq + 1), 256);
  pl.off_order = align_up(pl.off_pair_prefix + sizeof(long long) * (size_t)(p->num_seq + 1), 256);
  const size_t order_bytes = p->cu_seqlens != nullptr ? align_up(sizeof(int2) * (size_t)pl.tiles_cap, 256) : 0;
  pl.off_order2 = pl.off_order + order_bytes;                       // every second tile: the backward's dq kernel
  pl.off_bnd = pl.off_order2 + ((backward && tc) ? order_bytes : 0);
  // the tensor-core path records the carried values four times per 128-key tile
  pl.bnd_halves = tc ? 4 : 1;   // keys 0, 32, 64, 96 of every 128-key tile
  pl.bnd_bytes_per_head = align_up((size_t)pl.pairs_cap * pl.tile * pl.bnd_halves * sizeof(float), 256);
  // Stored-tiles mode (128-column head sizes): 64 KiB per (query tile, key tile) pair and head.  Taken when at least one
  // head fits the budget and the caller did not ask for the small-workspace mode.
  const size_t budget = g_scratch_budget.load(std::memory_order_relaxed);
  pl.az_bytes_per_head = (size_t)pl.pairs_cap * 2 * kTcTile * kTcTile * 2;
  pl.store_az = backward && tc && !(p->flags & SB_FLAG_BWD_RECOMPUTE) && pl.az_bytes_per_head <= budget;
  const size_t per_head = pl.store_az ? pl.az_bytes_per_head : 2 * pl.bnd_bytes_per_head;
  size_t chunk = per_head ? budget / per_head : (size_t)p->heads;
  if (chunk < 1) chunk = 1;
  if (chunk > (size_t)p->heads) chunk = p->heads;
  pl.chunk_heads = (int)chunk;
#ifdef SB_TRACE   // diagnostic builds: reserved & 0x100 appends the event log to the workspace
  const size_t trace_bytes = (p->reserved & 0x100) ? kTraceBytes : 0;
#else
  if (p->reserved != 0) return fail(SB_ERR_ARGUMENT, "reserved must be 0");
  const size_t trace_bytes = 0;
#endif
  pl.total_fwd = pl.off_bnd + trace_bytes;
  pl.off_drem = align_up(pl.off_bnd + per_head * chunk, 256);
  const size_t drem_bytes =
      (p->flags & SB_FLAG_FUSE_REM_V) ? align_up(sizeof(float) * (size_t)p->batch * p->heads * (size_t)T, 256) : 0;
  pl.total_bwd = pl.off_drem + drem_bytes + trace_bytes;
  return SB_OK;
}

static TensorRef ref_of(const SbTensor &t) {
  return TensorRef{reinterpret_cast<char *>(t.ptr), (long long)t.stride_b, (long long)t.stride_h, (long long)t.stride_t};
}

static int device_ok() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(SB_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  static int cached_major[64];
  if (dev < 0 || dev >= 64) return fail(SB_ERR_CUDA, "device ordinal %d not supported", dev);
  if (cached_major[dev] == 0) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail(SB_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    cached_major[dev] = major;
  }
  if (cached_major[dev] != 10)
    return fail(SB_ERR_NO_DEVICE_CODE, "device %d has compute capability %d.x; this library holds sm_100a code only",
                dev, cached_major[dev]);
  return SB_OK;
}

static int fill_kparams(const SbParams *p, const Plan &pl, bool backward, KParams &k) {
  memset(&k, 0, sizeof(k));
  int rc;
  if ((rc = check_tensor(p->q, "q", true)) || (rc = check_tensor(p->k, "k", true)) || (rc = check_tensor(p->v, "v", true)))
    return rc;
  if (p->log_rem == nullptr) return fail(SB_ERR_ARGUMENT, "log_rem is NULL");
  if (!backward) {
    if ((rc = check_tensor(p->o, "o", true))) return rc;
    if (p->rem == nullptr) return fail(SB_ERR_ARGUMENT, "rem is NULL");
  } else {
    if ((rc = check_tensor(p->d_o, "d_o", true)) || (rc = check_tensor(p->dq, "dq", true)) ||
        (rc = check_tensor(p->dk, "dk", true)) || (rc = check_tensor(p->dv, "dv", true)))
      return rc;
    if (p->d_rem == nullptr && !(p->flags & SB_FLAG_FUSE_REM_V)) return fail(SB_ERR_ARGUMENT, "d_rem is NULL");
  }
  const size_t need = backward ? pl.total_bwd : pl.total_fwd;
  if (p->workspace == nullptr || p->workspace_bytes < need)
    return fail(SB_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", p->workspace_bytes, need);
  if (reinterpret_cast<uintptr_t>(p->workspace) % 256) return fail(SB_ERR_WORKSPACE, "workspace is not 256-byte aligned");

  k.q = ref_of(p->q); k.k = ref_of(p->k); k.v = ref_of(p->v); k.o = ref_of(p->o);
  k.d_o = ref_of(p->d_o); k.dq = ref_of(p->dq); k.dk = ref_of(p->dk); k.dv = ref_of(p->dv);
  k.rem = reinterpret_cast<char *>(p->rem);
  k.d_rem = reinterpret_cast<const char *>(p->d_rem);
  k.log_rem = p->log_rem;
  k.cu = p->cu_seqlens;
  k.cu64 = p->cu_seqlens_int64;
  k.batch = p->batch; k.heads = p->heads; k.head_dim = p->head_dim; k.num_seq = p->num_seq;
  k.tokens = p->tokens;
  char *ws_end = reinterpret_cast<char *>(p->workspace) + (backward ? pl.total_bwd : pl.total_fwd);
  k.attend_current = p->attend_current ? 1 : 0;
  k.scale = p->logit_scale;
  k.check_leading_zero = (p->cu_seqlens != nullptr && (p->flags & SB_FLAG_CHECK_LEADING_ZERO)) ? 1 : 0;
  // Tiles of one sequence that stay neighbours in the launch order.  The backward kernels gain more from sharing
  // K/V or Q/dO reads through L2 (measured: -4 % at 2048-token, -8 % at 4096-token sequences) than they lose in the
  // tail; the forward's blocks are persistent with a fixed item assignment, which wants the pure weight order (keeping the
  // tiles of a short sequence adjacent was measured too: +4 % time on 1024 x 128..512-token sequences).
  k.order_span = backward ? 16 : 1;
#ifdef SB_TRACE
  k.dbg = p->reserved & 0xff;
  k.trace_mode = (p->reserved >> 8) & 3;
  k.trace = (p->reserved & 0x100) ? reinterpret_cast<unsigned long long *>(ws_end - kTraceBytes) : nullptr;
#else
  (void)ws_end;
#endif
  k.skip_dq = (p->flags & SB_FLAG_BWD_SKIP_DQ) ? 1 : 0;
  k.skip_dkv = (p->flags & SB_FLAG_BWD_SKIP_DKV) ? 1 : 0;
  k.dense = (p->flags & SB_FLAG_DENSE_ROW_PASS) ? 1 : 0;
  k.tile = pl.tile; k.tiles_cap = pl.tiles_cap; k.n_max = pl.n_max; k.max_seqlen = pl.max_seqlen;
  char *ws = reinterpret_cast<char *>(p->workspace);
  k.hdr = reinterpret_cast<int *>(ws);
  k.tile_prefix = reinterpret_cast<int *>(ws + pl.off_tile_prefix);
  k.pair_prefix = reinterpret_cast<long long *>(ws + pl.off_pair_prefix);
  if (p->cu_seqlens != nullptr) {
    k.order = reinterpret_cast<const int2 *>(ws + pl.off_order);
    if (pl.off_bnd != pl.off_order2) k.order2 = reinterpret_cast<const int2 *>(ws + pl.off_order2);
  }
  if (backward && pl.store_az) {
    k.az = reinterpret_cast<unsigned short *>(ws + pl.off_bnd);
  } else {
    k.bnd_r1 = reinterpret_cast<float *>(ws + pl.off_bnd);
    k.bnd_s2 = reinterpret_cast<float *>(ws + pl.off_bnd + pl.bnd_bytes_per_head * pl.chunk_heads);
  }
  k.pairs_cap = pl.pairs_cap;
  k.fuse_rem_v = (p->flags & SB_FLAG_FUSE_REM_V) ? 1 : 0;
  if (!backward && p->attn_weights != nullptr) {
    if (p->attn_cols < 1) return fail(SB_ERR_ARGUMENT, "attn_cols must be >= 1 with attn_weights");
    k.attn = p->attn_weights;
    k.attn_cols = p->attn_cols;
  }
  if (backward && k.fuse_rem_v) k.d_rem_fused = ws + pl.off_drem;
  k.status = p->status;
  return SB_OK;
}

static int run(const SbParams *p, void *stream, bool backward) {
  g_err[0] = 0;
  g_launches = 0;
  Plan pl;
  int rc = make_plan(p, pl, backward);
  if (rc) return rc;
  if ((rc = device_ok())) return rc;
  KParams k;
  if ((rc = fill_kparams(p, pl, backward, k))) return rc;
  if (p->tokens == 0) return SB_OK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = launch_prep(k, s);
  g_launches += (p->cu_seqlens != nullptr && k.trace != nullptr) ? 2 : 1;   // prep kernel or header clear (both with the event log)
  if (e != cudaSuccess) return fail(SB_ERR_CUDA, "prep launch: %s", cudaGetErrorString(e));
  if (backward && k.fuse_rem_v) {
    e = launch_fused_drem(k, p->dtype, s);
    g_launches += 1;
    if (e != cudaSuccess) return fail(SB_ERR_CUDA, "d_rem launch: %s", cudaGetErrorString(e));
    k.d_rem = k.d_rem_fused;   // what the backward kernels read from here on
  }
  const int chunk = backward ? pl.chunk_heads : p->heads;
  for (int h0 = 0; h0 < p->heads; h0 += chunk) {
    k.head0 = h0;
    k.head_cnt = (p->heads - h0 < chunk) ? p->heads - h0 : chunk;
    if (pl.path == SB_PATH_TCGEN05)
      e = backward ? launch_tc_bwd(k, p->dtype, s, &g_launches) : launch_tc_fwd(k, p->dtype, s, &g_launches);
    else
      e = backward ? launch_simt_bwd(k, p->dtype, s, &g_launches) : launch_simt_fwd(k, p->dtype, s, &g_launches);
    if (e != cudaSuccess) return fail(SB_ERR_CUDA, "%s launch: %s", backward ? "backward" : "forward", cudaGetErrorString(e));
    if (p->cu_seqlens != nullptr) {
      e = launch_zero_tail(k, p->dtype, backward, s);
      g_launches += 1;
      if (e != cudaSuccess) return fail(SB_ERR_CUDA, "tail launch: %s", cudaGetErrorString(e));
    }
  }
  // the stored-tiles dK/dV kernel adds rem * d_out in its own epilogue; the other kernels leave it to one more pass
  if (backward && k.fuse_rem_v && !k.skip_dkv && !(pl.path == SB_PATH_TCGEN05 && pl.store_az)) {
    e = launch_fused_dv(k, p->dtype, s);
    g_launches += 1;
    if (e != cudaSuccess) return fail(SB_ERR_CUDA, "dv launch: %s", cudaGetErrorString(e));
  }
  return SB_OK;
}

// ---- built-in scratch for callers that cannot allocate ---------------------------------------------
// One array per device that loads the library, resident until the process exits.  Host code may not use
// the symbol as an address: the device address is looked up once per device and cached.
static __device__ __align__(256) unsigned char g_static_scratch[SB_STATIC_SCRATCH_BYTES];
static std::mutex g_static_scratch_mu;
static void *g_static_scratch_ptr[64];

static int static_scratch_address(void **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(SB_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(SB_ERR_CUDA, "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> guard(g_static_scratch_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);   // resolves for the current device
    if (e != cudaSuccess || ptr == nullptr)
      return fail(SB_ERR_CUDA, "cudaGetSymbolAddress(built-in scratch): %s", cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return SB_OK;
}

static int run_fwd_static_scratch(const SbParams *p, void *stream) {
  g_err[0] = 0;
  g_launches = 0;
  Plan pl;
  int rc = make_plan(p, pl, false);
  if (rc) return rc;
  if (pl.total_fwd > (size_t)SB_STATIC_SCRATCH_BYTES)
    return fail(SB_ERR_WORKSPACE,
                "sb_fwd_static_scratch: this call needs %zu bytes of scratch but the built-in scratch holds %d "
                "(sb_workspace_bytes(p, 0) is the measure); use sb_fwd with a caller-provided workspace",
                pl.total_fwd, (int)SB_STATIC_SCRATCH_BYTES);
  if ((rc = device_ok())) return rc;
  void *scratch = nullptr;
  if ((rc = static_scratch_address(&scratch))) return rc;
  SbParams with_scratch = *p;
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = SB_STATIC_SCRATCH_BYTES;
  return run(&with_scratch, stream, false);
}

}  // namespace sb

extern "C" {

size_t sb_workspace_bytes(const SbParams *p, int backward) {
  sb::Plan pl;
  if (sb::make_plan(p, pl, backward != 0)) return (size_t)-1;
  return backward ? pl.total_bwd : pl.total_fwd;
}

int sb_fwd(const SbParams *p, void *stream) { return sb::run(p, stream, false); }

int sb_bwd(const SbParams *p, void *stream) { return sb::run(p, stream, true); }

int sb_kernel_path(const SbParams *p) {
  sb::Plan pl;
  if (sb::make_plan(p, pl, false)) return -1;
  return pl.path;
}

int sb_last_launch_count(void) { return sb::g_launches; }

const char *sb_last_error(void) { return sb::g_err; }

int sb_fwd_static_scratch(const SbParams *p, void *stream) { return sb::run_fwd_static_scratch(p, stream); }

size_t sb_set_backward_scratch_budget(size_t bytes) {
  if (bytes == 0) return sb::g_scratch_budget.load(std::memory_order_relaxed);
  return sb::g_scratch_budget.exchange(bytes, std::memory_order_relaxed);
}

int sb_abi_version(void) { return SB_ABI_VERSION; }

}  // extern "C"
