// Host side of the tensor-core path: TMA tensor maps, which shapes take the path, the forward dispatch.
#include <cstring>

#ifndef SB_SHORT_SEQ
#define SB_SHORT_SEQ 1024
#endif

#include "sb_tc_common.cuh"

namespace sb {

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

// Encoded maps are pure functions of (base, dims, strides, box, type), and a training loop presents the same few
// tensors again and again (the caching allocator hands the same blocks back), so each thread keeps the maps it has
// encoded in a small direct-mapped table and skips the driver call on a hit.
struct MapKey {
  const void *ptr;
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box_rows;
  int dtype;
  bool operator==(const MapKey &o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kMapSlots = 128;

static cudaError_t encode_cached(CUtensorMap *map, const void *ptr, const cuuint64_t (&dims)[4], const cuuint64_t (&strides)[3],
                                 int box_rows, int dtype) {
  static thread_local MapSlot table[kMapSlots];
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.ptr = ptr;
  for (int i = 0; i < 4; ++i) key.dims[i] = dims[i];
  for (int i = 0; i < 3; ++i) key.strides[i] = strides[i];
  key.box_rows = (cuuint32_t)box_rows;
  key.dtype = dtype;
  uint64_t h = (uint64_t)(uintptr_t)ptr * 0x9E3779B97F4A7C15ull;
  h ^= (dims[1] + 0x1000193u * box_rows + 31u * strides[0] + 17u * strides[1]) * 0xC2B2AE3D27D4EB4Full;
  MapSlot &slot = table[(h >> 32) % kMapSlots];
  if (slot.used && slot.key == key) {
    *map = slot.map;
    return cudaSuccess;
  }
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return cudaErrorNotSupported;
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dtype == SB_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  slot.key = key;
  slot.map = *map;
  slot.used = true;
  return cudaSuccess;
}

cudaError_t make_tile_map(CUtensorMap *map, const TensorRef &t, const KParams &p, int dtype, int box_rows) {
  const cuuint64_t esz = 2;
  long long sb_el = t.sb > 0 ? t.sb : (t.sh > 0 ? t.sh * p.heads : (long long)p.tokens * p.head_dim);
  long long sh_el = t.sh > 0 ? t.sh : (long long)p.tokens * p.head_dim;
  cuuint64_t dims[4] = {(cuuint64_t)p.head_dim, (cuuint64_t)p.tokens, (cuuint64_t)p.heads, (cuuint64_t)p.batch};
  cuuint64_t strides[3] = {(cuuint64_t)t.st * esz, (cuuint64_t)sh_el * esz, (cuuint64_t)sb_el * esz};
  return encode_cached(map, t.ptr, dims, strides, box_rows, dtype);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is needed once per kernel and device, not once per launch.
cudaError_t allow_dynamic_smem(const void *kernel, int bytes) {
  struct Done { const void *kernel; int dev; };
  static thread_local Done done[64];
  static thread_local int n_done = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  for (int i = 0; i < n_done; ++i)
    if (done[i].kernel == kernel && done[i].dev == dev) return cudaSuccess;
  if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)) != cudaSuccess) return e;
  if (n_done < 64) done[n_done++] = Done{kernel, dev};
  return cudaSuccess;
}

cudaError_t make_az_map(CUtensorMap *map, const KParams &p, int dtype, int box_rows) {
  const cuuint64_t tile_bytes = (cuuint64_t)kBM * kBM * 2;
  cuuint64_t dims[4] = {(cuuint64_t)kBM, (cuuint64_t)p.pairs_cap * kBM, 2, (cuuint64_t)p.head_cnt};
  cuuint64_t strides[3] = {(cuuint64_t)kBM * 2, (cuuint64_t)p.pairs_cap * tile_bytes, 2 * (cuuint64_t)p.pairs_cap * tile_bytes};
  return encode_cached(map, p.az, dims, strides, box_rows, dtype);
}

// The forward works on 256 query rows per item (two 128-row tiles sharing the K/V stream), except for head sizes up
// to 64 with sequences of at most kShortSeq tokens (the caller's max_seqlen bound), where two independent 128-row
// tiles per block do better (sb_tc_fwd128.cu).
constexpr int kShortSeq = SB_SHORT_SEQ;
int tc_tile(int head_dim, bool backward, int max_seqlen) {
  if (backward) return kBM;
  return (head_dim <= 64 && max_seqlen <= kShortSeq) ? kBM : 256;
}

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

cudaError_t launch_tc_fwd(const KParams &p, int dtype, cudaStream_t s, int *launches) {
  *launches += 1;
  return p.tile == kBM ? launch_tc_fwd128(p, dtype, s) : launch_tc_fwd256(p, dtype, s);
}

}  // namespace sb
