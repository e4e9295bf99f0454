// Host-side runtime of the kernel library: device status word, error strings, SM count,
// and the TMA tensor-map cache.
//
// Replaces the reference's error macros (csrc/operators/logging.h:53-121) with error
// codes + a message buffer (no exceptions cross the C boundary), and its per-call
// cuBLASLt handle / workspace creation (csrc/operators/gemm.cu:77-79,
// dhellam/common/common.py:7-13) with caches that are filled once.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

namespace dh {

static thread_local char g_err[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static constexpr int kMaxDev = 32;
static DeviceStatus* g_status_ptr[kMaxDev] = {nullptr};
static int g_sm_count[kMaxDev] = {0};
static std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static EncodeTiledFn get_encode() {
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
    set_last_error("cuTensorMapEncodeTiled entry point unavailable (%s)", cudaGetErrorString(e));
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}

struct TmapKey {
  uint64_t w[8];
  bool operator==(const TmapKey& o) const { return memcmp(w, o.w, sizeof(w)) == 0; }
};
struct TmapHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 8; ++i) {
      h ^= k.w[i];
      h *= 1099511628211ull;
    }
    return (size_t)h;
  }
};
// Tensor maps are immutable once encoded.  Entries are never evicted (callers keep the returned
// pointer until their launch, without a lock), so the cache is capped instead: a training job
// touches a few hundred distinct (pointer, shape) pairs; once kMaxCached maps exist, further
// ones are encoded into a small per-thread ring and stay valid for the next kRing calls of that
// thread, which is far more than one launch needs.
static std::unordered_map<TmapKey, CUtensorMap*, TmapHash> g_tmaps;
static constexpr size_t kMaxCached = 16384;
static constexpr int kRing = 64;

static const CUtensorMap* encode_cached(const TmapKey& key, CUtensorMapDataType dt, int rank, void* base,
                                        const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                                        bool swizzle128) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) return it->second;
  EncodeTiledFn enc = get_encode();
  if (!enc) return nullptr;
  const bool cache_full = g_tmaps.size() >= kMaxCached;
  static thread_local CUtensorMap ring[kRing];
  static thread_local int ring_pos = 0;
  CUtensorMap* m = cache_full ? &ring[ring_pos++ % kRing] : new CUtensorMap;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(m, dt, (cuuint32_t)rank, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed: code %d (base %p, dims %llu x %llu, stride %llu, box %u x %u)", (int)r,
                   base, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)strides[0], box[0],
                   box[1]);
    if (!cache_full) delete m;
    return nullptr;
  }
  if (!cache_full) g_tmaps.emplace(key, m);
  return m;
}

static CUtensorMapDataType dtype_of(int elem_bytes) {
  return elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
}

const CUtensorMap* get_tmap_2d(const void* base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                               uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0) {
    set_last_error("TMA operand must be 16-byte aligned with a 16-byte multiple row stride (base %p, stride %llu)", base,
                   (unsigned long long)row_stride_bytes);
    return nullptr;
  }
  TmapKey key = {{(uint64_t)(uintptr_t)base, inner, outer, row_stride_bytes, ((uint64_t)box_inner << 32) | box_outer,
                  (uint64_t)elem_bytes | ((uint64_t)swizzle128 << 8), 2, 0}};
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  return encode_cached(key, dtype_of(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, swizzle128);
}

const CUtensorMap* get_tmap_3d(const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                               bool swizzle128) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (stride1_bytes & 15) != 0 || (stride2_bytes & 15) != 0) {
    set_last_error("TMA operand must be 16-byte aligned with 16-byte multiple strides (base %p)", base);
    return nullptr;
  }
  TmapKey key = {{(uint64_t)(uintptr_t)base, d0 | (d1 << 32), d2, stride1_bytes, stride2_bytes,
                  ((uint64_t)b0 << 40) | ((uint64_t)b1 << 20) | b2, (uint64_t)elem_bytes | ((uint64_t)swizzle128 << 8), 3}};
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  return encode_cached(key, dtype_of(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, swizzle128);
}

const CUtensorMap* get_tmap_4d(const void* base, int elem_bytes, const uint64_t dims[4], const uint64_t strides_bytes[3],
                               const uint32_t box[4], bool swizzle128) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (strides_bytes[0] & 15) != 0 || (strides_bytes[1] & 15) != 0 ||
      (strides_bytes[2] & 15) != 0) {
    set_last_error("TMA operand must be 16-byte aligned with 16-byte multiple strides (base %p)", base);
    return nullptr;
  }
  TmapKey key = {{(uint64_t)(uintptr_t)base, dims[0] | (dims[1] << 32), dims[2] | (dims[3] << 32), strides_bytes[0],
                  strides_bytes[1], strides_bytes[2],
                  ((uint64_t)box[0] << 48) | ((uint64_t)box[1] << 32) | ((uint64_t)box[2] << 16) | box[3],
                  (uint64_t)elem_bytes | ((uint64_t)swizzle128 << 8) | (4ull << 16)}};
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t st[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  return encode_cached(key, dtype_of(elem_bytes), 4, const_cast<void*>(base), d, st, bx, swizzle128);
}

}  // namespace dh

extern "C" {

void* dh_status_device_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= dh::kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lock(dh::g_mu);
  if (dh::g_status_ptr[dev] == nullptr) {
    dh::DeviceStatus* p = nullptr;
    if (cudaMalloc(&p, sizeof(dh::DeviceStatus)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(dh::DeviceStatus));
    dh::g_status_ptr[dev] = p;
  }
  return dh::g_status_ptr[dev];
}

int dh_status_read(dh_status_t* out, int clear) {
  void* p = dh_status_device_ptr();
  if (!p) return (int)cudaErrorInvalidDevice;
  cudaError_t e = cudaMemcpy(out, p, sizeof(dh_status_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  if (clear && out->code != 0) e = cudaMemset(p, 0, sizeof(dh_status_t));
  return (int)e;
}

const char* dh_last_error_string() { return dh::g_err; }

int dh_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= dh::kMaxDev) return 0;
  if (dh::g_sm_count[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    dh::g_sm_count[dev] = n;
  }
  return dh::g_sm_count[dev];
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Bounded-wait self test: one thread waits (for at most `budget_cycles`) on a flag that the
// caller controls; used to check that a wait which cannot succeed returns an error status
// instead of hanging.
// ---------------------------------------------------------------------------
namespace dh {
__global__ void probe_flag_wait_kernel(const uint32_t* flag, uint32_t expect, long long budget, DeviceStatus* st) {
  if (threadIdx.x == 0 && blockIdx.x == 0) flag_wait_geq_gpu(flag, expect, budget, st, 900);
}
}  // namespace dh

extern "C" int dh_probe_flag_wait(const void* flag, uint32_t expect, long long budget_cycles, cudaStream_t s) {
  dh::probe_flag_wait_kernel<<<1, 32, 0, s>>>(reinterpret_cast<const uint32_t*>(flag), expect, budget_cycles,
                                              reinterpret_cast<dh::DeviceStatus*>(dh_status_device_ptr()));
  return (int)cudaGetLastError();
}

// Encodes a 4-D tensor map straight into caller-provided storage (no cache entry, no heap).
namespace dh {
bool encode_tmap_2d_into(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                         uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0) {
    set_last_error("TMA operand must be 16-byte aligned with a 16-byte multiple row stride (base %p, stride %llu)", base,
                   (unsigned long long)row_stride_bytes);
    return false;
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled (output) failed: code %d (base %p, dims %llu x %llu, stride %llu)", (int)r, base,
                   (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_stride_bytes);
    return false;
  }
  return true;
}
bool encode_tmap_4d_into(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims[4], const uint64_t strides_bytes[3],
                         const uint32_t box[4], bool swizzle128) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (strides_bytes[0] & 15) != 0 || (strides_bytes[1] & 15) != 0 ||
      (strides_bytes[2] & 15) != 0) {
    set_last_error("TMA operand must be 16-byte aligned with 16-byte multiple strides (base %p)", base);
    return false;
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t st[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 4, const_cast<void*>(base), d, st, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed: code %d", (int)r);
    return false;
  }
  return true;
}
}  // namespace dh
