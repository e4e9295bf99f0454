// Host-side cache of TMA tensor maps (cuTensorMapEncodeTiled obtained through the
// runtime's driver entry point, so the library does not link libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dh {

// 2-D bf16/fp32 tensor: `inner` contiguous elements per row, `outer` rows,
// `row_stride_bytes` between rows; box = box_inner x box_outer; 128-byte swizzle when
// box_inner * elem_bytes == 128, none otherwise.
// Returns nullptr on failure (dh_last_error_string() has the reason).
const CUtensorMap* get_tmap_2d(const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                               uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128);

// 3-D variant (inner, mid, outer) with strides for mid and outer in bytes.
const CUtensorMap* get_tmap_3d(const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                               uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                               bool swizzle128);

// 4-D variant: dims/box innermost first, strides (bytes) for dimensions 1..3.
const CUtensorMap* get_tmap_4d(const void* base, int elem_bytes, const uint64_t dims[4], const uint64_t strides_bytes[3],
                               const uint32_t box[4], bool swizzle128);

// Encodes a 2-D map into caller-provided storage without touching the cache: for output tensors,
// whose addresses change from call to call.  Returns false on failure.
bool encode_tmap_2d_into(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                         uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128);

void set_last_error(const char* fmt, ...);

// cudaFuncSetAttribute applies to the function on the CURRENT device only, so "already
// configured" has to be remembered per device: a process that drives a second GPU would
// otherwise launch there without the shared-memory opt-in and fail.  A zero-initialised static
// of this type plus device_flag() replaces the usual `static bool configured`.
struct PerDeviceFlags {
  bool done[64];
};
inline bool& device_flag(PerDeviceFlags& f) {
  int dev = 0;
  cudaGetDevice(&dev);
  return f.done[dev & 63];
}

}  // namespace dh

inline void set_last_error_c(const char* what, const char* msg) { dh::set_last_error("%s: %s", what, msg); }
