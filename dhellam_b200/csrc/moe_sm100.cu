// Mixture-of-experts token exchange without the host in the loop.
//
// The reference advertises expert parallelism (README.md:8) but ships no router, dispatch or
// expert GEMM; the only trace is an all_to_all_single entry in its micro-benchmark
// (micro_benchmark/overlap.py:141-145).  These kernels are therefore new.  Together with the
// grouped form of the CTA-pair GEMM (gemm_sm100.cu, group_mode) they replace a host-driven
// pipeline (sort, bincount, two .tolist() reads per layer, variable-size all_to_all_single, a Python
// loop of per-expert GEMMs) by device-resident steps whose sizes never reach the host:
//
//   moe_plan      one CTA per expert scans the [tokens x k] routing table and gives every copy its
//                 stable position among the copies of its expert; per-expert counts
//   moe_offsets   from the count matrix of all source ranks: where each (source, expert) group lands
//                 on the expert's owner.  Every expert's region is padded to 256 rows (the tile
//                 height of the grouped GEMM) so tiles never straddle two experts
//   moe_dispatch  one warp per copy: stores the token row (optionally scaled, optionally with a dot
//                 product on the side for the gate gradient) into the OWNER rank's expert-major
//                 buffer over NVLink peer memory; the last CTA raises an arrival counter on every rank
//   moe_zero_pad  the owner clears the padding rows of its buffer (nothing else writes them)
//   moe_combine   one warp per token: PULLS the k expert outputs of the token from their owners
//                 (plain peer loads), writes the weighted sum and, for the backward, the copies
//
// Every wait is bounded and reports through the status word.  No load is a multi-CTA broadcast.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"
#include "comm_device.cuh"
#include "ptx.cuh"
#include "tmap.h"

namespace dh {
namespace moe {

constexpr int PAD = 256;          // expert regions are multiples of the grouped GEMM's tile height
constexpr int MAX_EXPERTS = 256;
constexpr int MAX_RANKS = 8;

// ------------------------------------------------------------------------------------------ plan
// grid = E, block = 256.  pos[i] = number of earlier copies (i' < i) routed to the same expert.
__global__ void __launch_bounds__(256) moe_plan_kernel(const int* __restrict__ topi, int n, int* __restrict__ pos, int* __restrict__ counts) {
  __shared__ int warp_sums[8];
  __shared__ int base_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  for (int i0 = 0; i0 < n; i0 += 256) {
    const int i = i0 + threadIdx.x;
    const int hit = (i < n && topi[i] == e) ? 1 : 0;
    // inclusive scan inside the warp
    int v = hit;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    int before = base_s;
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
    if (hit) pos[i] = before + v - 1;
    __syncthreads();
    if (threadIdx.x == 255) base_s = before + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = base_s;
}

// ------------------------------------------------------------------------------------------ offsets
// cnt_all [ep][E]: copies that source rank s routes to expert e.  One CTA.
//   dst_base[e]        row on the owner of e where THIS rank's copies for e start
//   offs[el + 1]       padded region starts of this rank's local experts (multiples of 256); offs[el] = rows in use
//   rows_e[el]         real rows per local expert
// `capacity` is the row capacity of the landing buffers: a plan that does not fit is reported (code 3)
// and every region is clamped to empty so that nothing is written out of bounds.
__global__ void __launch_bounds__(256) moe_offsets_kernel(const int* __restrict__ cnt_all, int ep, int E, int me, int capacity,
                                                          int* __restrict__ dst_base, int* __restrict__ offs, int* __restrict__ rows_e,
                                                          int* __restrict__ overflow, DeviceStatus* st) {
  __shared__ int tot[MAX_EXPERTS];
  __shared__ int before_me[MAX_EXPERTS];
  __shared__ int region[MAX_EXPERTS];
  __shared__ int bad;
  const int el = E / ep;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < ep; ++s) {
      const int c = cnt_all[s * E + e];
      if (s < me) b += c;
      t += c;
    }
    tot[e] = t;
    before_me[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < ep) {                       // one thread per owner rank: padded prefix over its experts
    const int d = threadIdx.x;
    int acc = 0;
    for (int le = 0; le < el; ++le) {
      region[d * el + le] = acc;
      acc += (tot[d * el + le] + PAD - 1) / PAD * PAD;
    }
    if (acc > capacity) atomicExch(&bad, 1);
    if (d == me) offs[el] = acc;
  }
  __syncthreads();
  if (bad) {
    if (threadIdx.x == 0) { *overflow = 1; report_error(st, ERR_BOUNDS, 810, capacity); }
    for (int e = threadIdx.x; e < E; e += blockDim.x) dst_base[e] = -1;        // dispatch skips every copy
    for (int le = threadIdx.x; le <= el; le += blockDim.x) { offs[le] = 0; if (le < el) rows_e[le] = 0; }
    return;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) dst_base[e] = region[e] + before_me[e];
  for (int le = threadIdx.x; le < el; le += blockDim.x) {
    offs[le] = region[me * el + le];
    rows_e[le] = tot[me * el + le];
  }
}

// ------------------------------------------------------------------------------------------ zero padding rows
// grid = (blocks, el).  Clears rows [offs[e] + rows_e[e], offs[e+1]) of buf (row width h elements).
__global__ void __launch_bounds__(256) moe_zero_pad_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ offs,
                                                           const int* __restrict__ rows_e, int h) {
  const int e = blockIdx.y;
  const long long r0 = (long long)offs[e] + rows_e[e], r1 = offs[e + 1];
  const long long nvec = (r1 - r0) * (h >> 3);
  uint4* p = reinterpret_cast<uint4*>(buf + r0 * h);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x)
    p[i] = make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------------------------------ dispatch (push)
struct DispatchParams {
  const __nv_bfloat16* src;        // [T, h] rows, row stride ld_src
  long long ld_src;
  const int* topi;                 // [T * k] expert of every copy
  const int* pos;                  // [T * k] position among the copies of its expert
  const int* dst_base;             // [E]
  const float* scale;              // [T * k] multiplier of every copy, or null
  const __nv_bfloat16* other;      // [T * k, h] rows to take a dot product with (gate gradient), or null
  float* dots;                     // [T * k] <src row, other row>
  __nv_bfloat16* dst[MAX_RANKS];   // landing buffers of every expert-parallel rank (dst[me] is local)
  int* dest_rank;                  // [T * k] (out, may be null) owner rank of every copy
  int* dest_row;                   // [T * k] (out, may be null) row on the owner
  uint32_t* arrived[MAX_RANKS];    // arrival counter on every rank (+1 per source and call)
  unsigned int* done_ctas;         // local scratch counter (zero before the call, reset by the last CTA)
  int n, k, h, el, ep;
};

__global__ void __launch_bounds__(256) moe_dispatch_kernel(const DispatchParams p) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  const int vecs = p.h >> 3;
  for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < p.n; i += warps_total) {
    const int e = p.topi[i];
    const int base = p.dst_base[e];
    const int d = e / p.el;
    const int row = base + p.pos[i];
    if (lane == 0) {
      if (p.dest_rank != nullptr) p.dest_rank[i] = d;
      if (p.dest_row != nullptr) p.dest_row[i] = base < 0 ? -1 : row;
    }
    if (base < 0) continue;                        // the plan did not fit: nothing is written
    const int t = i / p.k;
    const uint4* s = reinterpret_cast<const uint4*>(p.src + (long long)t * p.ld_src);
    uint4* dst = reinterpret_cast<uint4*>(p.dst[d] + (long long)row * p.h);
    const float mul = p.scale != nullptr ? p.scale[i] : 1.f;
    const uint4* oth = p.other != nullptr ? reinterpret_cast<const uint4*>(p.other + (long long)i * p.h) : nullptr;
    float dot = 0.f;
    for (int v = lane; v < vecs; v += 32) {
      uint4 x = s[v];
      if (oth != nullptr) {
        const uint4 y = oth[v];
        const float2 a0 = unpack_bf16x2(x.x), a1 = unpack_bf16x2(x.y), a2 = unpack_bf16x2(x.z), a3 = unpack_bf16x2(x.w);
        const float2 b0 = unpack_bf16x2(y.x), b1 = unpack_bf16x2(y.y), b2 = unpack_bf16x2(y.z), b3 = unpack_bf16x2(y.w);
        dot += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
      }
      if (p.scale != nullptr) {
        const float2 a0 = unpack_bf16x2(x.x), a1 = unpack_bf16x2(x.y), a2 = unpack_bf16x2(x.z), a3 = unpack_bf16x2(x.w);
        x.x = pack_bf16x2(a0.x * mul, a0.y * mul); x.y = pack_bf16x2(a1.x * mul, a1.y * mul);
        x.z = pack_bf16x2(a2.x * mul, a2.y * mul); x.w = pack_bf16x2(a3.x * mul, a3.y * mul);
      }
      dst[v] = x;
    }
    if (oth != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == 0) p.dots[i] = dot;
    }
  }
  // the last CTA to finish tells every rank that this source's rows are in place
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(p.done_ctas, 1u) + 1u;
    if (done == gridDim.x) {
      *p.done_ctas = 0u;
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int d = 0; d < p.ep; ++d) red_add_relaxed_sys(p.arrived[d], 1u);      // released by the fence above
    }
  }
}

// ------------------------------------------------------------------------------------------ combine (pull)
struct CombineParams {
  const __nv_bfloat16* src[MAX_RANKS];   // expert-output buffers of every rank
  const int* dest_rank;                  // [T * k]
  const int* dest_row;                   // [T * k]
  const float* gates;                    // [T * k] weights, or null (plain sum: dispatch backward)
  __nv_bfloat16* out;                    // [T, h]
  __nv_bfloat16* copies;                 // [T * k, h] the pulled rows (kept for the backward), or null
  const uint32_t* ready;                 // local counter: every owner adds 1 when its outputs are complete
  uint32_t target;
  int T, k, h;
  DeviceStatus* status;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const CombineParams p) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = comm::wait_counter_sys(p.ready, p.target, nullptr, p.status, 820) ? 1 : 0;
  __syncthreads();
  if (!ok_s) return;
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  const int vecs = p.h >> 3;
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < p.T; t += warps_total) {
    for (int v = lane; v < vecs; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < p.k; ++j) {
        const int i = t * p.k + j;
        const int row = p.dest_row[i];
        if (row < 0) continue;
        const uint4 x = comm::ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(p.src[p.dest_rank[i]] + (long long)row * p.h) + v);
        if (p.copies != nullptr) reinterpret_cast<uint4*>(p.copies + (long long)i * p.h)[v] = x;
        const float g = p.gates != nullptr ? p.gates[i] : 1.f;
        const float2 a0 = unpack_bf16x2(x.x), a1 = unpack_bf16x2(x.y), a2 = unpack_bf16x2(x.z), a3 = unpack_bf16x2(x.w);
        acc[0] += g * a0.x; acc[1] += g * a0.y; acc[2] += g * a1.x; acc[3] += g * a1.y;
        acc[4] += g * a2.x; acc[5] += g * a2.y; acc[6] += g * a3.x; acc[7] += g * a3.y;
      }
      reinterpret_cast<uint4*>(p.out + (long long)t * p.h)[v] =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
}

}  // namespace moe
}  // namespace dh

using namespace dh;
using namespace dh::moe;

static int moe_rc(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("%s launch failed: %s", what, cudaGetErrorString(e));
  return (int)e;
}

extern "C" {

// topi [n] int32 (n = tokens x k), E experts -> pos [n], counts [E].
int dh_moe_plan(const void* topi, int n, int E, void* pos, void* counts, cudaStream_t s) {
  if (E < 1 || E > MAX_EXPERTS) { set_last_error("dh_moe_plan: %d experts not in [1, %d]", E, MAX_EXPERTS); return (int)cudaErrorInvalidValue; }
  moe_plan_kernel<<<E, 256, 0, s>>>((const int*)topi, n, (int*)pos, (int*)counts);
  return moe_rc("dh_moe_plan");
}

// cnt_all [ep][E] int32 -> dst_base [E], offs [E/ep + 1], rows_e [E/ep], overflow [1] (set to 1 if the plan needs more than
// `capacity` rows on some rank).
int dh_moe_offsets(const void* cnt_all, int ep, int E, int me, int capacity, void* dst_base, void* offs, void* rows_e, void* overflow,
                   cudaStream_t s) {
  if (E < 1 || E > MAX_EXPERTS || ep < 1 || ep > MAX_RANKS || E % ep != 0) {
    set_last_error("dh_moe_offsets: E=%d ep=%d unsupported", E, ep);
    return (int)cudaErrorInvalidValue;
  }
  moe_offsets_kernel<<<1, 256, 0, s>>>((const int*)cnt_all, ep, E, me, capacity, (int*)dst_base, (int*)offs, (int*)rows_e, (int*)overflow,
                                      reinterpret_cast<DeviceStatus*>(dh_status_device_ptr()));
  return moe_rc("dh_moe_offsets");
}

int dh_moe_zero_pad(void* buf, const void* offs, const void* rows_e, int el, int h, cudaStream_t s) {
  if (h % 8 != 0) { set_last_error("dh_moe_zero_pad: row width must be a multiple of 8"); return (int)cudaErrorInvalidValue; }
  moe_zero_pad_kernel<<<dim3(8, el), 256, 0, s>>>((__nv_bfloat16*)buf, (const int*)offs, (const int*)rows_e, h);
  return moe_rc("dh_moe_zero_pad");
}

// Pushes every copy's source row (src[i / k], optionally scaled by scale[i]) to row dst_base[e] + pos[i] of the owner of its
// expert e = topi[i]; optionally dots[i] = <src row, other[i]>.  dst_ptrs / arrived_ptrs: `ep` device pointers.
int dh_moe_dispatch(const void* src, int64_t ld_src, const void* topi, const void* pos, const void* dst_base, const void* scale,
                    const void* other, void* dots, void* const* dst_ptrs, void* dest_rank, void* dest_row, void* const* arrived_ptrs,
                    void* done_ctas, int n, int k, int h, int el, int ep, int ctas, cudaStream_t s) {
  if (ep < 1 || ep > MAX_RANKS || h % 8 != 0 || ld_src % 8 != 0) { set_last_error("dh_moe_dispatch: ep=%d h=%d unsupported", ep, h); return (int)cudaErrorInvalidValue; }
  DispatchParams p;
  p.src = (const __nv_bfloat16*)src; p.ld_src = ld_src;
  p.topi = (const int*)topi; p.pos = (const int*)pos; p.dst_base = (const int*)dst_base;
  p.scale = (const float*)scale; p.other = (const __nv_bfloat16*)other; p.dots = (float*)dots;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.dst[i] = i < ep ? (__nv_bfloat16*)dst_ptrs[i] : nullptr;
    p.arrived[i] = i < ep ? (uint32_t*)arrived_ptrs[i] : nullptr;
  }
  p.dest_rank = (int*)dest_rank; p.dest_row = (int*)dest_row;
  p.done_ctas = (unsigned int*)done_ctas;
  p.n = n; p.k = k; p.h = h; p.el = el; p.ep = ep;
  if (ctas <= 0) ctas = 64;
  moe_dispatch_kernel<<<ctas, 256, 0, s>>>(p);
  return moe_rc("dh_moe_dispatch");
}

// out[t] = sum_j gates[t*k+j] * src[dest_rank][dest_row] (gates null: plain sum); copies (nullable) keeps the pulled rows.
// Waits (bounded) until the local counter `ready` has reached `target` (every owner adds 1 when its rows are complete).
int dh_moe_combine(void* const* src_ptrs, const void* dest_rank, const void* dest_row, const void* gates, void* out, void* copies,
                   const void* ready, unsigned target, int T, int k, int h, int ep, int ctas, cudaStream_t s) {
  if (ep < 1 || ep > MAX_RANKS || h % 8 != 0) { set_last_error("dh_moe_combine: ep=%d h=%d unsupported", ep, h); return (int)cudaErrorInvalidValue; }
  CombineParams p;
  for (int i = 0; i < MAX_RANKS; ++i) p.src[i] = i < ep ? (const __nv_bfloat16*)src_ptrs[i] : nullptr;
  p.dest_rank = (const int*)dest_rank; p.dest_row = (const int*)dest_row; p.gates = (const float*)gates;
  p.out = (__nv_bfloat16*)out; p.copies = (__nv_bfloat16*)copies;
  p.ready = (const uint32_t*)ready; p.target = target;
  p.T = T; p.k = k; p.h = h;
  p.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  if (ctas <= 0) ctas = 64;
  moe_combine_kernel<<<ctas, 256, 0, s>>>(p);
  return moe_rc("dh_moe_combine");
}

}  // extern "C"
