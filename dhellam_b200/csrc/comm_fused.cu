// Stand-alone tensor-parallel collectives over NVLink / NVSwitch peer memory: small kernels
// without shared memory that share SMs with a GEMM running on another stream.  The device code
// is in comm_device.cuh and is also what the communication warps inside the CTA-pair GEMM kernel
// run (gemm_sm100.cu, dh_gemm_bf16_comm), so a collective can ride inside its GEMM or beside it.
//
//  ag_push / wait_counters : sequence all-gather: push this rank's shard to every rank and raise
//    per-128-row-block arrival counters; the consumer either waits for all counters in front of
//    its kernel (wait_counters) or, in the CTA-pair GEMM, per row block inside the kernel.
//
//  rs_reduce_blocks : sequence reduce-scatter over partial products that the ranks' GEMMs wrote
//    into their own symmetric buffers and signalled row block by row block; reduces each block of
//    this rank's rows as soon as every rank has delivered it (multimem.ld_reduce: the switch adds
//    the copies in fp32; plain peer loads without the multicast alias).
//
//  rs_reduce : the same reduction behind one whole-buffer announcement per rank, for producers
//    that cannot signal row blocks (anything that is not the CTA-pair GEMM).
//
// All buffers are double-buffered per call site with monotonically increasing counter targets (no
// resets, no host barriers).  Every wait is bounded and reports through the status word.
//
// Role in the reference: all_gather_into_tensor / reduce_scatter_tensor around torch.matmul
// (dhellam/operators/comm.py:13-58, dhellam/core/dstb.py:407-425) and the host-level
// chunk_allgather_gemm / chunk_gemm_reduce_scatter prototypes (comm.py:89-143).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"
#include "comm_device.cuh"
#include "ptx.cuh"
#include "tmap.h"

namespace dh {
namespace fused {

using namespace dh::comm;

struct CtaSync {
  __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

__global__ void __launch_bounds__(256) ag_push_kernel(const PushJob p) { push_rows(p, blockIdx.x, gridDim.x, threadIdx.x, blockDim.x, CtaSync()); }

// Waits (bounded, `budget` cycles; 0 = the default of about 20 s) until `n` counters have reached
// `target`; a later kernel on the same stream then reads the staged rows.
__global__ void __launch_bounds__(256) wait_counters_kernel(const uint32_t* count, int n, uint32_t target, long long budget, DeviceStatus* st) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    if (budget <= 0) wait_counter_sys(count + i, target, nullptr, st, 640);
    else flag_wait_geq_sys(count + i, target, budget, st, 641);
  }
}

__global__ void __launch_bounds__(256) rs_reduce_blocks_kernel(const ReduceJob p, DeviceStatus* status) {
  __shared__ int flag;
  reduce_rows(p, blockIdx.x, gridDim.x, threadIdx.x, blockDim.x, CtaSync(), &flag, status, 660);
}

// Whole-buffer form: tell every peer that this rank's partial product is complete (the kernel runs
// after the producing kernel in stream order), wait (bounded) for the same announcement from every
// peer, then reduce this rank's rows.
struct RsrParams {
  const __nv_bfloat16* part[MAX_RANKS];
  const __nv_bfloat16* part_mc;
  uint32_t* flag[MAX_RANKS];      // flag[p]: rank p's array of `world` announcement words
  __nv_bfloat16* out;
  int M, N, rank, world;
  uint32_t target;
  DeviceStatus* status;
};

__global__ void __launch_bounds__(256) rs_reduce_kernel(const RsrParams p) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    st_release_sys(p.flag[threadIdx.x] + p.rank, p.target);
  }
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!wait_counter_sys(p.flag[p.rank] + threadIdx.x, p.target, nullptr, p.status, 650)) ok_s = 0;
  }
  __syncthreads();
  if (!ok_s) return;
  const int rows = p.M / p.world;
  const long long nvec = (long long)rows * p.N / 8;
  const long long base = (long long)p.rank * rows * p.N;       // element offset of this rank's rows
  constexpr int U = 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 v[U];
    if (p.part_mc != nullptr) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < nvec) v[u] = multimem_ld_reduce_bf16x8(p.part_mc + base + (i0 + u * stride) * 8);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * stride >= nvec) continue;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f, a5 = 0.f, a6 = 0.f, a7 = 0.f;
        for (int r = 0; r < p.world; ++r) {
          const uint4 w = ld_relaxed_sys_v4(p.part[(p.rank + r) % p.world] + base + (i0 + u * stride) * 8);
          const float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z), f3 = unpack_bf16x2(w.w);
          a0 += f0.x; a1 += f0.y; a2 += f1.x; a3 += f1.y; a4 += f2.x; a5 += f2.y; a6 += f3.x; a7 += f3.y;
        }
        v[u] = make_uint4(pack_bf16x2(a0, a1), pack_bf16x2(a2, a3), pack_bf16x2(a4, a5), pack_bf16x2(a6, a7));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i0 + u * stride < nvec) st_v4(p.out + (i0 + u * stride) * 8, v[u]);
  }
}

}  // namespace fused
}  // namespace dh

using namespace dh;
using namespace dh::fused;

// Fills a PushJob; shared with the GEMM-resident form (gemm_sm100.cu).
int dh_fill_push_job(dh::comm::PushJob& p, const char* who, const void* shard, void* const* stage_ptrs, void* const* count_ptrs,
                     void* stage_mc, int M, int K, int rank, int world, int slices) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("%s: world size %d not in [2, %d]", who, world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (M % (world * ROW_BLOCK) != 0 || K % 64 != 0) { set_last_error("%s: M must divide by world*128 and K by 64 (M=%d K=%d)", who, M, K); return (int)cudaErrorInvalidValue; }
  if (slices < 1 || K % (slices * 8) != 0) { set_last_error("%s: %d column slices do not divide K=%d into multiples of 8", who, slices, K); return (int)cudaErrorInvalidValue; }
  p.shard = (const __nv_bfloat16*)shard;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.stage[i] = i < world ? (__nv_bfloat16*)stage_ptrs[i] : nullptr;
    p.count[i] = i < world ? (uint32_t*)count_ptrs[i] : nullptr;
  }
  p.stage_mc = (__nv_bfloat16*)stage_mc;
  p.K = K;
  p.src_ld = K;
  p.rank = rank; p.world = world;
  p.blocks_per_rank = M / world / ROW_BLOCK;
  p.dst_block0 = rank * p.blocks_per_rank;
  p.slices = slices;
  return 0;
}

int dh_fill_reduce_job(dh::comm::ReduceJob& p, const char* who, void* const* part_ptrs, const void* part_mc, const void* ready, void* out,
                       int M, int N, int rank, int world, unsigned target, int slices) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("%s: world size %d not in [2, %d]", who, world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (M % (world * ROW_BLOCK) != 0 || N % 8 != 0) { set_last_error("%s: M must divide by world*128 and N by 8 (M=%d N=%d)", who, M, N); return (int)cudaErrorInvalidValue; }
  if (slices < 1 || N % (slices * 8) != 0) { set_last_error("%s: %d column slices do not divide N=%d into multiples of 8", who, slices, N); return (int)cudaErrorInvalidValue; }
  for (int i = 0; i < MAX_RANKS; ++i) p.part[i] = i < world ? (const __nv_bfloat16*)part_ptrs[i] : nullptr;
  p.part_mc = (const __nv_bfloat16*)part_mc;
  p.ready = (const uint32_t*)ready;
  p.ready_stride = 1;
  p.out = (__nv_bfloat16*)out;
  p.out_ld = N;
  p.N = N; p.rank = rank; p.world = world;
  p.rows = M / world;
  p.in_block0 = rank * (p.rows / ROW_BLOCK);
  p.blocks = (p.rows + ROW_BLOCK - 1) / ROW_BLOCK;
  p.slices = slices;
  p.target = target;
  return 0;
}

extern "C" {

// Column slices per 128-row block for (blocks x slices) work items over about `groups` thread groups.
int dh_comm_slices(int blocks, int width, int groups) { return dh::comm::slices_for(blocks, width, groups); }

// Stand-alone all-gather of a row shard into every rank's staging buffer (push only; pair it with
// dh_wait_counters on the consumer's stream or with the in-kernel wait of dh_gemm_bf16_sync).
// stage_ptrs / count_ptrs: `world` device pointers (index = rank); stage_mc: multicast address of the
// same staging buffer or null.  Every row-block counter on every rank rises by `slices`.
int dh_ag_push(const void* shard, void* const* stage_ptrs, void* const* count_ptrs, void* stage_mc, int M, int K, int rank, int world,
               int ctas, int threads, int slices, cudaStream_t stream) {
  PushJob p;
  int rc = dh_fill_push_job(p, "dh_ag_push", shard, stage_ptrs, count_ptrs, stage_mc, M, K, rank, world, slices);
  if (rc) return rc;
  if (ctas <= 0) ctas = 16;
  if (threads <= 0 || threads > 256 || threads % 32 != 0) threads = 256;
  ag_push_kernel<<<ctas, threads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_ag_push launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Generic placement form of the push, used by context parallelism to gather the key / value rows of all
// ranks in global sequence order: `n_blocks` 128-row blocks of `src` (row stride src_ld elements, width K)
// land at row block `dst_block0` of every rank's buffer; each of those blocks' counters rises by `slices`.
int dh_push_blocks(const void* src, int64_t src_ld, void* const* dst_ptrs, void* const* count_ptrs, void* dst_mc, int K, int n_blocks,
                   int dst_block0, int rank, int world, int ctas, int threads, int slices, cudaStream_t stream) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("dh_push_blocks: world size %d not in [2, %d]", world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (K % 8 != 0 || slices < 1 || K % (slices * 8) != 0 || src_ld % 8 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0) {
    set_last_error("dh_push_blocks: rows must be 16-byte aligned and %d slices must divide K=%d into multiples of 8", slices, K);
    return (int)cudaErrorInvalidValue;
  }
  PushJob p;
  p.shard = (const __nv_bfloat16*)src;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.stage[i] = i < world ? (__nv_bfloat16*)dst_ptrs[i] : nullptr;
    p.count[i] = i < world ? (uint32_t*)count_ptrs[i] : nullptr;
  }
  p.stage_mc = (__nv_bfloat16*)dst_mc;
  p.K = K;
  p.src_ld = src_ld;
  p.rank = rank; p.world = world;
  p.blocks_per_rank = n_blocks;
  p.dst_block0 = dst_block0;
  p.slices = slices;
  if (ctas <= 0) ctas = 16;
  if (threads <= 0 || threads > 256 || threads % 32 != 0) threads = 256;
  ag_push_kernel<<<ctas, threads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_push_blocks launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Adds `value` to one counter on every rank (system-scope release): "everything this rank launched before on
// this stream is in memory".  Pairs with dh_reduce_blocks(ready_stride = 0).
__global__ void announce_kernel(uint32_t* c0, uint32_t* c1, uint32_t* c2, uint32_t* c3, uint32_t* c4, uint32_t* c5, uint32_t* c6, uint32_t* c7,
                                int world, uint32_t value) {
  uint32_t* c[8] = {c0, c1, c2, c3, c4, c5, c6, c7};
  if ((int)threadIdx.x < world) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    red_add_release_sys(c[threadIdx.x], value);
  }
}
int dh_announce(void* const* counter_ptrs, int world, unsigned value, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS) { set_last_error("dh_announce: world size %d not in [1, %d]", world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  uint32_t* c[8];
  for (int i = 0; i < 8; ++i) c[i] = i < world ? (uint32_t*)counter_ptrs[i] : nullptr;
  announce_kernel<<<1, 32, 0, stream>>>(c[0], c[1], c[2], c[3], c[4], c[5], c[6], c[7], world, value);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_announce launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Generic placement form of the reduction: `rows` rows starting at row block `in_block0` of every rank's buffer
// (width N) are summed over the ranks into out (row stride out_ld).  ready / ready_stride / target: the counters
// that say the rows are complete on every rank (stride 0: one counter for all of them).
int dh_reduce_blocks(void* const* part_ptrs, const void* part_mc, const void* ready, int ready_stride, void* out, int64_t out_ld, int N,
                     int in_block0, int rows, int rank, int world, unsigned target, int ctas, int threads, cudaStream_t stream) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("dh_reduce_blocks: world size %d not in [2, %d]", world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (N % 8 != 0 || out_ld % 8 != 0 || rows <= 0) { set_last_error("dh_reduce_blocks: N and out_ld must be multiples of 8"); return (int)cudaErrorInvalidValue; }
  if (ctas <= 0) ctas = 32;
  if (threads <= 0 || threads > 256 || threads % 32 != 0) threads = 256;
  ReduceJob p;
  for (int i = 0; i < MAX_RANKS; ++i) p.part[i] = i < world ? (const __nv_bfloat16*)part_ptrs[i] : nullptr;
  p.part_mc = (const __nv_bfloat16*)part_mc;
  p.ready = (const uint32_t*)ready;
  p.ready_stride = ready_stride ? 1 : 0;
  p.out = (__nv_bfloat16*)out;
  p.out_ld = out_ld;
  p.N = N; p.rank = rank; p.world = world;
  p.rows = rows;
  p.in_block0 = in_block0;
  p.blocks = (rows + ROW_BLOCK - 1) / ROW_BLOCK;
  p.slices = dh::comm::reduce_slices_for(N, ctas);
  p.target = target;
  rs_reduce_blocks_kernel<<<ctas, threads, 0, stream>>>(p, reinterpret_cast<DeviceStatus*>(dh_status_device_ptr()));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_reduce_blocks launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// budget_cycles: how long the wait may last before it gives up with status code 2 (0 = default, about 20 s).
int dh_wait_counters(const void* counters, int n, unsigned target, long long budget_cycles, cudaStream_t stream) {
  wait_counters_kernel<<<1, 256, 0, stream>>>((const uint32_t*)counters, n, target, budget_cycles,
                                              reinterpret_cast<DeviceStatus*>(dh_status_device_ptr()));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_wait_counters launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Row-block-wise reduce-scatter.  ready: this rank's per-block counters; target: the value a complete block
// reaches in this call; part_ptrs: every rank's partial buffer [M][N]; part_mc: their multicast alias or null.
int dh_rs_reduce_blocks(void* const* part_ptrs, const void* part_mc, const void* ready, void* out, int M, int N, int rank, int world,
                        unsigned target, int ctas, int threads, cudaStream_t stream) {
  if (ctas <= 0) ctas = 32;
  if (threads <= 0 || threads > 256 || threads % 32 != 0) threads = 256;
  ReduceJob p;
  const int blocks = (M / (world > 0 ? world : 1) + ROW_BLOCK - 1) / ROW_BLOCK;
  int rc = dh_fill_reduce_job(p, "dh_rs_reduce_blocks", part_ptrs, part_mc, ready, out, M, N, rank, world, target,
                              dh::comm::reduce_slices_for(N, ctas));
  if (rc) return rc;
  rs_reduce_blocks_kernel<<<ctas, threads, 0, stream>>>(p, reinterpret_cast<DeviceStatus*>(dh_status_device_ptr()));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_rs_reduce_blocks launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Whole-buffer reduce-scatter of per-rank partial products that already sit in symmetric memory.
// part_ptrs / flag_ptrs: `world` device pointers (every rank's partial buffer [M][N] and announcement
// words); part_mc: multicast alias of the partial buffers or null; `target` is the announcement value of
// this call (strictly increasing per buffer).
int dh_rs_reduce(void* const* part_ptrs, const void* part_mc, void* const* flag_ptrs, void* out, int M, int N, int rank, int world,
                 unsigned target, int ctas, cudaStream_t stream) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("dh_rs_reduce: world size %d not in [2, %d]", world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (M % world != 0 || N % 8 != 0) { set_last_error("dh_rs_reduce: M must divide by world and N by 8 (M=%d N=%d)", M, N); return (int)cudaErrorInvalidValue; }
  RsrParams p;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.part[i] = i < world ? (const __nv_bfloat16*)part_ptrs[i] : nullptr;
    p.flag[i] = i < world ? (uint32_t*)flag_ptrs[i] : nullptr;
  }
  p.part_mc = (const __nv_bfloat16*)part_mc;
  p.out = (__nv_bfloat16*)out;
  p.M = M; p.N = N; p.rank = rank; p.world = world;
  p.target = target;
  p.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  if (ctas <= 0) ctas = 32;
  rs_reduce_kernel<<<ctas, 256, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_rs_reduce launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

}  // extern "C"
