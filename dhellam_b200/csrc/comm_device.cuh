// Device-side pieces of the tensor-parallel collectives over NVLink / NVSwitch peer memory,
// shared by the stand-alone communication kernels (comm_fused.cu) and by the communication warps
// that ride inside the CTA-pair GEMM kernel (gemm_sm100.cu).
//
//   push_rows     sequence all-gather, sender side: read this rank's row shard once and store it
//                 into every rank's staging buffer (one multimem.st per 16 bytes reaches all GPUs
//                 through the switch; per-peer stores without the multicast alias), then bump the
//                 per-128-row-block arrival counter on every receiver with a system-scope release.
//   reduce_rows   sequence reduce-scatter, owner side: wait (bounded) per 128-row block until
//                 every rank has delivered its partial product of that block, then reduce the
//                 block (multimem.ld_reduce adds the copies in fp32 inside the switch; plain peer
//                 loads + fp32 adds without the alias) into the bf16 output shard.
//
// Role in the reference: all_gather_into_tensor / reduce_scatter_tensor along the sequence dimension
// (dhellam/operators/comm.py:13-58) and its chunked prototypes (comm.py:89-143).
//
// Both are written for "a group of T threads of one CTA" (a whole 256-thread CTA of a stand-alone
// kernel, or the 64 threads of the two communication warps of a GEMM CTA); `group_sync` is the
// barrier of that group.  Work items are (row block, column slice) and are spread over `ngroups`
// groups.  No load here is a multi-CTA broadcast; peer memory is only the target of plain /
// multimem stores and the source of plain / multimem loads.  Every wait is bounded.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx.cuh"

namespace dh {
namespace comm {

constexpr int ROW_BLOCK = 128;
constexpr int MAX_RANKS = 8;
constexpr long long PEER_WAIT_CYCLES = 40000000000ll;     // ~20 s: covers start-up skew between ranks

__device__ __forceinline__ bool wait_counter_sys(const uint32_t* p, uint32_t want, volatile int* abort_flag, DeviceStatus* st, int where) {
  if (ld_acquire_sys(p) >= want) return true;
  const long long t0 = clock64();
  while (true) {
    if (ld_acquire_sys(p) >= want) return true;
    __nanosleep(100);
    if (abort_flag != nullptr && *abort_flag) return false;
    if (clock64() - t0 > PEER_WAIT_CYCLES) {
      if (abort_flag != nullptr) *abort_flag = 1;
      report_error(st, ERR_FLAG_TIMEOUT, where, (int)want);
      return false;
    }
  }
}

// One 16-byte store that the NVSwitch replicates into the buffer of every rank of the group.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// One 16-byte load whose eight bf16 values are the fp32-accumulated sums over all ranks' copies.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// ------------------------------------------------------------------------------------------ all-gather push
struct PushJob {
  const __nv_bfloat16* shard;            // [blocks_per_rank * 128, K] this rank's rows (any memory), row stride src_ld
  __nv_bfloat16* stage[MAX_RANKS];       // staging [M, K] on every rank (stage[rank] is local)
  __nv_bfloat16* stage_mc;               // the same staging through the multicast address (null: per-peer stores)
  uint32_t* count[MAX_RANKS];            // per row-block arrival counters on every rank
  int K;                                 // row width in elements
  long long src_ld;                      // elements between consecutive source rows (K when contiguous)
  int rank, world, blocks_per_rank;
  int dst_block0;                        // 128-row block of the staging buffer where the first pushed block lands
  int slices;                            // column slices per row block = counter increments per block and call
};

template <typename Sync>
__device__ __forceinline__ void push_rows(const PushJob& p, int group, int ngroups, int tid, int nthreads, Sync group_sync) {
  constexpr int U = 8;
  const int items = p.blocks_per_rank * p.slices;
  const int cw = p.K / p.slices;                            // columns per slice (multiple of 8)
  const int vec_per_row = cw >> 3;
  const int total = ROW_BLOCK * vec_per_row;
  for (int it = group; it < items; it += ngroups) {
    const int lb = it / p.slices, sl = it - lb * p.slices;
    const int gb = p.dst_block0 + lb;                       // row block in the staging buffer
    const long long src_base = (long long)lb * ROW_BLOCK * p.src_ld + (long long)sl * cw;
    const long long dst_base = (long long)gb * ROW_BLOCK * p.K + (long long)sl * cw;
    for (int i0 = tid; i0 < total; i0 += nthreads * U) {
      uint4 v[U];
      long long off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * nthreads;
        if (i < total) {
          const int r = i / vec_per_row, c = i - r * vec_per_row;
          off[u] = (long long)r * p.K + c * 8;
          v[u] = ld_nc_v4(p.shard + src_base + (long long)r * p.src_ld + c * 8);
        }
      }
      if (p.stage_mc != nullptr) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * nthreads < total) multimem_st_v4(p.stage_mc + dst_base + off[u], v[u]);
      } else {
        for (int j = 0; j < p.world; ++j) {
          __nv_bfloat16* dst = p.stage[(p.rank - j + p.world) % p.world] + dst_base;
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * nthreads < total) *reinterpret_cast<uint4*>(dst + off[u]) = v[u];
        }
      }
    }
    group_sync();
    if (tid == 0) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      // one fence, then relaxed reductions: a release reduction per rank would repeat the fence world times
      for (int j = 0; j < p.world; ++j) red_add_relaxed_sys(p.count[(p.rank - j + p.world) % p.world] + gb, 1u);
    }
  }
}

// ------------------------------------------------------------------------------------------ row-block-wise reduce
struct ReduceJob {
  const __nv_bfloat16* part[MAX_RANKS];  // every rank's partial product [M][N] (symmetric memory)
  const __nv_bfloat16* part_mc;          // the same through the multicast address (null: peer loads)
  const uint32_t* ready;                 // this rank's completion counters (local memory)
  int ready_stride;                      // 1: one counter per row block; 0: one counter for the whole buffer
  __nv_bfloat16* out;                    // [rows, N]: the reduced rows, row stride out_ld
  long long out_ld;
  int N, rank, world;
  int in_block0;                         // first 128-row block of this rank's rows inside the partial products
  int rows;                              // number of rows to reduce (blocks = ceil(rows / 128))
  int blocks, slices;
  uint32_t target;                       // counter value that means "every rank has delivered"
};

// Returns false if a bounded wait gave up (the status word says where).  `flag` is one int of shared
// memory owned by the group.
template <typename Sync>
__device__ __forceinline__ bool reduce_rows(const ReduceJob& p, int group, int ngroups, int tid, int nthreads, Sync group_sync, int* flag,
                                            DeviceStatus* status, int where) {
  constexpr int U = 8;
  const int cw = p.N / p.slices;                            // columns per slice (multiple of 8)
  const int vec_per_row = cw >> 3;
  const int items = p.blocks * p.slices;
  for (int it = group; it < items; it += ngroups) {
    const int b = it / p.slices, sl = it - b * p.slices;
    group_sync();
    if (tid == 0) *flag = wait_counter_sys(p.ready + b * p.ready_stride, p.target, nullptr, status, where) ? 1 : 0;
    group_sync();
    if (!*flag) return false;
    const int rows = min(ROW_BLOCK, p.rows - b * ROW_BLOCK);
    const int total = rows * vec_per_row;
    const long long in_base = ((long long)p.in_block0 + b) * ROW_BLOCK * p.N + (long long)sl * cw;
    const long long out_base = (long long)b * ROW_BLOCK * p.out_ld + (long long)sl * cw;
    for (int i0 = tid; i0 < total; i0 += nthreads * U) {
      uint4 v[U];
      long long off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * nthreads;
        if (i < total) {
          const int r = i / vec_per_row, c = i - r * vec_per_row;
          off[u] = (long long)r * p.N + c * 8;
          if (p.part_mc != nullptr) v[u] = multimem_ld_reduce_bf16x8(p.part_mc + in_base + off[u]);
        }
      }
      if (p.part_mc == nullptr) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * nthreads >= total) continue;
          float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f, a5 = 0.f, a6 = 0.f, a7 = 0.f;
          for (int q = 0; q < p.world; ++q) {
            const uint4 w = ld_relaxed_sys_v4(p.part[(p.rank + q) % p.world] + in_base + off[u]);
            const float2 f0 = unpack_bf16x2(w.x), f1 = unpack_bf16x2(w.y), f2 = unpack_bf16x2(w.z), f3 = unpack_bf16x2(w.w);
            a0 += f0.x; a1 += f0.y; a2 += f1.x; a3 += f1.y; a4 += f2.x; a5 += f2.y; a6 += f3.x; a7 += f3.y;
          }
          v[u] = make_uint4(pack_bf16x2(a0, a1), pack_bf16x2(a2, a3), pack_bf16x2(a4, a5), pack_bf16x2(a6, a7));
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * nthreads >= total) continue;
        const int i = i0 + u * nthreads;
        const int r = i / vec_per_row, c = i - r * vec_per_row;
        st_v4(p.out + out_base + (long long)r * p.out_ld + c * 8, v[u]);
      }
    }
  }
  return true;
}

// Column slices per 128-row block: (row blocks x slices) work items are dealt to `groups` thread groups block by
// block.  Enough slices that only about four row blocks are in flight at a time (the first blocks of a pushed
// shard arrive early, and every group works on the row block of a reduction that has just become complete), at
// most 32 (an item then still moves 64 KB per fence / per counter wait at width 8192), and at least one item per
// group.  A pure function of its arguments, so every rank and the host agree on the counter increments.
__host__ __device__ inline int slices_for(int blocks, int width, int groups) {
  int s = 1;
  while ((blocks * s < groups || s * 4 < groups) && s < 32 && (width / (s * 2)) % 8 == 0 && width / (s * 2) >= 64) s *= 2;
  return s;
}

__host__ __device__ inline int reduce_slices_for(int width, int groups) { return slices_for(1 << 20, width, groups); }

}  // namespace comm
}  // namespace dh
