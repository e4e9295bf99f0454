// Tensor-parallel collectives over NVLink / NVSwitch peer memory: inside the tcgen05 GEMM kernels
// and as stand-alone kernels that share SMs with a GEMM running on another stream.
//
//  ag_gemm : sequence all-gather -> GEMM            (QKV / FC1 forward, proj / FC2 dgrad)
//    A few "copy" CTAs of the same grid push this rank's row shard into every rank's symmetric
//    staging buffer (one multimem.st per 16 bytes reaches all GPUs through the switch; per-peer
//    stores without the multicast alias; data is read once from HBM) and bump a per-row-block
//    counter on every receiver with a system-scope release.  The GEMM CTAs walk the row blocks
//    starting with the local shard; the TMA producer of a tile waits (bounded) on the counter of
//    its row block and then loads A from LOCAL memory only.  The gathered operand stays in the
//    staging buffer for the weight-gradient GEMM of the same layer.
//
//  gemm_rs : GEMM -> sequence reduce-scatter        (proj / FC2 forward, QKV / FC1 dgrad)
//    The epilogue stages each partial tile through shared memory and stores it, 256 bytes per
//    row segment, straight into the row OWNER's symmetric buffer (slot = source rank), then bumps
//    a per-source arrival counter there; row blocks of remote owners are computed first, the
//    local ones last.  After its last tile every CTA waits (bounded) for all sources and the
//    whole grid reduces the owner's slots in fp32 to the bf16 shard.
//
//  ag_push / wait_counters : the all-gather alone (push on the communication stream, counter
//    wait in front of the consumer), used where the schedule hides the transfer behind the other
//    strand's kernels and to re-gather a saved shard for a weight gradient.
//
//  rs_reduce : the reduce-scatter alone over partial products that a plain local GEMM wrote
//    into symmetric memory: announcement flags, then multimem.ld_reduce (the switch adds the
//    copies in fp32) or peer loads.
//
// All buffers are double-buffered per call site with monotonically increasing counter targets
// (no resets, no host barriers).  Kernels that wait for peers inside the kernel are launched one
// at a time and in the same order on every rank, which makes the double buffering sufficient: a
// rank can only finish call c after every peer has started call c, i.e. finished call c-1.
//
// No load in this file is a multi-CTA broadcast; peer memory is only ever the target of plain or
// multimem stores / reductions or the source of plain or multimem loads.
//
// Role in the reference: all_gather_into_tensor / reduce_scatter_tensor around torch.matmul
// (dhellam/operators/comm.py:13-58, dhellam/core/dstb.py:407-425) and the host-level
// chunk_allgather_gemm / chunk_gemm_reduce_scatter prototypes (comm.py:89-143).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

namespace dh {
namespace fused {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2, STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_ACC = 2, ACC_COLS = BN, TMEM_COLS = 512;
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;
constexpr int MAX_RANKS = 8;
constexpr long long PEER_WAIT_CYCLES = 40000000000ll;     // ~20 s: covers start-up skew between ranks
// Barriers inside the CTA sit downstream of a peer wait (the MMA warp waits for a stage that the
// producer fills only after a peer's data arrived), so they must outlast it.
constexpr long long LOCAL_WAIT_CYCLES = 2 * PEER_WAIT_CYCLES;

struct __align__(8) Control {
  uint64_t full[STAGES], empty[STAGES], acc_full[NUM_ACC], acc_empty[NUM_ACC];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int RS_STAGE_BYTES = 4 * 32 * 256;
constexpr int RS_SMEM_BYTES = SMEM_BYTES + RS_STAGE_BYTES;

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band = GROUP_M * tiles_n;
  const int g = t / band;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = t - g * band;
  tm = first_m + (r % rows);
  tn = r / rows;
}

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

// ------------------------------------------------------------------ shared main-loop pieces
template <bool B_MN>
__device__ __forceinline__ void load_stage(uint8_t* a_dst, uint8_t* b_dst, const CUtensorMap* ta, const CUtensorMap* tb, uint64_t* bar,
                                           int m0, int n0, int k0) {
  mbar_expect_tx(bar, STAGE_BYTES);
  tma_load_2d(a_dst, ta, bar, k0, m0);
  if (B_MN) {
#pragma unroll
    for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), tb, bar, n0 + 64 * j, k0);
  } else {
    tma_load_2d(b_dst, tb, bar, k0, n0);
  }
}

template <bool B_MN>
__device__ __forceinline__ void mma_stage(uint32_t tmem_acc, uint32_t a_base, uint32_t b_base, bool first) {
  constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, B_MN ? 1 : 0);
#pragma unroll
  for (int kk = 0; kk < BK / UMMA_K; ++kk) {
    const uint64_t adesc = umma_smem_desc(a_base + kk * 32, 16, 1024);
    const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + kk * 2048, BK * 128, 1024) : umma_smem_desc(b_base + kk * 32, 16, 1024);
    umma_bf16(tmem_acc, adesc, bdesc, idesc, (!first || kk != 0) ? 1u : 0u);
  }
}

// ============================================================================ all-gather -> GEMM
struct AgParams {
  const __nv_bfloat16* shard;            // [rows_per_rank, K] this rank's rows (any memory)
  __nv_bfloat16* stage[MAX_RANKS];       // staging [M, K] on every rank (stage[rank] is local)
  __nv_bfloat16* stage_mc;               // the same staging through the NVSwitch multicast address (null: unicast stores)
  uint32_t* count[MAX_RANKS];            // per row-block arrival counters on every rank
  __nv_bfloat16* d;                      // output [M, N]
  long long ldd;
  int M, N, K;
  int tiles_m, tiles_n;
  int rank, world, rows_per_rank, blocks_per_rank;
  int copy_ctas, slices;                 // slices per row block (column split of the push work)
  uint32_t target;                       // counter value that means "this call's block is complete"
  DeviceStatus* status;
};

// One 16-byte store that the NVSwitch replicates into the buffer of every rank of the group.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Pushes this rank's shard into every rank's staging buffer and raises the row-block counters.
// Work items are (row block, column slice); `cta`/`ncta` spread them over the calling CTAs.
// Eight independent 16-byte loads are in flight per thread; with the multicast address one
// store reaches all ranks, otherwise the registers are stored to each rank in turn (the rank
// that consumes this shard earliest first).
__device__ __forceinline__ void push_shard(const AgParams& p, int cta, int ncta) {
  constexpr int U = 8;
  const int items = p.blocks_per_rank * p.slices;
  const int cw = p.K / p.slices;                            // columns per slice (multiple of 8)
  const int vec_per_row = cw >> 3;
  const int total = BM * vec_per_row;
  for (int it = cta; it < items; it += ncta) {
    const int lb = it / p.slices, sl = it - lb * p.slices;
    const int gb = p.rank * p.blocks_per_rank + lb;         // global row block
    const long long src_base = (long long)lb * BM * p.K + (long long)sl * cw;
    const long long dst_base = (long long)gb * BM * p.K + (long long)sl * cw;
    for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * U) {
      uint4 v[U];
      long long off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < total) {
          const int r = i / vec_per_row, c = i - r * vec_per_row;
          off[u] = (long long)r * p.K + c * 8;
          v[u] = ld_nc_v4(p.shard + src_base + off[u]);
        }
      }
      if (p.stage_mc != nullptr) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * blockDim.x < total) multimem_st_v4(p.stage_mc + dst_base + off[u], v[u]);
      } else {
        for (int j = 0; j < p.world; ++j) {
          __nv_bfloat16* dst = p.stage[(p.rank - j + p.world) % p.world] + dst_base;
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * blockDim.x < total) *reinterpret_cast<uint4*>(dst + off[u]) = v[u];
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int j = 0; j < p.world; ++j) red_add_release_sys(p.count[(p.rank - j + p.world) % p.world] + gb, 1u);
    }
  }
}

// Stand-alone all-gather: only the push (used to re-gather a saved shard for a weight gradient).
__global__ void __launch_bounds__(256) ag_push_kernel(const AgParams p) { push_shard(p, blockIdx.x, gridDim.x); }

// Waits (bounded) until `n` counters have reached `target`; a later kernel on the same stream
// then reads the staged rows.
__global__ void __launch_bounds__(256) wait_counters_kernel(const uint32_t* count, int n, uint32_t target, DeviceStatus* st) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) wait_counter_sys(count + i, target, nullptr, st, 640);
}


// Stand-alone sequence reduce-scatter over partial products that every rank wrote into its
// own symmetric buffer `part[rank]` ([M][N], all rows).  The kernel first tells every peer
// that this rank's partial is complete (it runs after the producing GEMM in stream order),
// waits (bounded) for the same announcement from every peer, and then reduces its own
// M/world rows: with a multicast alias of the buffers one `multimem.ld_reduce` per 16 bytes
// lets the NVSwitch add the eight copies in fp32 and return the sum, so a GPU receives
// M/world x N values instead of (world-1) times that; without the alias it reads the rows of
// every peer with plain loads and adds in fp32.  A few CTAs without shared memory: they
// share SMs with a GEMM that is running on the compute stream.
struct RsrParams {
  const __nv_bfloat16* part[MAX_RANKS];
  const __nv_bfloat16* part_mc;
  uint32_t* flag[MAX_RANKS];      // flag[p]: rank p's array of `world` announcement words
  __nv_bfloat16* out;
  int M, N, rank, world;
  uint32_t target;
  DeviceStatus* status;
};

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
  constexpr int U = 4;
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
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r = 0; r < p.world; ++r) {
          const uint4 w = ld_relaxed_sys_v4(p.part[(p.rank + r) % p.world] + base + (i0 + u * stride) * 8);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(ww[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
        v[u] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i0 + u * stride < nvec) st_v4(p.out + (i0 + u * stride) * 8, v[u]);
  }
}

// Row-block-wise form of the reduction above.  The producing GEMMs (dh_gemm_bf16_sync with
// sig_ptrs) bump, on the rank that owns a 128-row block, that block's counter once per stored
// 32-row piece of every tile; a block is complete on all ranks when its counter reaches
// `target`.  Work items are (row block, column slice); a CTA waits (bounded) for its item's
// block only, so the reduction of the first blocks runs while every rank's GEMM is still
// producing the later ones.  Eight independent 16-byte reductions are in flight per thread:
// the reduction is bound by the round trip through the switch, not by bytes.
struct RsbParams {
  const __nv_bfloat16* part[MAX_RANKS];
  const __nv_bfloat16* part_mc;
  const uint32_t* ready;          // this rank's per-block counters (local memory)
  __nv_bfloat16* out;
  int M, N, rank, world, blocks, slices;
  uint32_t target;
  DeviceStatus* status;
};

__global__ void __launch_bounds__(256) rs_reduce_blocks_kernel(const RsbParams p) {
  __shared__ int ok_s;
  constexpr int U = 8;
  const int rows_per_rank = p.M / p.world;
  const int cw = p.N / p.slices;                              // columns per slice (multiple of 8)
  const int vec_per_row = cw >> 3;
  const int items = p.blocks * p.slices;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int b = it / p.slices, sl = it - b * p.slices;
    __syncthreads();
    if (threadIdx.x == 0) ok_s = wait_counter_sys(p.ready + b, p.target, nullptr, p.status, 660) ? 1 : 0;
    __syncthreads();
    if (!ok_s) return;
    const int rows = min(BM, rows_per_rank - b * BM);
    const int total = rows * vec_per_row;
    const long long in_base = ((long long)p.rank * rows_per_rank + (long long)b * BM) * p.N + (long long)sl * cw;
    const long long out_base = (long long)b * BM * p.N + (long long)sl * cw;
    for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * U) {
      uint4 v[U];
      long long off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < total) {
          const int r = i / vec_per_row, c = i - r * vec_per_row;
          off[u] = (long long)r * p.N + c * 8;
          if (p.part_mc != nullptr) v[u] = multimem_ld_reduce_bf16x8(p.part_mc + in_base + off[u]);
        }
      }
      if (p.part_mc == nullptr) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * blockDim.x >= total) continue;
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int q = 0; q < p.world; ++q) {
            const uint4 w = ld_relaxed_sys_v4(p.part[(p.rank + q) % p.world] + in_base + off[u]);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16x2(ww[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
          v[u] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * blockDim.x < total) st_v4(p.out + out_base + off[u], v[u]);
    }
  }
}

template <bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const AgParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  Control* ctl = reinterpret_cast<Control*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ------------------------------------------------------------------ copy CTAs
  if ((int)blockIdx.x < p.copy_ctas) {
    push_shard(p, blockIdx.x, p.copy_ctas);
    return;
  }

  // ------------------------------------------------------------------ GEMM CTAs
  const int gemm_ctas = gridDim.x - p.copy_ctas;
  const int cta = blockIdx.x - p.copy_ctas;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < NUM_ACC; ++a) { mbar_init(&ctl->acc_full[a], 1); mbar_init(&ctl->acc_empty[a], 4); }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ctl->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  const int rot = p.rank * p.blocks_per_rank;               // local row blocks first

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int ready_block = -1;
      for (int t = cta; t < num_tiles && ok; t += gemm_ctas) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        tm = (tm + rot) % p.tiles_m;
        if (tm != ready_block) {
          if (!wait_counter_sys(p.count[p.rank] + tm, p.target, abort_flag, p.status, 610)) { ok = false; break; }
          fence_proxy_async_all();                          // peer / other-CTA stores -> visible to the TMA reads below
          ready_block = tm;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 611, LOCAL_WAIT_CYCLES)) { ok = false; break; }
          load_stage<B_MN>(sA + s * A_STAGE_BYTES, sB + s * B_STAGE_BYTES, &tmap_a, &tmap_b, &ctl->full[s], tm * BM, tn * BN, kb * BK);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += gemm_ctas) {
        if (!mbar_wait(&ctl->acc_empty[acc], acc_ph ^ 1, abort_flag, p.status, 620, LOCAL_WAIT_CYCLES)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, p.status, 621, LOCAL_WAIT_CYCLES)) { ok = false; break; }
          tc_fence_after();
          mma_stage<B_MN>(tmem_base + acc * ACC_COLS, smem_u32(sA + s * A_STAGE_BYTES), smem_u32(sB + s * B_STAGE_BYTES), kb == 0);
          umma_commit(&ctl->empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&ctl->acc_full[acc]);
        if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += gemm_ctas) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      tm = (tm + rot) % p.tiles_m;
      if (!mbar_wait(&ctl->acc_full[acc], acc_ph, abort_flag, p.status, 630, LOCAL_WAIT_CYCLES)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row >= p.M) continue;
        __nv_bfloat16* dst = p.d + (long long)row * p.ldd + col0;
        if (col0 + 32 <= p.N) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            reinterpret_cast<uint4*>(dst)[j] = v;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[acc]);
      if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ============================================================================ GEMM -> reduce-scatter
struct RsParams {
  __nv_bfloat16* part[MAX_RANKS];        // partial buffers [world][rows_per_rank, N] on every rank (slot = source rank)
  uint32_t* arrived[MAX_RANKS];          // per-source tile arrival counters on every rank
  __nv_bfloat16* out;                    // [rows_per_rank, N] reduced shard
  int M, N, K;
  int tiles_m, tiles_n;
  int rank, world, rows_per_rank, blocks_per_rank;
  uint32_t target;                       // arrival count (per source) that completes this call
  DeviceStatus* status;
};

template <bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const RsParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sStage = smem + STAGES * STAGE_BYTES;                       // 4 epilogue warps x 32 rows x 256 B
  Control* ctl = reinterpret_cast<Control*>(smem + STAGES * STAGE_BYTES + RS_STAGE_BYTES);
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < NUM_ACC; ++a) { mbar_init(&ctl->acc_full[a], 1); mbar_init(&ctl->acc_empty[a], 4); }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ctl->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  // remote owners first (rank+1, rank+2, ...), the local rows last
  const int rot = ((p.rank + 1) % p.world) * p.blocks_per_rank;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        tm = (tm + rot) % p.tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 700, LOCAL_WAIT_CYCLES)) { ok = false; break; }
          load_stage<B_MN>(sA + s * A_STAGE_BYTES, sB + s * B_STAGE_BYTES, &tmap_a, &tmap_b, &ctl->full[s], tm * BM, tn * BN, kb * BK);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&ctl->acc_empty[acc], acc_ph ^ 1, abort_flag, p.status, 710, LOCAL_WAIT_CYCLES)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, p.status, 711, LOCAL_WAIT_CYCLES)) { ok = false; break; }
          tc_fence_after();
          mma_stage<B_MN>(tmem_base + acc * ACC_COLS, smem_u32(sA + s * A_STAGE_BYTES), smem_u32(sB + s * B_STAGE_BYTES), kb == 0);
          umma_commit(&ctl->empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&ctl->acc_full[acc]);
        if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      tm = (tm + rot) % p.tiles_m;
      if (!mbar_wait(&ctl->acc_full[acc], acc_ph, abort_flag, p.status, 720, LOCAL_WAIT_CYCLES)) { ok = false; break; }
      tc_fence_after();
      const int owner = tm / p.blocks_per_rank;
      const int lrow0 = (tm - owner * p.blocks_per_rank) * BM + quarter * 32;            // first of this warp's 32 rows in the owner's shard
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      __nv_bfloat16* slot = p.part[owner] + ((long long)p.rank * p.rows_per_rank + lrow0) * p.N;
      // The accumulator rows are staged through shared memory so that one warp store covers
      // two whole 256-byte row segments: NVLink moves 128..256-byte payloads efficiently,
      // while 32 scattered 16-byte segments per store would not.
      uint8_t* stg = sStage + (warp - 2) * (32 * 256);
#pragma unroll 1
      for (int g = 0; g < BN / 128; ++g) {
        const int colg = tn * BN + g * 128;
        if (colg >= p.N) break;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t r[32];
          tmem_ld32(taddr + g * 128 + c4 * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            const int chunk = c4 * 4 + j;
            *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = v;
          }
        }
        __syncwarp();
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int rr = 2 * i + (lane >> 4), ch = lane & 15;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((ch ^ (rr & 15)) << 4));
          const int col = colg + ch * 8;
          if (col < p.N) *reinterpret_cast<uint4*>(slot + (long long)rr * p.N + col) = v;
        }
        __syncwarp();
      }
      tc_fence_before();
      // this warp's 32 rows of the tile are stored -> tell the owner (four arrivals per tile)
      __syncwarp();
      if (lane == 0) {
        red_add_release_sys(p.arrived[owner] + p.rank, 1u);
        mbar_arrive(&ctl->acc_empty[acc]);
      }
      if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }

  // ------------------------------------------------------------------ owner-side reduction
  if (threadIdx.x == 0) {
    int ok = ctl->abort_flag ? 0 : 1;
    for (int s = 0; s < p.world && ok; ++s)
      ok = wait_counter_sys(p.arrived[p.rank] + s, p.target, nullptr, p.status, 730) ? 1 : 0;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const long long vecs = (long long)p.rows_per_rank * p.N / 8;
  const long long slot_elems = (long long)p.rows_per_rank * p.N;
  const __nv_bfloat16* base = p.part[p.rank];
  for (long long i = (long long)blockIdx.x * THREADS + threadIdx.x; i < vecs; i += (long long)gridDim.x * THREADS) {
    float accv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) accv[j] = 0.f;
    for (int s = 0; s < p.world; ++s) {
      const uint4 u = ld_v4(base + s * slot_elems + i * 8);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      accv[0] += a.x; accv[1] += a.y; accv[2] += b.x; accv[3] += b.y; accv[4] += c.x; accv[5] += c.y; accv[6] += d.x; accv[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16x2(accv[0], accv[1]); o.y = pack_bf16x2(accv[2], accv[3]); o.z = pack_bf16x2(accv[4], accv[5]); o.w = pack_bf16x2(accv[6], accv[7]);
    reinterpret_cast<uint4*>(p.out)[i] = o;
  }
}

template <typename Kern>
static int configure(Kern kern, bool& done, int smem_bytes = SMEM_BYTES) {
  if (done) return 0;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) { set_last_error("fused GEMM: shared memory opt-in failed: %s", cudaGetErrorString(e)); return (int)e; }
  done = true;
  return 0;
}

}  // namespace fused
}  // namespace dh

using namespace dh;
using namespace dh::fused;

extern "C" {

// Counter increments that one all-gather adds to every row-block counter: the number of
// column slices a row block is pushed in.  A pure function of the shape, so that the fused
// kernel, the stand-alone push and the host agree without exchanging state.
int dh_ag_slices(int M, int K, int world) {
  const int bpr = M / world / BM;
  int slices = 1;
  while (bpr * slices < 32 && (K / (slices * 2)) % 8 == 0 && slices < 64) slices *= 2;
  return slices;
}

static int fill_ag_params(AgParams& p, const char* who, const void* shard, void* const* stage_ptrs, void* const* count_ptrs, void* stage_mc,
                          int M, int K, int rank, int world, unsigned target_base) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("%s: world size %d not in [2, %d]", who, world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (M % (world * BM) != 0 || K % 64 != 0) { set_last_error("%s: M must divide by world*128 and K by 64 (M=%d K=%d)", who, M, K); return (int)cudaErrorInvalidValue; }
  p.shard = (const __nv_bfloat16*)shard;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.stage[i] = i < world ? (__nv_bfloat16*)stage_ptrs[i] : nullptr;
    p.count[i] = i < world ? (uint32_t*)count_ptrs[i] : nullptr;
  }
  p.stage_mc = (__nv_bfloat16*)stage_mc;
  p.d = nullptr;
  p.ldd = 0;
  p.M = M; p.N = 0; p.K = K;
  p.tiles_m = M / BM;
  p.tiles_n = 0;
  p.rank = rank; p.world = world;
  p.rows_per_rank = M / world;
  p.blocks_per_rank = p.rows_per_rank / BM;
  p.copy_ctas = 0;
  p.slices = dh_ag_slices(M, K, world);
  p.target = target_base + (unsigned)p.slices;            // target_base = counter value before this call
  p.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  return 0;
}

// stage_ptrs / count_ptrs: `world` device pointers (index = rank); stage_mc: multicast address
// of the same staging buffer or null.  The local shard has M / world rows (a multiple of 128).
// After the call the local staging buffer holds the gathered [M, K] operand.
int dh_ag_gemm_bf16(const void* shard, void* const* stage_ptrs, void* const* count_ptrs, void* stage_mc, const void* b, int64_t ldb,
                    int b_mn_major, void* d, int64_t ldd, int M, int N, int K, int rank, int world, int copy_ctas, unsigned target_base,
                    int sm_budget, cudaStream_t stream) {
  AgParams p;
  int rc = fill_ag_params(p, "dh_ag_gemm_bf16", shard, stage_ptrs, count_ptrs, stage_mc, M, K, rank, world, target_base);
  if (rc) return rc;
  if ((ldd % 8) != 0) { set_last_error("dh_ag_gemm_bf16: ldd must be a multiple of 8"); return (int)cudaErrorInvalidValue; }
  const CUtensorMap* ta = get_tmap_2d(stage_ptrs[rank], 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, BM, true);
  const CUtensorMap* tb = b_mn_major ? get_tmap_2d(b, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true)
                                     : get_tmap_2d(b, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN, true);
  if (!ta || !tb) return (int)cudaErrorInvalidValue;
  p.d = (__nv_bfloat16*)d;
  p.ldd = ldd;
  p.N = N;
  p.tiles_n = (N + BN - 1) / BN;
  const int sms = dh_sm_count();
  int budget = (sm_budget <= 0 || sm_budget > sms) ? sms : sm_budget;
  if (copy_ctas <= 0) copy_ctas = 8;
  if (copy_ctas > budget / 2) copy_ctas = budget / 2;
  p.copy_ctas = copy_ctas;
  static PerDeviceFlags f0, f1;
  rc = b_mn_major ? configure(ag_gemm_kernel<true>, device_flag(f1)) : configure(ag_gemm_kernel<false>, device_flag(f0));
  if (rc) return rc;
  if (b_mn_major) ag_gemm_kernel<true><<<budget, THREADS, SMEM_BYTES, stream>>>(*ta, *tb, p);
  else ag_gemm_kernel<false><<<budget, THREADS, SMEM_BYTES, stream>>>(*ta, *tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_ag_gemm_bf16 launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Stand-alone all-gather of a row shard into every rank's staging buffer (push only; pair it
// with dh_wait_counters on the consumer's stream).
int dh_ag_push(const void* shard, void* const* stage_ptrs, void* const* count_ptrs, void* stage_mc, int M, int K, int rank, int world,
               int ctas, unsigned target_base, cudaStream_t stream) {
  AgParams p;
  int rc = fill_ag_params(p, "dh_ag_push", shard, stage_ptrs, count_ptrs, stage_mc, M, K, rank, world, target_base);
  if (rc) return rc;
  if (ctas <= 0) ctas = 16;
  ag_push_kernel<<<ctas, 256, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_ag_push launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Row-block-wise reduce-scatter (see rs_reduce_blocks_kernel).  ready: this rank's per-block counters; target: the
// value a complete block reaches in this call; part_ptrs / part_mc as in dh_rs_reduce.
int dh_rs_reduce_blocks(void* const* part_ptrs, const void* part_mc, const void* ready, void* out, int M, int N, int rank, int world,
                        unsigned target, int ctas, cudaStream_t stream) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("dh_rs_reduce_blocks: world size %d not in [2, %d]", world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (M % world != 0 || N % 8 != 0) { set_last_error("dh_rs_reduce_blocks: M must divide by world and N by 8 (M=%d N=%d)", M, N); return (int)cudaErrorInvalidValue; }
  RsbParams p;
  for (int i = 0; i < MAX_RANKS; ++i) p.part[i] = i < world ? (const __nv_bfloat16*)part_ptrs[i] : nullptr;
  p.part_mc = (const __nv_bfloat16*)part_mc;
  p.ready = (const uint32_t*)ready;
  p.out = (__nv_bfloat16*)out;
  p.M = M; p.N = N; p.rank = rank; p.world = world;
  p.blocks = (M / world + BM - 1) / BM;
  if (ctas <= 0) ctas = 32;
  int slices = 1;
  while (p.blocks * slices < ctas && (N / (slices * 2)) % 8 == 0 && slices < 64) slices *= 2;
  p.slices = slices;
  p.target = target;
  p.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  rs_reduce_blocks_kernel<<<ctas, 256, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_rs_reduce_blocks launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

int dh_wait_counters(const void* counters, int n, unsigned target, cudaStream_t stream) {
  wait_counters_kernel<<<1, 256, 0, stream>>>((const uint32_t*)counters, n, target, reinterpret_cast<DeviceStatus*>(dh_status_device_ptr()));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_wait_counters launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// part_ptrs / arrived_ptrs: `world` device pointers.  A is [M, K] local, the result is this
// rank's [M/world, N] shard of the sum over ranks.  target = tiles per owner block x call count.
int dh_gemm_rs_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, int b_mn_major, void* const* part_ptrs,
                    void* const* arrived_ptrs, void* out, int M, int N, int K, int rank, int world, unsigned call_count, int sm_budget,
                    cudaStream_t stream) {
  if (world < 2 || world > MAX_RANKS) { set_last_error("dh_gemm_rs_bf16: world size %d not in [2, %d]", world, MAX_RANKS); return (int)cudaErrorInvalidValue; }
  if (M % (world * BM) != 0 || N % 8 != 0) { set_last_error("dh_gemm_rs_bf16: M must divide by world*128 and N by 8 (M=%d N=%d)", M, N); return (int)cudaErrorInvalidValue; }
  const CUtensorMap* ta = get_tmap_2d(a, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true);
  const CUtensorMap* tb = b_mn_major ? get_tmap_2d(b, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true)
                                     : get_tmap_2d(b, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN, true);
  if (!ta || !tb) return (int)cudaErrorInvalidValue;
  RsParams p;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.part[i] = i < world ? (__nv_bfloat16*)part_ptrs[i] : nullptr;
    p.arrived[i] = i < world ? (uint32_t*)arrived_ptrs[i] : nullptr;
  }
  p.out = (__nv_bfloat16*)out;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.rank = rank; p.world = world;
  p.rows_per_rank = M / world;
  p.blocks_per_rank = p.rows_per_rank / BM;
  p.target = call_count + (unsigned)(p.blocks_per_rank * p.tiles_n * 4);   // call_count = counter value before this call; four warps arrive per tile
  p.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  const int sms = dh_sm_count();
  int budget = (sm_budget <= 0 || sm_budget > sms) ? sms : sm_budget;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int grid = num_tiles < budget ? num_tiles : budget;
  static PerDeviceFlags f0, f1;
  int rc = b_mn_major ? configure(gemm_rs_kernel<true>, device_flag(f1), RS_SMEM_BYTES) : configure(gemm_rs_kernel<false>, device_flag(f0), RS_SMEM_BYTES);
  if (rc) return rc;
  if (b_mn_major) gemm_rs_kernel<true><<<grid, THREADS, RS_SMEM_BYTES, stream>>>(*ta, *tb, p);
  else gemm_rs_kernel<false><<<grid, THREADS, RS_SMEM_BYTES, stream>>>(*ta, *tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_gemm_rs_bf16 launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Reduce-scatter of per-rank partial products that already sit in symmetric memory.
// part_ptrs / flag_ptrs: `world` device pointers (every rank's partial buffer [M][N] and
// announcement words); part_mc: multicast alias of the partial buffers or null; `target` is
// the announcement value of this call (strictly increasing per buffer).
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
