// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   warp 0      : TMA producer  (cp.async.bulk.tensor -> 128B-swizzled shared-memory ring)
//   warp 1      : MMA issuer    (one elected thread issues tcgen05.mma, accumulators in TMEM)
//   warps 2..5  : epilogue      (tcgen05.ld -> registers -> global), overlapped with the
//                               next tile's main loop through two TMEM accumulator buffers
//
// One CTA per SM (or per SM of the caller's budget) walks a grouped tile order that
// keeps a band of A rows and a band of B rows resident in L2.
//
// Operand layouts cover the three products of a linear layer without any transposes
// in memory:  forward  Y = X W^T      (A K-major,  B K-major)
//             dgrad    dX = dY W      (A K-major,  B MN-major)
//             wgrad    dW += dY^T X   (A MN-major, B MN-major, fp32 accumulate in place)
// which is the role of the reference's cuBLASLt wrapper with TN/NN/NT and beta = 1
// (csrc/operators/gemm.cu:3-142) and of torch.matmul / torch.addmm(out=main_grad) on
// its training path (dhellam/operators/layernorm_column.py:32,239,290-292).
#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

#include <cstdlib>

namespace dh {

namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_ACC = 2;
constexpr int ACC_COLS = BN;                 // fp32 columns per accumulator
constexpr int TMEM_COLS = NUM_ACC * ACC_COLS;  // 512 = whole TMEM
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;                   // m-tiles per L2 band

struct __align__(8) Control {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[NUM_ACC];
  uint64_t acc_empty[NUM_ACC];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*control*/;

struct Params {
  void* d;
  int64_t ldd;
  int M, N, K;
  int tiles_m, tiles_n;
  int accumulate;
  int stages, group_m;          // CTA-pair kernel: ring depth in use, m-tiles per L2 band
  DeviceStatus* status;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band = GROUP_M * tiles_n;
  const int g = t / band;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = t - g * band;
  tm = first_m + (r % rows);
  tn = r / rows;
}

// Epilogue of one accumulator row: thread `lane` of an epilogue warp owns output row `row`
// (TMEM lane = row within the tile) and walks the BN columns in chunks of 32.
template <bool OUT_F32>
__device__ __forceinline__ void store_acc_row(const Params& p, int row, bool row_ok, uint32_t taddr, int n_base) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    const int col0 = n_base + c * 32;
    if (col0 >= p.N) break;          // uniform across the warp
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    if (!row_ok) continue;
    if (OUT_F32) {
      float* dst = reinterpret_cast<float*>(p.d) + (int64_t)row * p.ldd + col0;
      if (col0 + 32 <= p.N) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                 __uint_as_float(r[4 * j + 3]));
          float4* q = reinterpret_cast<float4*>(dst) + j;
          if (p.accumulate) {
            float4 o = *q;
            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
          }
          *q = v;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col0 + j < p.N) {
            float v = __uint_as_float(r[j]);
            dst[j] = p.accumulate ? dst[j] + v : v;
          }
        }
      }
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.d) + (int64_t)row * p.ldd + col0;
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
  }
}

template <bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  Control* ctl = reinterpret_cast<Control*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&ctl->acc_full[a], 1);
      mbar_init(&ctl->acc_empty[a], 4);   // one arrive per epilogue warp
    }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 100)) { ok = false; break; }
          mbar_expect_tx(&ctl->full[s], STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmap_a, &ctl->full[s], m0 + 64 * j, k0);
          } else {
            tma_load_2d(a_dst, &tmap_a, &ctl->full[s], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmap_b, &ctl->full[s], n0 + 64 * j, k0);
          } else {
            tma_load_2d(b_dst, &tmap_b, &ctl->full[s], k0, n0);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&ctl->acc_empty[acc], acc_ph ^ 1, abort_flag, p.status, 200)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, p.status, 201)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // K-major: 16 elements = 32 bytes further inside the 128-byte swizzle row;
            //          8-row groups 1024 bytes apart.
            // MN-major: each group of 8 k-rows is one 1024-byte swizzle atom; 64-element
            //          column blocks are BK*128 bytes apart.
            const uint64_t adesc = A_MN ? umma_smem_desc(a_base + kk * 2048, BK * 128, 1024)
                                        : umma_smem_desc(a_base + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + kk * 2048, BK * 128, 1024)
                                        : umma_smem_desc(b_base + kk * 32, 16, 1024);
            umma_bf16(tmem_acc, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&ctl->empty[s]);   // frees the stage once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&ctl->acc_full[acc]);
        if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;           // TMEM lanes [32*quarter, 32*quarter+32)
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      if (!mbar_wait(&ctl->acc_full[acc], acc_ph, abort_flag, p.status, 300)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const bool row_ok = row < p.M;
      store_acc_row<OUT_F32>(p, row, row_ok, taddr, tn * BN);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[acc]);
      if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, bool OUT_F32>
static int launch(const CUtensorMap* ta, const CUtensorMap* tb, const Params& p, int grid, cudaStream_t stream) {
  auto kern = gemm_kernel<A_MN, B_MN, OUT_F32>;
  static PerDeviceFlags configured_on;
  bool& configured = device_flag(configured_on);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) {
      set_last_error("cudaFuncSetAttribute(smem=%d) failed: %s", SMEM_BYTES, cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  kern<<<grid, THREADS, SMEM_BYTES, stream>>>(*ta, *tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("gemm launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}


// ---------------------------------------------------------------------------------------
// CTA-pair variant (tcgen05 cta_group::2).  Two CTAs of a cluster share one 256 x 256
// output tile: each loads its own 128 rows of A and its own 128-column half of B, the
// leader's elected thread issues M = 256 MMAs that read both CTAs' shared memory, and each
// CTA ends up with its own 128 accumulator rows in its own TMEM.  Per CTA and k-block this
// moves 32 KiB through TMA instead of 48 KiB and leaves room for a deeper ring, which is
// what the single-CTA kernel lacks at large shapes (its tensor pipe idles ~20% of the time
// waiting for operands).
//
// Barrier protocol (all barriers exist in both CTAs at the same offsets):
//   full[s]      leader only; the leader's producer arms it with the bytes of BOTH CTAs,
//                the peer's TMA credits its bytes to the leader's barrier (cta_group::2 form)
//   empty[s]     one per CTA; the MMA thread commits to its own and to the peer's copy
//   acc_full[a]  one per CTA, committed the same way
//   acc_empty[a] leader only; 4 epilogue warps of each CTA arrive (count 8)
// A cluster barrier after setup keeps remote arrivals from reaching an uninitialised
// barrier, and one before the TMEM release keeps either CTA from leaving while the other
// can still signal it.
// ---------------------------------------------------------------------------------------
namespace pair {
constexpr int STAGES2 = 7;                        // ring slots allocated; Params.stages of them are used
constexpr int TILE_M = 2 * BM;                     // 256 rows per CTA pair
constexpr int BN_HALF = BN / 2;                    // B columns loaded by each CTA
constexpr int A2_STAGE_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B2_STAGE_BYTES = BN_HALF * BK * 2;   // 16 KiB
constexpr int STAGE2_BYTES = A2_STAGE_BYTES + B2_STAGE_BYTES;

struct __align__(8) Control2 {
  uint64_t full[STAGES2];
  uint64_t empty[STAGES2];
  uint64_t acc_full[NUM_ACC];
  uint64_t acc_empty[NUM_ACC];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 1024 + 256;

__device__ __forceinline__ void tile_coords2(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int band = group_m * tiles_n;
  const int g = t / band;
  const int first_m = g * group_m;
  const int rows = min(group_m, tiles_m - first_m);
  const int r = t - g * band;
  tm = first_m + (r % rows);
  tn = r / rows;
}

template <bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES2 * A2_STAGE_BYTES;
  Control2* ctl = reinterpret_cast<Control2*>(smem + STAGES2 * STAGE2_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;      // tiles of 256 x 256
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&ctl->acc_full[a], 1);
      mbar_init(&ctl->acc_empty[a], 8);
    }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_2sm(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        int tm, tn;
        tile_coords2(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
        const int m0 = tm * TILE_M + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * BN_HALF;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 110)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(&ctl->full[s], 2 * STAGE2_BYTES);
          const uint32_t full_leader = mapa_u32(smem_u32(&ctl->full[s]), 0);
          uint8_t* a_dst = sA + s * A2_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B2_STAGE_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_2sm(a_dst + j * (BK * 128), &tmap_a, full_leader, m0 + 64 * j, k0);
          } else {
            tma_load_2d_2sm(a_dst, &tmap_a, full_leader, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN_HALF / 64; ++j) tma_load_2d_2sm(b_dst + j * (BK * 128), &tmap_b, full_leader, n0 + 64 * j, k0);
          } else {
            tma_load_2d_2sm(b_dst, &tmap_b, full_leader, k0, n0);
          }
          if (++s == p.stages) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait<true>(&ctl->acc_empty[acc], acc_ph ^ 1, abort_flag, p.status, 210)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, p.status, 211)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A2_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B2_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? umma_smem_desc(a_base + kk * 2048, BK * 128, 1024)
                                        : umma_smem_desc(a_base + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + kk * 2048, BK * 128, 1024)
                                        : umma_smem_desc(b_base + kk * 32, 16, 1024);
            umma_bf16_2sm(tmem_acc, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          const uint32_t e = smem_u32(&ctl->empty[s]);
          umma_commit_2sm(mapa_u32(e, 0));
          umma_commit_2sm(mapa_u32(e, 1));
          if (++s == p.stages) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        const uint32_t f = smem_u32(&ctl->acc_full[acc]);
        umma_commit_2sm(mapa_u32(f, 0));
        umma_commit_2sm(mapa_u32(f, 1));
        if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      int tm, tn;
      tile_coords2(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      if (!mbar_wait(&ctl->acc_full[acc], acc_ph, abort_flag, p.status, 310)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * TILE_M + (int)rank * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      store_acc_row<OUT_F32>(p, row, row < p.M, taddr, tn * BN);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&ctl->acc_empty[acc], 0);
      if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, bool OUT_F32>
static int launch_pair(const CUtensorMap* ta, const CUtensorMap* tb, const Params& p, int pairs, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT_F32>;
  static PerDeviceFlags configured_on;
  bool& configured = device_flag(configured_on);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
    if (e != cudaSuccess) {
      set_last_error("cudaFuncSetAttribute(smem=%d) failed: %s", SMEM2_BYTES, cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM2_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *ta, *tb, p);
  if (e != cudaSuccess) set_last_error("pair gemm launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}
}  // namespace pair

// 0 = choose per problem, 1 = single-CTA kernel only, 2 = CTA-pair kernel whenever M > 128.
static int g_gemm_mode = -1;
static int gemm_mode() {
  if (g_gemm_mode < 0) {
    const char* e = getenv("DHELLAM_GEMM_MODE");
    g_gemm_mode = e ? atoi(e) : 0;
  }
  return g_gemm_mode;
}

}  // namespace gemm
}  // namespace dh

extern "C" void dh_gemm_set_mode(int mode) { dh::gemm::g_gemm_mode = mode; }

extern "C" int dh_gemm_bf16(const void* a, int64_t lda, int a_mn_major, const void* b, int64_t ldb, int b_mn_major, void* d,
                            int64_t ldd, int d_fp32, int accumulate, int M, int N, int K, int epilogue, int sm_budget,
                            cudaStream_t stream) {
  using namespace dh;
  using namespace dh::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (epilogue != 0) {
    set_last_error("dh_gemm_bf16: unknown epilogue %d", epilogue);
    return (int)cudaErrorInvalidValue;
  }
  if (accumulate && !d_fp32) {
    set_last_error("dh_gemm_bf16: accumulate needs an fp32 output");
    return (int)cudaErrorInvalidValue;
  }
  const int out_vec = d_fp32 ? 4 : 8;
  if ((ldd % out_vec) != 0 || (reinterpret_cast<uintptr_t>(d) & 15) != 0) {
    set_last_error("dh_gemm_bf16: output must be 16-byte aligned with ldd a multiple of %d", out_vec);
    return (int)cudaErrorInvalidValue;
  }
  const int mode = gemm_mode();
  const bool use_pair = mode != 1 && M > BM;
  const int b_rows = use_pair ? pair::BN_HALF : BN;
  static int pair_stages = 0, pair_group = 0;
  if (pair_stages == 0) {
    const char* e = getenv("DHELLAM_GEMM_STAGES");
    pair_stages = e ? atoi(e) : 6;
    if (pair_stages < 2 || pair_stages > pair::STAGES2) pair_stages = 6;
    e = getenv("DHELLAM_GEMM_GROUP");
    pair_group = e ? atoi(e) : 8;        // 8 x 256 rows per L2 band measured best at the large shapes
    if (pair_group < 1) pair_group = 8;
  }
  // K-major operand: tensor (inner K, outer rows); MN-major operand: (inner rows, outer K).
  const CUtensorMap* ta = a_mn_major ? get_tmap_2d(a, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, true)
                                     : get_tmap_2d(a, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true);
  const CUtensorMap* tb = b_mn_major ? get_tmap_2d(b, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true)
                                     : get_tmap_2d(b, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, b_rows, true);
  if (!ta || !tb) return (int)cudaErrorInvalidValue;

  Params p;
  p.d = d;
  p.ldd = ldd;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tiles_m = use_pair ? (M + pair::TILE_M - 1) / pair::TILE_M : (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.accumulate = accumulate;
  p.stages = pair_stages;
  p.group_m = pair_group;
  p.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  const int sms = dh_sm_count();
  int budget = (sm_budget <= 0 || sm_budget > sms) ? sms : sm_budget;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int sel = (a_mn_major ? 4 : 0) | (b_mn_major ? 2 : 0) | (d_fp32 ? 1 : 0);
  if (use_pair) {
    int pairs = budget / 2;
    if (pairs < 1) pairs = 1;
    if (pairs > num_tiles) pairs = num_tiles;
    switch (sel) {
      case 0: return pair::launch_pair<false, false, false>(ta, tb, p, pairs, stream);
      case 1: return pair::launch_pair<false, false, true>(ta, tb, p, pairs, stream);
      case 2: return pair::launch_pair<false, true, false>(ta, tb, p, pairs, stream);
      case 3: return pair::launch_pair<false, true, true>(ta, tb, p, pairs, stream);
      case 4: return pair::launch_pair<true, false, false>(ta, tb, p, pairs, stream);
      case 5: return pair::launch_pair<true, false, true>(ta, tb, p, pairs, stream);
      case 6: return pair::launch_pair<true, true, false>(ta, tb, p, pairs, stream);
      default: return pair::launch_pair<true, true, true>(ta, tb, p, pairs, stream);
    }
  }
  const int grid = num_tiles < budget ? num_tiles : budget;
  switch (sel) {
    case 0: return launch<false, false, false>(ta, tb, p, grid, stream);
    case 1: return launch<false, false, true>(ta, tb, p, grid, stream);
    case 2: return launch<false, true, false>(ta, tb, p, grid, stream);
    case 3: return launch<false, true, true>(ta, tb, p, grid, stream);
    case 4: return launch<true, false, false>(ta, tb, p, grid, stream);
    case 5: return launch<true, false, true>(ta, tb, p, grid, stream);
    case 6: return launch<true, true, false>(ta, tb, p, grid, stream);
    default: return launch<true, true, true>(ta, tb, p, grid, stream);
  }
}
