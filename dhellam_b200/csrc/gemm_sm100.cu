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
#include "comm_device.cuh"
#include "ptx.cuh"
#include "tmap.h"

#include <cstdlib>
#include <cstring>

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
// moves 32 KiB through TMA instead of 48 KiB, which leaves room for a six-slot ring.
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
//
// Epilogue.  Each epilogue warp drains its 32 accumulator rows in chunks of 128 bytes per row
// (64 bf16 or 32 fp32 columns): tcgen05.ld -> registers -> a 4 KiB swizzled staging tile in
// shared memory -> one TMA store of a 32-row box (two staging tiles per warp, so the store of
// chunk c overlaps the TMEM read of chunk c+1).  Whole 128-byte lines reach L2 instead of 32
// scattered 16-byte pieces per store instruction.  An accumulating fp32 output (a weight
// gradient added into main_grad) uses the reducing form of the bulk store: L2 adds the tile
// in place and nothing is read back into the SM.  Because that add is atomic, such a GEMM may
// also be split along K ("split_k" work items per tile, each adding its share), which fills
// the last wave when the tile count is a poor multiple of the SM pairs.
//
// Collective hooks (tensor-parallel sequence all-gather in front, reduce-scatter behind):
//   wait_count   the A operand is a staging buffer that peers are still filling; before the
//                first load of a 128-row block the producer waits (bounded) for that block's
//                arrival counter in LOCAL memory and then reads local memory only;
//   sig[]        after a warp's 32 rows of a tile are stored (store completion waited for),
//                it bumps the row block's counter on the rank that owns those rows, so the
//                owner's reduction kernel can start on a block as soon as every rank has
//                delivered it instead of after every rank's whole GEMM;
//   perm_mode    visiting order of the 256-row tile rows: 1 = own shard first, then the other
//                ranks' shards row block by row block (the order in which a simultaneous push
//                from all ranks completes them); 2 = row block by row block over all owners.
// ---------------------------------------------------------------------------------------
namespace pair {
constexpr int RING = 6;                            // ring slots
constexpr int TILE_M = 2 * BM;                     // 256 rows per CTA pair
constexpr int BN_HALF = BN / 2;                    // B columns loaded by each CTA
constexpr int A2_STAGE_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B2_STAGE_BYTES = BN_HALF * BK * 2;   // 16 KiB
constexpr int STAGE2_BYTES = A2_STAGE_BYTES + B2_STAGE_BYTES;
constexpr int EPI_TILE_BYTES = 32 * 128;           // 32 rows x 128 bytes
constexpr int EPI_BYTES = 4 * 2 * EPI_TILE_BYTES;  // 4 warps x 2 staging tiles = 32 KiB
constexpr long long PEER_WAIT_CYCLES = 40000000000ll;   // ~20 s: a peer may still be starting up

struct __align__(8) Control2 {
  uint64_t full[RING];
  uint64_t empty[RING];
  uint64_t acc_full[NUM_ACC];
  uint64_t acc_empty[NUM_ACC];
  uint32_t tmem_base;
  int abort_flag;
  int comm_flag;
  uint32_t epi_done[4];            // tiles whose stores are complete, per epilogue warp (read by the signal warp)
};
constexpr int SIGNAL_THREADS = 32;                 // one more warp when the GEMM signals finished row blocks
constexpr int COMM_THREADS = 64;                   // two communication warps per CTA in the COMM form of the kernel
constexpr int SMEM2_BYTES = RING * STAGE2_BYTES + EPI_BYTES + 1024 + 256;

struct PairParams {
  int M, N, K;
  int tiles_m, tiles_n;
  int stages, group_m;
  int split_k, kb_per_split;           // work item = (tile, k range)
  int reduce_add;                      // epilogue: 1 = add into the output (bulk reduce), 0 = plain store
  // collective hooks (all off when null / 0)
  const uint32_t* wait_count;          // arrival counters of A's 128-row blocks (local memory)
  uint32_t wait_target;
  uint32_t* sig[8];                    // per-owner arrays of row-block completion counters
  int sig_bpr;                         // 128-row blocks per owner
  int perm_mode, perm_world, perm_rank;
  long long wait_budget;               // cycles for the barriers inside the CTA
  unsigned start_id;                   // != 0: announce "every CTA of this launch is resident" (g_start_flag = start_id)
  DeviceStatus* status;
  // grouped (ragged) form for mixture-of-experts layers: `groups` experts share one launch.
  //   group_mode 1  rows grouped: A and D rows are expert-major with region starts group_offs[e] (multiples of 256,
  //                 device memory: the sizes never reach the host); B is the stack of the experts' weights
  //   group_mode 2  contraction grouped (weight gradients): D is the stack of per-expert [M, N] outputs, the
  //                 contraction of expert e runs over rows [group_offs[e], group_offs[e+1]) of A and B
  int group_mode, groups;
  const int* group_offs;
  // collective carried by the communication warps (COMM form of the kernel only):
  // 0 none, 1 = push this rank's shard of the gathered A operand, 2 = reduce this rank's rows of the partial products
  int comm_kind;
  comm::PushJob push;
  comm::ReduceJob reduce;
};

// "Every CTA of launch `id` is resident": a kernel on another stream that spins on this GEMM's row-block signals
// must not start before that, because with a static tile assignment a CTA pair that finds no room on its SMs
// (taken by the spinning kernel's CTAs) would leave exactly the tiles undone that the spinning kernel waits for.
// The consumer's stream runs a one-CTA wait on g_start_flag >= id in front of its kernel.
__device__ unsigned g_start_count = 0;
__device__ unsigned g_start_flag = 0;

__device__ __forceinline__ int perm_tile_m(int i, const PairParams& p) {
  if (p.perm_mode == 0) return i;
  const int per = p.tiles_m / p.perm_world;
  if (p.perm_mode == 1) {
    if (i < per) return p.perm_rank * per + i;
    const int k = i - per, w1 = p.perm_world - 1;
    const int j = k / w1, r = k - j * w1;
    return ((p.perm_rank + 1 + r) % p.perm_world) * per + j;
  }
  const int j = i / p.perm_world, r = i - j * p.perm_world;
  return ((p.perm_rank + 1 + r) % p.perm_world) * per + j;
}

// Work item -> (tile row, tile column, first k-block, end k-block) plus, in the grouped forms, the expert.
struct Item {
  int tm, tn, kb0, kb1;
  int b_off;            // added to B's outer coordinate (expert's weight inside the stack)
  int d_row_off;        // added to D's row coordinate (expert's output inside the stack)
};

__device__ __forceinline__ int num_items_of(const PairParams& p, int& num_tiles) {
  if (p.group_mode == 1) {
    num_tiles = (p.group_offs[p.groups] / TILE_M) * p.tiles_n;       // rows in use are known on the device only
    return num_tiles;
  }
  if (p.group_mode == 2) {
    num_tiles = p.groups * p.tiles_m * p.tiles_n;
    return num_tiles;
  }
  num_tiles = p.tiles_m * p.tiles_n;
  return num_tiles * p.split_k;
}

__device__ __forceinline__ Item item_coords(int item, const PairParams& p, int num_tiles, int num_kb) {
  Item it;
  it.b_off = 0;
  it.d_row_off = 0;
  if (p.group_mode == 2) {
    const int per = p.tiles_m * p.tiles_n;
    const int e = item / per;
    const int t = item - e * per;
    it.tm = t % p.tiles_m;
    it.tn = t / p.tiles_m;
    it.kb0 = p.group_offs[e] / BK;
    it.kb1 = p.group_offs[e + 1] / BK;
    it.d_row_off = e * p.M;
    return it;
  }
  const int tiles_m = p.group_mode == 1 ? num_tiles / p.tiles_n : p.tiles_m;
  const int ks = item / num_tiles;
  const int t = item - ks * num_tiles;
  const int band = p.group_m * p.tiles_n;
  const int g = t / band;
  const int first_m = g * p.group_m;
  const int rows = min(p.group_m, tiles_m - first_m);
  const int r = t - g * band;
  it.tm = perm_tile_m(first_m + (r % rows), p);
  it.tn = r / rows;
  it.kb0 = ks * p.kb_per_split;
  it.kb1 = min(num_kb, it.kb0 + p.kb_per_split);
  if (p.group_mode == 1) {
    const int row = it.tm * TILE_M;
    int e = 0;
    while (e + 1 < p.groups && row >= p.group_offs[e + 1]) ++e;
    it.b_off = e;                                  // expert index; scaled by the caller (B's major decides by what)
  }
  return it;
}

__device__ __forceinline__ bool wait_block_counter(const uint32_t* c, uint32_t want, volatile int* abort_flag, DeviceStatus* st, int where) {
  if (ld_acquire_sys(c) >= want) return true;
  const long long t0 = clock64();
  while (true) {
    if (ld_acquire_sys(c) >= want) return true;
    __nanosleep(100);
    if (*abort_flag) return false;
    if (clock64() - t0 > PEER_WAIT_CYCLES) {
      *abort_flag = 1;
      report_error(st, ERR_FLAG_TIMEOUT, where, (int)want);
      return false;
    }
  }
}

// COMM = true adds two communication warps to every CTA (256 threads instead of 192): they carry the
// collective that belongs to this GEMM (the push of this rank's shard of the gathered A operand, or the
// row-block-wise reduction of the partial products this GEMM and its peers signal), spread evenly over all
// SMs, so that compute and transfer are ONE kernel and no SM carries more communication work than another.
template <bool A_MN, bool B_MN, bool OUT_F32, bool COMM>
__global__ void __launch_bounds__((COMM ? THREADS + COMM_THREADS : THREADS) + SIGNAL_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_d, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // layout: A ring | B ring | epilogue staging | control, sized for the ring depth in use (p.stages), so that a
  // shallower ring really leaves shared memory to small kernels that share the SM
  uint8_t* sA = smem;
  uint8_t* sB = smem + p.stages * A2_STAGE_BYTES;
  uint8_t* sEpi = smem + p.stages * STAGE2_BYTES;
  Control2* ctl = reinterpret_cast<Control2*>(smem + p.stages * STAGE2_BYTES + EPI_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  int num_tiles;                                    // tiles of 256 x 256
  const int num_items = num_items_of(p, num_tiles);
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RING; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(&ctl->acc_full[a], 1);
      mbar_init(&ctl->acc_empty[a], 8);
    }
    ctl->abort_flag = 0;
    ctl->comm_flag = 1;
    for (int q = 0; q < 4; ++q) ctl->epi_done[q] = 0;
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
  if (p.start_id != 0 && threadIdx.x == 0) {
    if (atomicAdd(&g_start_count, 1u) + 1u == gridDim.x) {       // the last CTA to become resident
      atomicExch(&g_start_count, 0u);
      __threadfence();
      atomicMax(&g_start_flag, p.start_id);
    }
  }

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int ready_block = -1;
      for (int it = pair_id; it < num_items && ok; it += num_pairs) {
        const Item im = item_coords(it, p, num_tiles, num_kb);
        const int tm = im.tm, tn = im.tn, kb0 = im.kb0, kb1 = im.kb1;
        const int m0 = tm * TILE_M + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * BN_HALF;
        // grouped rows: B is the stack of the experts' weights ([groups * N, K] K-major, or [groups * K, N] MN-major)
        const int bn_off = (p.group_mode == 1 && !B_MN) ? im.b_off * p.N : 0;
        const int bk_off = (p.group_mode == 1 && B_MN) ? im.b_off * p.K : 0;
        if (p.wait_count != nullptr) {
          const int blk = m0 / BM;
          if (blk != ready_block && m0 < p.M) {
            if (!wait_block_counter(p.wait_count + blk, p.wait_target, abort_flag, p.status, 115)) { ok = false; break; }
            fence_proxy_async_all();                // peers' stores -> visible to the TMA reads below
            ready_block = blk;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, p.status, 110, p.wait_budget)) { ok = false; break; }
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
            for (int j = 0; j < BN_HALF / 64; ++j) tma_load_2d_2sm(b_dst + j * (BK * 128), &tmap_b, full_leader, n0 + 64 * j, k0 + bk_off);
          } else {
            tma_load_2d_2sm(b_dst, &tmap_b, full_leader, k0, n0 + bn_off);
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
      for (int it = pair_id; it < num_items && ok; it += num_pairs) {
        const Item im = item_coords(it, p, num_tiles, num_kb);
        const int kb0 = im.kb0, kb1 = im.kb1;
        if (kb0 >= kb1) continue;                       // an expert without rows: nothing to add (all roles skip the item)
        if (!mbar_wait<true>(&ctl->acc_empty[acc], acc_ph ^ 1, abort_flag, p.status, 210, p.wait_budget)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, p.status, 211, p.wait_budget)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * A2_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B2_STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? umma_smem_desc(a_base + kk * 2048, BK * 128, 1024)
                                        : umma_smem_desc(a_base + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(b_base + kk * 2048, BK * 128, 1024)
                                        : umma_smem_desc(b_base + kk * 32, 16, 1024);
            umma_bf16_2sm(tmem_acc, adesc, bdesc, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
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
  } else if (warp == (COMM ? 8 : 6)) {
    // ------------------------------ signal warp (both CTAs; launched only with row-block signals) -----------
    // Tells the rank that owns a row block that this CTA's 128 rows of a tile are in memory.  The system-scope
    // fence and the remote reduction take microseconds; here they delay nobody: the epilogue warps only publish
    // "stores of tile k complete" in shared memory and go on.
    if (lane == 0 && p.sig[0] != nullptr) {
      // One system-scope fence per BATCH of finished tiles, then one relaxed remote reduction per tile: the fence
      // (microseconds) is the only part that waits, and a backlog costs one fence, not one per tile.
      uint32_t done = 0;                            // tiles of this CTA signalled so far
      int it = pair_id;                             // work item of tile number `done`
      bool ok = true;
      while (ok) {
        while (it < num_items) {                    // skip items without work (no tile, no signal)
          const Item im = item_coords(it, p, num_tiles, num_kb);
          if (im.kb0 < im.kb1) break;
          it += num_pairs;
        }
        if (it >= num_items) break;
        uint32_t ready = done;
        const long long t0 = clock64();
        while (true) {
          ready = ld_acquire_cta_u32(&ctl->epi_done[0]);
          for (int q = 1; q < 4; ++q) ready = min(ready, ld_acquire_cta_u32(&ctl->epi_done[q]));
          if (ready > done) break;
          __nanosleep(64);
          if (*abort_flag) { ok = false; break; }
          if (clock64() - t0 > p.wait_budget) {
            *abort_flag = 1;
            report_error(p.status, ERR_FLAG_TIMEOUT, 330, (int)done);
            ok = false;
            break;
          }
        }
        if (!ok) break;
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        while (done < ready && it < num_items) {
          const Item im = item_coords(it, p, num_tiles, num_kb);
          it += num_pairs;
          if (im.kb0 >= im.kb1) continue;
          const int m0 = im.tm * TILE_M + (int)rank * BM;
          if (m0 < p.M) {
            const int blk = m0 / BM;
            red_add_relaxed_sys(p.sig[blk / p.sig_bpr] + (blk % p.sig_bpr), 1u);
          }
          ++done;
        }
      }
    }
    __syncwarp();
  } else if (COMM && warp >= 6) {
    // ------------------------------ communication warps (both CTAs) -----------
    const int tid = (int)threadIdx.x - THREADS;
    auto group_sync = [] { asm volatile("bar.sync 1, 64;" ::: "memory"); };
    if (p.comm_kind == 1) {
      comm::push_rows(p.push, (int)blockIdx.x, (int)gridDim.x, tid, COMM_THREADS, group_sync);
    } else if (p.comm_kind == 2) {
      comm::reduce_rows(p.reduce, (int)blockIdx.x, (int)gridDim.x, tid, COMM_THREADS, group_sync, &ctl->comm_flag, p.status, 665);
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------
    constexpr int CH_COLS = OUT_F32 ? 32 : 64;      // columns per 128-byte chunk
    constexpr int NCH = BN / CH_COLS;
    const int quarter = warp & 3;
    uint8_t* stg = sEpi + quarter * (2 * EPI_TILE_BYTES);
    int acc = 0;
    uint32_t acc_ph = 0;
    uint32_t cc = 0;                                // running chunk count -> staging tile parity
    bool owed = false;                              // a tile's completion has not been published yet (lane 0)
    uint32_t published = 0;
    bool ok = true;
    for (int it = pair_id; it < num_items && ok; it += num_pairs) {
      const Item im = item_coords(it, p, num_tiles, num_kb);
      const int tm = im.tm, tn = im.tn;
      if (im.kb0 >= im.kb1) continue;
      if (!mbar_wait(&ctl->acc_full[acc], acc_ph, abort_flag, p.status, 310, p.wait_budget)) { ok = false; break; }
      tc_fence_after();
      const int row0 = tm * TILE_M + (int)rank * BM + quarter * 32;     // first of this warp's 32 output rows
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      int chunks_done = 0;
#pragma unroll 1
      for (int c = 0; c < NCH; ++c) {
        const int col0 = tn * BN + c * CH_COLS;
        if (col0 >= p.N) break;                     // uniform across the warp
        ++chunks_done;
        uint32_t r[OUT_F32 ? 32 : 64];
        tmem_ld32(taddr + c * CH_COLS, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        if (!OUT_F32) tmem_ld32(taddr + c * CH_COLS + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        // the store that read this staging tile two chunks ago must have finished reading it
        if (lane == 0) tma_store_wait_read<1>();
        tmem_ld_wait();
        __syncwarp();
        if (row0 < p.M) {
          uint8_t* tile = stg + (cc & 1) * EPI_TILE_BYTES;
          uint8_t* rowp = tile + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v;
            if (OUT_F32) {
              v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            } else {
              v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            }
            // 128-byte swizzle: 16-byte chunk j of row `lane` sits at chunk position j ^ (lane & 7)
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (p.reduce_add) tma_reduce_add_2d(&tmap_d, tile, col0, row0 + im.d_row_off);
            else tma_store_2d(&tmap_d, tile, col0, row0 + im.d_row_off);
            tma_store_commit();
          }
          ++cc;
        }
      }
      // the accumulator has been read out: hand the TMEM buffer back before the stores drain
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&ctl->acc_empty[acc], 0);
      if (p.sig[0] != nullptr) {
        // Publish "the stores of the PREVIOUS tile are complete" to the signal warp: after the stores of this tile
        // have been issued, waiting for all but the newest NCH groups completes the previous tile without stalling.
        if (lane == 0) {
          if (owed) {
            if (chunks_done == NCH) tma_store_wait<NCH>();
            else tma_store_wait<0>();
            fence_proxy_async_all();
            st_release_cta_u32(&ctl->epi_done[quarter], ++published);
          }
          owed = true;
        }
        __syncwarp();
      }
      if (++acc == NUM_ACC) { acc = 0; acc_ph ^= 1; }
    }
    if (lane == 0) {
      tma_store_wait<0>();                          // shared memory must outlive the bulk stores
      if (owed) {
        fence_proxy_async_all();
        st_release_cta_u32(&ctl->epi_done[quarter], ++published);
      }
    }
    __syncwarp();
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

template <bool A_MN, bool B_MN, bool OUT_F32, bool COMM = false>
static int launch_pair(const CUtensorMap* ta, const CUtensorMap* tb, const CUtensorMap* td, const PairParams& p, int pairs,
                       cudaStream_t stream) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT_F32, COMM>;
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
  cfg.blockDim = dim3((COMM ? THREADS + COMM_THREADS : THREADS) + (p.sig[0] != nullptr ? SIGNAL_THREADS : 0));
  cfg.dynamicSmemBytes = SMEM2_BYTES - (RING - p.stages) * STAGE2_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *ta, *tb, *td, p);
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

namespace dh {
namespace gemm {

// Work items per tile along K for an accumulating (atomic-add) output: the smallest split that
// brings the last wave's occupancy above 93 %, or 1.  DHELLAM_GEMM_SPLITK = 0 / 1 turns it off,
// = n forces n.
static int g_splitk_override = -1;     // dh_gemm_set_splitk: -1 = follow the environment / heuristic

static int choose_split_k(int tiles, int pairs, int num_kb) {
  static int forced = -1;
  if (g_splitk_override >= 0) {
    int b = g_splitk_override < 1 ? 1 : g_splitk_override;
    while (b > 1 && num_kb / b < 2) --b;
    return b;
  }
  if (forced < 0) {
    const char* e = getenv("DHELLAM_GEMM_SPLITK");
    forced = e ? atoi(e) : 0;
    if (forced < 0) forced = 0;
    if (e && forced == 0) forced = 1;
  }
  int best = 1;
  if (forced >= 1) {
    best = forced;
  } else {
    auto eff = [&](int s) { const long long it = (long long)tiles * s; return (double)it / (double)(((it + pairs - 1) / pairs) * pairs); };
    double be = eff(1);
    if (be < 0.93) {
      for (int s = 2; s <= 4; ++s) {
        const double e2 = eff(s);
        if (e2 > be + 0.03) { be = e2; best = s; }
      }
    }
  }
  while (best > 1 && num_kb / best < 16) --best;       // keep every share long enough to amortise its prologue
  return best < 1 ? 1 : best;
}

struct SyncArgs {
  const void* wait_count = nullptr;
  unsigned wait_target = 0;
  void* const* sig_ptrs = nullptr;
  int sig_bpr = 0;
  int perm_mode = 0, world = 1, rank = 0;
  int comm_kind = 0;                       // collective carried by the kernel's own communication warps
  unsigned start_id = 0;                   // announce residency under this id (0 = no announcement)
  const comm::PushJob* push = nullptr;
  const comm::ReduceJob* reduce = nullptr;
};

static int gemm_impl(const void* a, int64_t lda, int a_mn_major, const void* b, int64_t ldb, int b_mn_major, void* d, int64_t ldd,
                     int d_fp32, int accumulate, int M, int N, int K, int sm_budget, const SyncArgs& sy, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (accumulate && !d_fp32) {
    set_last_error("dh_gemm_bf16: accumulate needs an fp32 output");
    return (int)cudaErrorInvalidValue;
  }
  const int out_vec = d_fp32 ? 4 : 8;
  if ((ldd % out_vec) != 0 || (reinterpret_cast<uintptr_t>(d) & 15) != 0) {
    set_last_error("dh_gemm_bf16: output must be 16-byte aligned with ldd a multiple of %d", out_vec);
    return (int)cudaErrorInvalidValue;
  }
  const bool hooks = sy.wait_count != nullptr || sy.sig_ptrs != nullptr || sy.perm_mode != 0;
  const int mode = gemm_mode();
  const bool use_pair = (mode != 1 && M > BM) || hooks;
  if (hooks && sy.world > 8) {
    set_last_error("dh_gemm_bf16_sync: at most 8 ranks");
    return (int)cudaErrorInvalidValue;
  }
  const int b_rows = use_pair ? pair::BN_HALF : BN;
  static int pair_stages = 0, pair_group = 0;
  if (pair_stages == 0) {
    const char* e = getenv("DHELLAM_GEMM_STAGES");
    pair_stages = e ? atoi(e) : pair::RING;
    if (pair_stages < 2 || pair_stages > pair::RING) pair_stages = pair::RING;
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
  const int sms = dh_sm_count();
  int budget = (sm_budget <= 0 || sm_budget > sms) ? sms : sm_budget;
  const int sel = (a_mn_major ? 4 : 0) | (b_mn_major ? 2 : 0) | (d_fp32 ? 1 : 0);
  DeviceStatus* status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());

  if (use_pair) {
    using namespace pair;
    PairParams p;
    memset(&p, 0, sizeof(p));
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + TILE_M - 1) / TILE_M;
    p.tiles_n = (N + BN - 1) / BN;
    // A GEMM that other resident kernels wait on (row-block signals) or that waits on them must never be kept off
    // an SM by those kernels' CTAs: with a static tile assignment a CTA pair that cannot become resident leaves
    // its tiles undone while the kernels that hold its shared memory spin on exactly those tiles.  One ring stage
    // less leaves 32 KB per SM, room for every small CTA that can share it.
    p.stages = hooks && pair_stages == RING ? RING - 1 : pair_stages;
    p.group_m = pair_group;
    p.status = status;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = (K + BK - 1) / BK;
    int pairs = budget / 2;
    if (pairs < 1) pairs = 1;
    p.reduce_add = accumulate ? 1 : 0;
    p.split_k = accumulate ? choose_split_k(num_tiles, pairs, num_kb) : 1;
    p.kb_per_split = (num_kb + p.split_k - 1) / p.split_k;
    while (p.split_k > 1 && (p.split_k - 1) * p.kb_per_split >= num_kb) --p.split_k;   // no empty share
    p.wait_count = reinterpret_cast<const uint32_t*>(sy.wait_count);
    p.wait_target = sy.wait_target;
    if (sy.sig_ptrs != nullptr) {
      for (int i = 0; i < sy.world && i < 8; ++i) p.sig[i] = reinterpret_cast<uint32_t*>(sy.sig_ptrs[i]);
      p.sig_bpr = sy.sig_bpr;
      if (p.sig_bpr <= 0) { set_last_error("dh_gemm_bf16_sync: blocks per rank must be positive"); return (int)cudaErrorInvalidValue; }
    }
    // the row order follows the ranks' shards only when every shard is a whole number of 256-row tiles
    if (sy.perm_mode != 0 && sy.world > 1 && p.tiles_m % sy.world == 0 && M % TILE_M == 0) {
      p.perm_mode = sy.perm_mode; p.perm_world = sy.world; p.perm_rank = sy.rank;
      p.group_m = sy.perm_mode == 1 ? (p.tiles_m / sy.world < pair_group ? p.tiles_m / sy.world : pair_group) : pair_group;
    }
    // barriers inside the CTA sit downstream of a peer wait, so they must outlast it
    p.wait_budget = (p.wait_count != nullptr) ? 2 * PEER_WAIT_CYCLES : (long long)DH_WAIT_BUDGET_CYCLES;
    p.start_id = sy.start_id;
    const int num_items = num_tiles * p.split_k;
    if (sy.comm_kind == 0 && pairs > num_items) pairs = num_items;     // the communication warps use every CTA of the budget
    CUtensorMap td;
    if (!encode_tmap_2d_into(&td, d, d_fp32 ? 4 : 2, (uint64_t)N, (uint64_t)M, (uint64_t)ldd * (d_fp32 ? 4 : 2), d_fp32 ? 32 : 64, 32, true))
      return (int)cudaErrorInvalidValue;
    if (sy.comm_kind != 0) {
      if (a_mn_major || d_fp32) { set_last_error("dh_gemm_bf16: a GEMM that carries a collective has a K-major A and a bf16 output"); return (int)cudaErrorInvalidValue; }
      p.comm_kind = sy.comm_kind;
      if (sy.push) p.push = *sy.push;
      if (sy.reduce) p.reduce = *sy.reduce;
      return b_mn_major ? launch_pair<false, true, false, true>(ta, tb, &td, p, pairs, stream)
                        : launch_pair<false, false, false, true>(ta, tb, &td, p, pairs, stream);
    }
    switch (sel) {
      case 0: return launch_pair<false, false, false>(ta, tb, &td, p, pairs, stream);
      case 1: return launch_pair<false, false, true>(ta, tb, &td, p, pairs, stream);
      case 2: return launch_pair<false, true, false>(ta, tb, &td, p, pairs, stream);
      case 3: return launch_pair<false, true, true>(ta, tb, &td, p, pairs, stream);
      case 4: return launch_pair<true, false, false>(ta, tb, &td, p, pairs, stream);
      case 5: return launch_pair<true, false, true>(ta, tb, &td, p, pairs, stream);
      case 6: return launch_pair<true, true, false>(ta, tb, &td, p, pairs, stream);
      default: return launch_pair<true, true, true>(ta, tb, &td, p, pairs, stream);
    }
  }
  Params p;
  p.d = d;
  p.ldd = ldd;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.accumulate = accumulate;
  p.stages = 0;
  p.group_m = 0;
  p.status = status;
  const int num_tiles = p.tiles_m * p.tiles_n;
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

}  // namespace gemm
}  // namespace dh

// Work items per tile along K for accumulating outputs: -1 = heuristic (default; DHELLAM_GEMM_SPLITK overrides),
// 0 / 1 = never split, n = always n (as far as K allows).
extern "C" void dh_gemm_set_splitk(int n) { dh::gemm::g_splitk_override = n; }

extern "C" int dh_gemm_bf16(const void* a, int64_t lda, int a_mn_major, const void* b, int64_t ldb, int b_mn_major, void* d,
                            int64_t ldd, int d_fp32, int accumulate, int M, int N, int K, int epilogue, int sm_budget,
                            cudaStream_t stream) {
  if (epilogue != 0) {
    dh::set_last_error("dh_gemm_bf16: unknown epilogue %d", epilogue);
    return (int)cudaErrorInvalidValue;
  }
  return dh::gemm::gemm_impl(a, lda, a_mn_major, b, ldb, b_mn_major, d, ldd, d_fp32, accumulate, M, N, K, sm_budget, dh::gemm::SyncArgs(),
                             stream);
}

// The same product with the tensor-parallel collective hooks of the CTA-pair kernel:
//   wait_count / wait_target  A is an all-gather staging buffer: wait per 128-row block for its arrival counter
//   sig_ptrs / sig_bpr        D is this rank's partial product of a reduce-scatter: after each stored row block bump
//                             its counter on the owning rank (sig_ptrs[owner][block within the owner's shard])
//   perm_mode                 0 natural row order, 1 own shard first then the others block by block, 2 block by
//                             block over all owners
static unsigned g_start_ids[64];             // per device: id of the newest signalling GEMM launched

extern "C" int dh_gemm_bf16_sync(const void* a, int64_t lda, int a_mn_major, const void* b, int64_t ldb, int b_mn_major, void* d,
                                 int64_t ldd, int d_fp32, int accumulate, int M, int N, int K, int sm_budget, const void* wait_count,
                                 unsigned wait_target, void* const* sig_ptrs, int sig_bpr, int perm_mode, int world, int rank,
                                 cudaStream_t stream) {
  dh::gemm::SyncArgs sy;
  sy.wait_count = wait_count;
  sy.wait_target = wait_target;
  sy.sig_ptrs = sig_ptrs;
  sy.sig_bpr = sig_bpr;
  sy.perm_mode = perm_mode;
  sy.world = world;
  sy.rank = rank;
  if (sig_ptrs != nullptr) {
    // a GEMM whose row-block signals another kernel may spin on: announce when all of its CTAs are resident
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64) sy.start_id = ++g_start_ids[dev];
  }
  return dh::gemm::gemm_impl(a, lda, a_mn_major, b, ldb, b_mn_major, d, ldd, d_fp32, accumulate, M, N, K, sm_budget, sy, stream);
}

// Device address of the word that holds the id of the newest signalling GEMM whose CTAs are all resident, and the id
// that the most recent dh_gemm_bf16_sync call with row-block signals on this device announced (0: none yet).
extern "C" const void* dh_gemm_start_flag_ptr() {
  void* ptr = nullptr;
  cudaGetSymbolAddress(&ptr, dh::gemm::pair::g_start_flag);
  return ptr;
}
extern "C" unsigned dh_gemm_last_start_id() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < 64) ? g_start_ids[dev] : 0u;
}

int dh_fill_push_job(dh::comm::PushJob& p, const char* who, const void* shard, void* const* stage_ptrs, void* const* count_ptrs,
                     void* stage_mc, int M, int K, int rank, int world, int slices);
int dh_fill_reduce_job(dh::comm::ReduceJob& p, const char* who, void* const* part_ptrs, const void* part_mc, const void* ready, void* out,
                       int M, int N, int rank, int world, unsigned target, int slices);

// Sequence all-gather -> GEMM in ONE kernel: the communication warps of every CTA push this rank's
// [M / world, K] shard into every rank's staging buffer (multimem.st through the switch, or per-peer
// stores) and raise the per-row-block arrival counters, while the tensor-core warps multiply the staged
// operand, own rows first, waiting per 128-row block for its counter and reading local memory only.
//   stage_ptrs / count_ptrs: `world` device pointers (index = rank); stage_mc: multicast alias or null
//   target_base: counter value before this call; every counter rises by `slices`
// After the call the local staging buffer holds the gathered [M, K] operand (kept for the weight gradient).
extern "C" int dh_ag_gemm_bf16(const void* shard, void* const* stage_ptrs, void* const* count_ptrs, void* stage_mc, const void* b,
                               int64_t ldb, int b_mn_major, void* d, int64_t ldd, int M, int N, int K, int rank, int world, int slices,
                               unsigned target_base, int sm_budget, cudaStream_t stream) {
  dh::comm::PushJob job;
  int rc = dh_fill_push_job(job, "dh_ag_gemm_bf16", shard, stage_ptrs, count_ptrs, stage_mc, M, K, rank, world, slices);
  if (rc) return rc;
  dh::gemm::SyncArgs sy;
  sy.wait_count = count_ptrs[rank];
  sy.wait_target = target_base + (unsigned)slices;
  sy.perm_mode = 1;
  sy.world = world;
  sy.rank = rank;
  sy.comm_kind = 1;
  sy.push = &job;
  return dh::gemm::gemm_impl(stage_ptrs[rank], K, 0, b, ldb, b_mn_major, d, ldd, 0, 0, M, N, K, sm_budget, sy, stream);
}

// GEMM -> sequence reduce-scatter in ONE kernel: the tensor-core warps write this rank's partial product
// [M, N] into its symmetric buffer, row block by row block over all owners, and signal every finished row
// block to its owner; the communication warps of the same kernel reduce this rank's own rows as soon as
// every rank has delivered a block (in-switch multimem.ld_reduce, or peer loads) into out [M / world, N].
//   part_ptrs / ready_ptrs: `world` device pointers (every rank's partial buffer and per-block counters)
//   target: the counter value of a block that every rank has delivered in this call
extern "C" int dh_gemm_rs_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, int b_mn_major, void* const* part_ptrs,
                               const void* part_mc, void* const* ready_ptrs, void* out, int M, int N, int K, int rank, int world,
                               unsigned target, int sm_budget, cudaStream_t stream) {
  if (world < 2 || world > 8 || M % (world * 128) != 0) {
    dh::set_last_error("dh_gemm_rs_bf16: world %d / M %d: need 2..8 ranks and M divisible by world*128", world, M);
    return (int)cudaErrorInvalidValue;
  }
  const int blocks = M / world / 128;
  dh::comm::ReduceJob job;
  int rc = dh_fill_reduce_job(job, "dh_gemm_rs_bf16", part_ptrs, part_mc, ready_ptrs[rank], out, M, N, rank, world, target,
                              dh::comm::reduce_slices_for(N, dh_sm_count()));
  if (rc) return rc;
  dh::gemm::SyncArgs sy;
  sy.sig_ptrs = ready_ptrs;
  sy.sig_bpr = blocks;
  sy.perm_mode = 2;
  sy.world = world;
  sy.rank = rank;
  sy.comm_kind = 2;
  sy.reduce = &job;
  return dh::gemm::gemm_impl(a, lda, 0, b, ldb, b_mn_major, part_ptrs[rank], N, 0, 0, M, N, K, sm_budget, sy, stream);
}

// Grouped (ragged) GEMM over the experts of a mixture-of-experts layer in ONE launch; the per-expert row ranges
// `offs` ([groups + 1] int32, multiples of 256) live in device memory and are never read by the host.
//   group_mode 1 (rows grouped):  D[rows, N] = A[rows, K] * op(B_e) for the rows of expert e.
//       A is [capacity, K] K-major, D is [capacity, N] bf16 (capacity = M);
//       b_mn_major = 0: B is the stack [groups * N, K] (forward: y = x W_e^T);
//       b_mn_major = 1: B is the stack [groups * K, N] (data gradient: dx = dy W_e).
//   group_mode 2 (contraction grouped, weight gradients):  D_e[M, N] += A_e^T B_e with A [capacity, M] and
//       B [capacity, N] both MN-major and the contraction of expert e over rows [offs[e], offs[e+1]);
//       D is the stack [groups * M, N] fp32, added in place.  M must be a multiple of 256.
extern "C" int dh_gemm_grouped_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, int b_mn_major, void* d, int64_t ldd, int M,
                                    int N, int K, int groups, int group_mode, const void* offs, int capacity, int sm_budget,
                                    cudaStream_t stream) {
  using namespace dh;
  using namespace dh::gemm;
  using namespace dh::gemm::pair;
  if (groups < 1 || (group_mode != 1 && group_mode != 2) || offs == nullptr || capacity <= 0 || capacity % TILE_M != 0) {
    set_last_error("dh_gemm_grouped_bf16: bad arguments (groups %d, mode %d, capacity %d)", groups, group_mode, capacity);
    return (int)cudaErrorInvalidValue;
  }
  const bool wgrad = group_mode == 2;
  if (wgrad && (M % TILE_M != 0)) { set_last_error("dh_gemm_grouped_bf16: grouped weight gradients need M %% 256 == 0 (M=%d)", M); return (int)cudaErrorInvalidValue; }
  const int elem = wgrad ? 4 : 2;
  if ((ldd % (wgrad ? 4 : 8)) != 0 || (reinterpret_cast<uintptr_t>(d) & 15) != 0) { set_last_error("dh_gemm_grouped_bf16: output alignment"); return (int)cudaErrorInvalidValue; }
  const CUtensorMap *ta, *tb;
  if (!wgrad) {
    ta = get_tmap_2d(a, 2, (uint64_t)K, (uint64_t)capacity, (uint64_t)lda * 2, BK, BM, true);
    tb = b_mn_major ? get_tmap_2d(b, 2, (uint64_t)N, (uint64_t)groups * K, (uint64_t)ldb * 2, 64, BK, true)
                    : get_tmap_2d(b, 2, (uint64_t)K, (uint64_t)groups * N, (uint64_t)ldb * 2, BK, BN_HALF, true);
  } else {
    ta = get_tmap_2d(a, 2, (uint64_t)M, (uint64_t)capacity, (uint64_t)lda * 2, 64, BK, true);
    tb = get_tmap_2d(b, 2, (uint64_t)N, (uint64_t)capacity, (uint64_t)ldb * 2, 64, BK, true);
  }
  if (!ta || !tb) return (int)cudaErrorInvalidValue;
  CUtensorMap td;
  const uint64_t d_rows = wgrad ? (uint64_t)groups * M : (uint64_t)capacity;
  if (!encode_tmap_2d_into(&td, d, elem, (uint64_t)N, d_rows, (uint64_t)ldd * elem, wgrad ? 32 : 64, 32, true)) return (int)cudaErrorInvalidValue;
  static int stages = 0;
  if (stages == 0) {
    const char* e = getenv("DHELLAM_GEMM_STAGES");
    stages = e ? atoi(e) : RING;
    if (stages < 2 || stages > RING) stages = RING;
  }
  PairParams p;
  memset(&p, 0, sizeof(p));
  p.M = wgrad ? M : capacity;
  p.N = N;
  p.K = wgrad ? capacity : K;
  p.tiles_m = wgrad ? M / TILE_M : capacity / TILE_M;
  p.tiles_n = (N + BN - 1) / BN;
  p.stages = stages;
  p.group_m = 8;
  p.split_k = 1;
  p.kb_per_split = (p.K + BK - 1) / BK;
  p.reduce_add = wgrad ? 1 : 0;
  p.group_mode = group_mode;
  p.groups = groups;
  p.group_offs = reinterpret_cast<const int*>(offs);
  p.wait_budget = (long long)DH_WAIT_BUDGET_CYCLES;
  p.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  const int sms = dh_sm_count();
  const int budget = (sm_budget <= 0 || sm_budget > sms) ? sms : sm_budget;
  const int pairs = budget / 2 < 1 ? 1 : budget / 2;
  if (wgrad) return launch_pair<true, true, true>(ta, tb, &td, p, pairs, stream);
  return b_mn_major ? launch_pair<false, true, false>(ta, tb, &td, p, pairs, stream) : launch_pair<false, false, false>(ta, tb, &td, p, pairs, stream);
}
