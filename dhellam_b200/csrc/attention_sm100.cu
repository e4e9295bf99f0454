// Flash attention forward and backward for sm_100a (head size 128, bf16, grouped KV heads,
// causal or full, strided [S, B, heads, d] operands so a packed QKV buffer needs no copies).
//
// Forward, one CTA per (128 query rows, batch, query head):
//   warp 0     TMA producer: Q once, then K_j / V_j tiles through 2-stage rings
//   warp 1     MMA issuer:   S_j = Q K_j^T and O_j = P_j V_j with tcgen05.mma, S and O tiles
//                            double-buffered in TMEM (4 x 128 columns = all 512)
//   warps 2-9  softmax:      two warps per TMEM lane quarter; both own the same 32 query rows, each
//                            takes 64 of the 128 score columns and 64 of the 128 output columns: two
//                            passes over its part of S_j in TMEM (row max, exchanged inside the pair
//                            through shared memory; then exp2 / row sum / bf16 P_j into swizzled
//                            shared memory), running output kept in registers (64 per thread) and
//                            rescaled once per block
//   S_{j+1} and P_{j-1} V_{j-1} run on the tensor cores while the softmax warps work on S_j.
//
// Backward is two kernels that share delta = rowsum(dO * O):
//   dK/dV: one CTA per (128 keys, batch, KV head) loops over the query heads of the group and
//     the query blocks that see these keys: S = Q K^T and dP = dO V^T into TMEM; eight math
//     warps form P = exp2(S - lse) and dS = P (dP - delta) into swizzled shared-memory images
//     that are consumed as MN-major operands (dV += P^T dO, dK += dS^T Q), so no transposed
//     copies exist anywhere; dK / dV accumulate in TMEM over the whole loop, which also sums
//     the query heads of a KV group.  When keys x batch x KV heads gives too few CTAs for the
//     machine (one KV head per GPU under tensor parallelism), the query heads of a group are
//     split over up to 8 CTAs that write fp32 partials, and attn_dkv_reduce_kernel adds them.
//   dQ: one CTA per (128 queries, batch, query head) loops over the key blocks, recomputes S
//     and dP and accumulates dQ += dS K in TMEM.  Recomputing two products per tile pair
//     replaces an fp32 atomic accumulation of dQ, which was bound by L2 atomic throughput.
//
// Role in the reference: the bundled flash-attention 2 sm80 kernels behind
// pymha_varlen_fwd / pymha_varlen_bwd (csrc/operators/flash_atten.cu:220-434, 479-757);
// its fp32 dq_accum and its separate GQA reduction pass (:637-652, 742-745) have no
// counterpart here.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include <cstdlib>
#include <mutex>

#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

namespace dh {
namespace attn {

constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int HALF_BYTES = 128 * 128;        // one [128 rows][64 elems] swizzled box
constexpr int TILE_BYTES = 2 * HALF_BYTES;   // [128][128] bf16
constexpr int THREADS = 192;
constexpr int BWD_THREADS = 320;           // TMA warp + MMA warp + 8 math warps (two per TMEM lane quarter)
constexpr float LOG2E = 1.4426950408889634f;

struct Geometry {
  int B, Hq, Hk, Sq, Sk, causal;
  float scale;
  long long o_s, o_b, o_h;        // output strides (elements)
  DeviceStatus* status;
  int x0, p0, ny;                 // SM budget: this launch covers tile columns from x0 and (head, batch) pairs from p0; ny = heads
};

// K-major operand descriptor for step kk (16 elements of the contraction) of a tile stored
// as two [128][64] swizzled boxes.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int kk) {
  return umma_smem_desc(base + (kk >> 2) * HALF_BYTES + (kk & 3) * 32, 16, 1024);
}
// MN-major operand descriptor: the contraction runs over the 128 rows of the tile.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int kk) {
  return umma_smem_desc(base + kk * 2048, HALF_BYTES, 1024);
}
// Byte offset of 16-byte chunk c (0..15) of row r in the two-box swizzled image.
__device__ __forceinline__ uint32_t swz_off(int r, int c) {
  return (uint32_t)((c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// ======================================================================= forward
struct FwdCtl {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_ready[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
  float xch[2 * 128];            // row maximum / row sum exchange between the two softmax warps of a row
};
constexpr int FWD_THREADS = 320;                         // TMA warp + MMA warp + 8 softmax warps
constexpr int FWD_SMEM = TILE_BYTES * 7 + 1024 + 1280;  // Q, K x2, V x2, P x2, control

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                __nv_bfloat16* __restrict__ out, float* __restrict__ lse, const Geometry g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;
  uint8_t* sV = smem + 3 * TILE_BYTES;
  uint8_t* sP = smem + 5 * TILE_BYTES;
  FwdCtl* ctl = reinterpret_cast<FwdCtl*>(smem + 7 * TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (g.Sq + BQ - 1) / BQ;
  const int qb = nqb - 1 - (g.x0 + (int)blockIdx.x);       // heaviest (latest) query blocks first
  const int pyz = g.p0 + (int)blockIdx.y + (int)blockIdx.z * (int)gridDim.y;
  const int hq = pyz % g.ny, b = pyz / g.ny;
  const int hk = hq / (g.Hq / g.Hk);
  const int off = g.Sk - g.Sq;                    // key j visible to query i iff j <= i + off
  int nblk = (g.Sk + BKV - 1) / BKV;
  if (g.causal) {
    const int last_key = qb * BQ + BQ - 1 + off;
    nblk = last_key < 0 ? 0 : min(nblk, last_key / BKV + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->k_full[i], 1); mbar_init(&ctl->k_empty[i], 1);
      mbar_init(&ctl->v_full[i], 1); mbar_init(&ctl->v_empty[i], 1);
      mbar_init(&ctl->s_full[i], 1); mbar_init(&ctl->p_ready[i], 8); mbar_init(&ctl->o_full[i], 1);
    }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ctl->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv);
      mbar_expect_tx(&ctl->q_full, TILE_BYTES);
      tma_load_4d(sQ, &tq, &ctl->q_full, 0, hq, b, qb * BQ);
      tma_load_4d(sQ + HALF_BYTES, &tq, &ctl->q_full, 64, hq, b, qb * BQ);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&ctl->k_empty[s], ph ^ 1, abort_flag, g.status, 400)) break;
        mbar_expect_tx(&ctl->k_full[s], TILE_BYTES);
        tma_load_4d(sK + s * TILE_BYTES, &tk, &ctl->k_full[s], 0, hk, b, j * BKV);
        tma_load_4d(sK + s * TILE_BYTES + HALF_BYTES, &tk, &ctl->k_full[s], 64, hk, b, j * BKV);
        if (!mbar_wait(&ctl->v_empty[s], ph ^ 1, abort_flag, g.status, 401)) break;
        mbar_expect_tx(&ctl->v_full[s], TILE_BYTES);
        tma_load_4d(sV + s * TILE_BYTES, &tv, &ctl->v_full[s], 0, hk, b, j * BKV);
        tma_load_4d(sV + s * TILE_BYTES + HALF_BYTES, &tv, &ctl->v_full[s], 64, hk, b, j * BKV);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_base = smem_u32(sQ);
      bool ok = mbar_wait(&ctl->q_full, 0, abort_flag, g.status, 410);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&ctl->k_full[s], (j >> 1) & 1, abort_flag, g.status, 411)) return false;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + s * 128, desc_kmajor(q_base, kk), desc_kmajor(k_base, kk), idesc_s, kk > 0);
        umma_commit(&ctl->k_empty[s]);
        umma_commit(&ctl->s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      if (ok && nblk > 1) ok = issue_s(1);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&ctl->p_ready[s], ph, abort_flag, g.status, 412)) break;
        if (!mbar_wait(&ctl->v_full[s], ph, abort_flag, g.status, 413)) break;
        tc_fence_after();
        const uint32_t p_base = smem_u32(sP + s * TILE_BYTES);
        const uint32_t v_base = smem_u32(sV + s * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 256 + s * 128, desc_kmajor(p_base, kk), desc_mnmajor(v_base, kk), idesc_pv, kk > 0);
        umma_commit(&ctl->v_empty[s]);
        umma_commit(&ctl->o_full[s]);
        if (j + 2 < nblk) ok = issue_s(j + 2);
      }
    }
    __syncwarp();
  } else {
    // Eight softmax warps: two per TMEM lane quarter.  Both warps of a pair own the same 32 query rows;
    // warp half `hf` handles score columns [64 hf, 64 hf + 64) of every key block and head-dim columns
    // [64 hf, 64 hf + 64) of the running output.  The row maximum is exchanged through shared memory
    // (one named barrier per pair), the row sums are added once at the end.  Two warps per scheduler hide
    // the TMEM round trips that a single warp per scheduler exposes.  A warp whose wait gives up keeps
    // walking the loop (every later wait returns at once through the CTA's abort flag), so the pair's
    // barriers always match.
    const int quarter = warp & 3;
    const int hf = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;               // row inside the tile
    const int qi = qb * BQ + r;                      // global query index
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sl2 = g.scale * LOG2E;
    float* xch = ctl->xch;                           // [2][128] exchange between the two warps of a pair
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };
    float m = -FLT_MAX, l = 0.f;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    bool ok = nblk > 0;
    for (int j = 0; j < nblk; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (ok && !mbar_wait(&ctl->s_full[s], ph, abort_flag, g.status, 420)) ok = false;
      tc_fence_after();
      const uint32_t ts = tmem + s * 128 + lane_base + hf * 64;
      const int key0 = j * BKV + hf * 64;            // first key of this warp's columns
      int limit = g.Sk - key0;                                        // keys beyond Sk are padding
      if (g.causal) limit = min(limit, qi + off - key0 + 1);
      const bool full_block = limit >= 64;
      // pass 1: row maximum over this warp's 64 columns, then over the pair
      float bm = -FLT_MAX;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(ts + c * 32, v);
        tmem_ld_wait();
        if (full_block) {
#pragma unroll
          for (int i = 0; i < 32; ++i) bm = fmaxf(bm, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) if (c * 32 + i < limit) bm = fmaxf(bm, __uint_as_float(v[i]));
        }
      }
      xch[hf * 128 + r] = bm;
      pair_sync();
      bm = fmaxf(bm, xch[(hf ^ 1) * 128 + r]);
      pair_sync();                                   // the partner has read before the next block overwrites
      const float m_new = fmaxf(m, bm);
      const float alpha = (m == -FLT_MAX) ? 0.f : exp2f((m - m_new) * sl2);
      const float mb = (m_new == -FLT_MAX) ? 0.f : m_new * sl2;
      // pass 2: probabilities -> shared memory (bf16, swizzled), partial row sum
      float rs = 0.f;
      uint8_t* pdst = sP + s * TILE_BYTES;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(ts + c * 32, v);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = exp2f(__uint_as_float(v[i]) * sl2 - mb);
          if (!full_block && c * 32 + i >= limit) e = 0.f;
          p[i] = e;
          rs += e;
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 u;
          u.x = pack_bf16x2(p[q4 * 8 + 0], p[q4 * 8 + 1]);
          u.y = pack_bf16x2(p[q4 * 8 + 2], p[q4 * 8 + 3]);
          u.z = pack_bf16x2(p[q4 * 8 + 4], p[q4 * 8 + 5]);
          u.w = pack_bf16x2(p[q4 * 8 + 6], p[q4 * 8 + 7]);
          *reinterpret_cast<uint4*>(pdst + swz_off(r, hf * 8 + c * 4 + q4)) = u;
        }
      }
      l = l * alpha + rs;
      m = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->p_ready[s]);
      // fold in the previous block's P V (relative to the previous maximum), then rescale: this warp's 64 head-dim columns
      if (j > 0) {
        const int sp = (j - 1) & 1;
        if (ok && !mbar_wait(&ctl->o_full[sp], ((j - 1) >> 1) & 1, abort_flag, g.status, 421)) ok = false;
        tc_fence_after();
        const uint32_t to = tmem + 256 + sp * 128 + lane_base + hf * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld32(to + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(v[i])) * alpha;
        }
        tc_fence_before();
      }
    }
    // the row sum of the whole row = the two halves' partial sums (same running maximum in both)
    xch[hf * 128 + r] = l;
    pair_sync();
    l += xch[(hf ^ 1) * 128 + r];
    if (nblk > 0) {
      const int sp = (nblk - 1) & 1;
      if (ok && !mbar_wait(&ctl->o_full[sp], ((nblk - 1) >> 1) & 1, abort_flag, g.status, 422)) ok = false;
      if (ok) {
        tc_fence_after();
        const uint32_t to = tmem + 256 + sp * 128 + lane_base + hf * 64;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = out + (long long)qi * g.o_s + (long long)b * g.o_b + (long long)hq * g.o_h + hf * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld32(to + c * 32, v);
          tmem_ld_wait();
          if (qi < g.Sq) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              const int i0 = q4 * 8;
              u.x = pack_bf16x2((o[c * 32 + i0 + 0] + __uint_as_float(v[i0 + 0])) * inv, (o[c * 32 + i0 + 1] + __uint_as_float(v[i0 + 1])) * inv);
              u.y = pack_bf16x2((o[c * 32 + i0 + 2] + __uint_as_float(v[i0 + 2])) * inv, (o[c * 32 + i0 + 3] + __uint_as_float(v[i0 + 3])) * inv);
              u.z = pack_bf16x2((o[c * 32 + i0 + 4] + __uint_as_float(v[i0 + 4])) * inv, (o[c * 32 + i0 + 5] + __uint_as_float(v[i0 + 5])) * inv);
              u.w = pack_bf16x2((o[c * 32 + i0 + 6] + __uint_as_float(v[i0 + 6])) * inv, (o[c * 32 + i0 + 7] + __uint_as_float(v[i0 + 7])) * inv);
              reinterpret_cast<uint4*>(orow + c * 32)[q4] = u;
            }
          }
        }
        if (hf == 0 && qi < g.Sq) lse[((long long)b * g.Hq + hq) * g.Sq + qi] = (l > 0.f) ? m * g.scale + logf(l) : -INFINITY;
      }
    } else if (qi < g.Sq) {
      __nv_bfloat16* orow = out + (long long)qi * g.o_s + (long long)b * g.o_b + (long long)hq * g.o_h + hf * 64;
      for (int i = 0; i < 64 / 8; ++i) reinterpret_cast<uint4*>(orow)[i] = make_uint4(0, 0, 0, 0);
      if (hf == 0) lse[((long long)b * g.Hq + hq) * g.Sq + qi] = -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ======================================================================= backward
// delta[b, h, s] = sum_d dO * O
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                                         float* __restrict__ delta, int B, int Hq, int Sq, long long do_s, long long do_b,
                                                         long long do_h, long long o_s, long long o_b, long long o_h) {
  const int wid = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int total = B * Hq * Sq;
  if (wid >= total) return;
  const int s = wid % Sq, h = (wid / Sq) % Hq, b = wid / (Sq * Hq);
  const uint2* a = reinterpret_cast<const uint2*>(dout + s * do_s + b * do_b + h * do_h) + lane;
  const uint2* c = reinterpret_cast<const uint2*>(out + s * o_s + b * o_b + h * o_h) + lane;
  const uint2 av = *a, cv = *c;
  float2 a0 = unpack_bf16x2(av.x), a1 = unpack_bf16x2(av.y), c0 = unpack_bf16x2(cv.x), c1 = unpack_bf16x2(cv.y);
  float v = a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) delta[((long long)b * Hq + h) * Sq + s] = v;
}

struct BwdCtl {
  uint64_t kv_full, qdo_full, qdo_empty, sdp_full, pds_ready, acc_full;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int BWD_SMEM = TILE_BYTES * 6 + 1024 + 256;     // K, V, Q, dO, P, dS

struct BwdGeometry {
  int B, Hq, Hk, Sq, Sk, causal;
  float scale;
  long long dk_s, dk_b, dk_h, dv_s, dv_b, dv_h;
  // Head split: the query heads of one KV head are divided over `hs` CTAs (grid.y = Hk * hs) when
  // KV blocks x batch x KV heads alone would leave SMs idle (tensor parallelism leaves one KV head per
  // GPU).  Each CTA then writes fp32 partial dV / dK to `part` ([2][hs][Sk][B][Hk][128]) and
  // attn_dkv_reduce_kernel adds them up.
  int hs;
  float* part;
  DeviceStatus* status;
  int x0, p0, ny;                 // as in Geometry; ny = Hk * hs
};

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                const __grid_constant__ CUtensorMap tdo, const float* __restrict__ lse, const float* __restrict__ delta,
                __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, const BwdGeometry g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;
  uint8_t* sDO = smem + 3 * TILE_BYTES;
  uint8_t* sP = smem + 4 * TILE_BYTES;
  uint8_t* sDS = smem + 5 * TILE_BYTES;
  BwdCtl* ctl = reinterpret_cast<BwdCtl*>(smem + 6 * TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pyz = g.p0 + (int)blockIdx.y + (int)blockIdx.z * (int)gridDim.y;
  const int by = pyz % g.ny;
  const int kb = g.x0 + (int)blockIdx.x, hk = by / g.hs, hpart = by % g.hs, b = pyz / g.ny;
  const int group = g.Hq / g.Hk;
  const int gpp = group / g.hs;                 // query heads handled by this CTA
  const int hq0 = hk * group + hpart * gpp;
  const int off = g.Sk - g.Sq;
  const int nqb = (g.Sq + BQ - 1) / BQ;
  // first query block that sees any key of this block: i + off >= kb*BKV
  int qb0 = 0;
  if (g.causal) {
    const int first_q = kb * BKV - off;
    qb0 = first_q <= 0 ? 0 : first_q / BQ;
  }
  const int n_iter = qb0 < nqb ? (nqb - qb0) * gpp : 0;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->kv_full, 1); mbar_init(&ctl->qdo_full, 1); mbar_init(&ctl->qdo_empty, 1);
    mbar_init(&ctl->sdp_full, 1); mbar_init(&ctl->pds_ready, 8); mbar_init(&ctl->acc_full, 1);
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ctl->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  // TMEM columns: [0,128) S, [128,256) dP, [256,384) dV, [384,512) dK

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv); tma_prefetch_desc(&tdo);
      mbar_expect_tx(&ctl->kv_full, 2 * TILE_BYTES);
      tma_load_4d(sK, &tk, &ctl->kv_full, 0, hk, b, kb * BKV);
      tma_load_4d(sK + HALF_BYTES, &tk, &ctl->kv_full, 64, hk, b, kb * BKV);
      tma_load_4d(sV, &tv, &ctl->kv_full, 0, hk, b, kb * BKV);
      tma_load_4d(sV + HALF_BYTES, &tv, &ctl->kv_full, 64, hk, b, kb * BKV);
      for (int it = 0; it < n_iter; ++it) {
        const int hq = hq0 + it % gpp;
        const int qb = qb0 + it / gpp;
        if (!mbar_wait(&ctl->qdo_empty, (it & 1) ^ 1, abort_flag, g.status, 500)) break;
        mbar_expect_tx(&ctl->qdo_full, 2 * TILE_BYTES);
        tma_load_4d(sQ, &tq, &ctl->qdo_full, 0, hq, b, qb * BQ);
        tma_load_4d(sQ + HALF_BYTES, &tq, &ctl->qdo_full, 64, hq, b, qb * BQ);
        tma_load_4d(sDO, &tdo, &ctl->qdo_full, 0, hq, b, qb * BQ);
        tma_load_4d(sDO + HALF_BYTES, &tdo, &ctl->qdo_full, 64, hq, b, qb * BQ);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t id_kk = umma_idesc_bf16(128, 128, 0, 0);   // S, dP: both operands K-major
      constexpr uint32_t id_mm = umma_idesc_bf16(128, 128, 1, 1);   // dV, dK: both operands MN-major
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), q_base = smem_u32(sQ), do_base = smem_u32(sDO);
      const uint32_t p_base = smem_u32(sP), ds_base = smem_u32(sDS);
      bool ok = mbar_wait(&ctl->kv_full, 0, abort_flag, g.status, 510);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(&ctl->qdo_full, ph, abort_flag, g.status, 511)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 0, desc_kmajor(q_base, kk), desc_kmajor(k_base, kk), id_kk, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 128, desc_kmajor(do_base, kk), desc_kmajor(v_base, kk), id_kk, kk > 0);
        umma_commit(&ctl->sdp_full);
        if (!mbar_wait(&ctl->pds_ready, ph, abort_flag, g.status, 513)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 256, desc_mnmajor(p_base, kk), desc_mnmajor(do_base, kk), id_mm, (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 384, desc_mnmajor(ds_base, kk), desc_mnmajor(q_base, kk), id_mm, (it | kk) != 0);
        umma_commit(&ctl->qdo_empty);           // Q and dO are free once dV and dK have read them
      }
      if (ok) umma_commit(&ctl->acc_full);
    }
    __syncwarp();
  } else {
    // warps 2..5 and 6..9 cover the four TMEM lane quarters twice: the first set works on
    // columns [0, 64), the second on [64, 128) of every 128-column tile
    const int quarter = warp & 3;
    const int c_lo = ((warp - 2) >> 2) * 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sl2 = g.scale * LOG2E;
    bool ok = n_iter > 0;
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t ph = it & 1;
      const int hq = hq0 + it % gpp;
      const int qb = qb0 + it / gpp;
      const int qi = qb * BQ + r;
      const bool row_ok = qi < g.Sq;
      const long long stat = ((long long)b * g.Hq + hq) * g.Sq + qi;
      const float L = row_ok ? lse[stat] * LOG2E : 0.f;
      const float dl = row_ok ? delta[stat] : 0.f;
      if (!mbar_wait(&ctl->sdp_full, ph, abort_flag, g.status, 520)) { ok = false; break; }
      tc_fence_after();
      const int key0 = kb * BKV;
      int limit = g.Sk - key0;
      if (g.causal) limit = min(limit, qi + off - key0 + 1);
      if (!row_ok) limit = 0;
#pragma unroll 1
      for (int c = c_lo; c < c_lo + 2; ++c) {
        uint32_t sv[32], dpv[32];
        tmem_ld32(tmem + 0 + lane_base + c * 32, sv);
        tmem_ld32(tmem + 128 + lane_base + c * 32, dpv);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float p[8], ds[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int col = c * 32 + q4 * 8 + i;
            float pe = exp2f(__uint_as_float(sv[q4 * 8 + i]) * sl2 - L);
            if (col >= limit) pe = 0.f;
            p[i] = pe;
            ds[i] = pe * (__uint_as_float(dpv[q4 * 8 + i]) - dl);
          }
          uint4 up, ud;
          up.x = pack_bf16x2(p[0], p[1]); up.y = pack_bf16x2(p[2], p[3]); up.z = pack_bf16x2(p[4], p[5]); up.w = pack_bf16x2(p[6], p[7]);
          ud.x = pack_bf16x2(ds[0], ds[1]); ud.y = pack_bf16x2(ds[2], ds[3]); ud.z = pack_bf16x2(ds[4], ds[5]); ud.w = pack_bf16x2(ds[6], ds[7]);
          const uint32_t o = swz_off(r, c * 4 + q4);
          *reinterpret_cast<uint4*>(sP + o) = up;
          *reinterpret_cast<uint4*>(sDS + o) = ud;
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->pds_ready);
    }
    // dK (times scale) and dV of this key block
    const int kj = kb * BKV + r;
    // fp32 partial rows of this CTA's head part (head split only)
    const long long part_elems = (long long)g.Sk * g.B * g.Hk * D;
    float* pdv = g.hs > 1 ? g.part + (long long)hpart * part_elems + (((long long)kj * g.B + b) * g.Hk + hk) * D : nullptr;
    float* pdk = g.hs > 1 ? pdv + (long long)g.hs * part_elems : nullptr;
    if (g.hs > 1) {
      if (ok && n_iter > 0) {
        if (mbar_wait(&ctl->acc_full, 0, abort_flag, g.status, 523)) {
          tc_fence_after();
#pragma unroll 1
          for (int c = c_lo; c < c_lo + 2; ++c) {
            uint32_t a[32], bb[32];
            tmem_ld32(tmem + 256 + lane_base + c * 32, a);      // warp-collective: no per-lane branch around it
            tmem_ld32(tmem + 384 + lane_base + c * 32, bb);
            tmem_ld_wait();
            if (kj < g.Sk) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                reinterpret_cast<float4*>(pdv + c * 32)[j] = make_float4(__uint_as_float(a[4 * j]), __uint_as_float(a[4 * j + 1]),
                                                                         __uint_as_float(a[4 * j + 2]), __uint_as_float(a[4 * j + 3]));
                reinterpret_cast<float4*>(pdk + c * 32)[j] =
                    make_float4(__uint_as_float(bb[4 * j]) * g.scale, __uint_as_float(bb[4 * j + 1]) * g.scale,
                                __uint_as_float(bb[4 * j + 2]) * g.scale, __uint_as_float(bb[4 * j + 3]) * g.scale);
              }
            }
          }
        }
      } else if (n_iter == 0 && kj < g.Sk) {
        for (int i = c_lo * 8; i < c_lo * 8 + 16; ++i) {
          reinterpret_cast<float4*>(pdv)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          reinterpret_cast<float4*>(pdk)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    } else if (ok && n_iter > 0) {
      if (mbar_wait(&ctl->acc_full, 0, abort_flag, g.status, 522)) {
        tc_fence_after();
        __nv_bfloat16* dvr = dv + (long long)kj * g.dv_s + (long long)b * g.dv_b + (long long)hk * g.dv_h;
        __nv_bfloat16* dkr = dk + (long long)kj * g.dk_s + (long long)b * g.dk_b + (long long)hk * g.dk_h;
#pragma unroll 1
        for (int c = c_lo; c < c_lo + 2; ++c) {
          uint32_t a[32], bb[32];
          tmem_ld32(tmem + 256 + lane_base + c * 32, a);
          tmem_ld32(tmem + 384 + lane_base + c * 32, bb);
          tmem_ld_wait();
          if (kj < g.Sk) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u, w;
              const int i0 = q4 * 8;
              u.x = pack_bf16x2(__uint_as_float(a[i0]), __uint_as_float(a[i0 + 1]));
              u.y = pack_bf16x2(__uint_as_float(a[i0 + 2]), __uint_as_float(a[i0 + 3]));
              u.z = pack_bf16x2(__uint_as_float(a[i0 + 4]), __uint_as_float(a[i0 + 5]));
              u.w = pack_bf16x2(__uint_as_float(a[i0 + 6]), __uint_as_float(a[i0 + 7]));
              w.x = pack_bf16x2(__uint_as_float(bb[i0]) * g.scale, __uint_as_float(bb[i0 + 1]) * g.scale);
              w.y = pack_bf16x2(__uint_as_float(bb[i0 + 2]) * g.scale, __uint_as_float(bb[i0 + 3]) * g.scale);
              w.z = pack_bf16x2(__uint_as_float(bb[i0 + 4]) * g.scale, __uint_as_float(bb[i0 + 5]) * g.scale);
              w.w = pack_bf16x2(__uint_as_float(bb[i0 + 6]) * g.scale, __uint_as_float(bb[i0 + 7]) * g.scale);
              reinterpret_cast<uint4*>(dvr + c * 32)[q4] = u;
              reinterpret_cast<uint4*>(dkr + c * 32)[q4] = w;
            }
          }
        }
      }
    } else if (n_iter == 0 && kj < g.Sk && c_lo == 0) {
      __nv_bfloat16* dvr = dv + (long long)kj * g.dv_s + (long long)b * g.dv_b + (long long)hk * g.dv_h;
      __nv_bfloat16* dkr = dk + (long long)kj * g.dk_s + (long long)b * g.dk_b + (long long)hk * g.dk_h;
      for (int i = 0; i < D / 8; ++i) {
        reinterpret_cast<uint4*>(dvr)[i] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(dkr)[i] = make_uint4(0, 0, 0, 0);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ----------------------------------------------------------------------- backward, dK/dV, pipelined form
// Same work split as attn_bwd_kernel (one CTA per 128 keys, loop over the query heads of its
// part of the KV group and over the query blocks that see these keys), rearranged so that the
// tensor cores, the TMA and the math warps overlap:
//   * the scores are formed transposed, S^T = K Q^T and dP^T = V dO^T (keys on the TMEM lanes,
//     64 queries per iteration on the columns), double-buffered in TMEM (4 x 64 columns), so the
//     products of iteration i+1 run while the math warps work on iteration i;
//   * a math thread owns one key row: it forms P^T = exp2(S^T - lse[q]) and dS^T = P^T (dP^T -
//     delta[q]) with the per-query statistics taken from registers of its warp (shuffles), and
//     writes its 64-byte piece of the row into a K-major [128 keys][64 queries] shared-memory
//     tile, which is the A operand of dV += P^T dO and dK += dS^T Q as it stands;
//   * Q / dO tiles are 64 rows (16 KiB each) in a 2-stage ring, P^T / dS^T tiles likewise, which
//     fits 192 KiB; the TMA for iteration i+1 is in flight during iteration i.
// dV / dK accumulate in TMEM columns [256, 512) exactly as in attn_bwd_kernel, so the epilogue
// (bf16 rows, or fp32 partials under the head split) is the same.
constexpr int BQT = 64;                          // queries per iteration
constexpr int QT_HALF = BQT * 128;               // one [64 rows][64 elems] swizzled box
constexpr int QT_TILE = 2 * QT_HALF;             // [64][128] bf16
constexpr int PT_TILE = BKV * 128;               // [128 keys][64 queries] bf16, one 128-byte row per key
struct BwdTCtl {
  uint64_t kv_full, qdo_full[2], stage_free[2], sdp_full[2], sdp_empty[2], pds_ready[2], acc_full;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int BWDT_SMEM = 2 * TILE_BYTES + 4 * QT_TILE + 4 * PT_TILE + 1024 + 256;

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_t_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                  const __grid_constant__ CUtensorMap tdo, const float* __restrict__ lse, const float* __restrict__ delta,
                  __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, const BwdGeometry g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;                     // 2 stages
  uint8_t* sDO = sQ + 2 * QT_TILE;                         // 2 stages
  uint8_t* sP = sDO + 2 * QT_TILE;                         // 2 stages
  uint8_t* sDS = sP + 2 * PT_TILE;                         // 2 stages
  BwdTCtl* ctl = reinterpret_cast<BwdTCtl*>(sDS + 2 * PT_TILE);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pyz = g.p0 + (int)blockIdx.y + (int)blockIdx.z * (int)gridDim.y;
  const int by = pyz % g.ny;
  const int kb = g.x0 + (int)blockIdx.x, hk = by / g.hs, hpart = by % g.hs, b = pyz / g.ny;
  const int group = g.Hq / g.Hk;
  const int gpp = group / g.hs;
  const int hq0 = hk * group + hpart * gpp;
  const int off = g.Sk - g.Sq;
  const int nqb = (g.Sq + BQT - 1) / BQT;
  int qb0 = 0;
  if (g.causal) {
    const int first_q = kb * BKV - off;
    qb0 = first_q <= 0 ? 0 : first_q / BQT;
  }
  const int n_iter = qb0 < nqb ? (nqb - qb0) * gpp : 0;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->kv_full, 1);
    mbar_init(&ctl->acc_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->qdo_full[i], 1);
      mbar_init(&ctl->stage_free[i], 1);
      mbar_init(&ctl->sdp_full[i], 1);
      mbar_init(&ctl->sdp_empty[i], 8);
      mbar_init(&ctl->pds_ready[i], 8);
    }
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ctl->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  // TMEM columns: S^T buffers [0,64) [64,128); dP^T buffers [128,192) [192,256); dV [256,384); dK [384,512)

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv); tma_prefetch_desc(&tdo);
      mbar_expect_tx(&ctl->kv_full, 2 * TILE_BYTES);
      tma_load_4d(sK, &tk, &ctl->kv_full, 0, hk, b, kb * BKV);
      tma_load_4d(sK + HALF_BYTES, &tk, &ctl->kv_full, 64, hk, b, kb * BKV);
      tma_load_4d(sV, &tv, &ctl->kv_full, 0, hk, b, kb * BKV);
      tma_load_4d(sV + HALF_BYTES, &tv, &ctl->kv_full, 64, hk, b, kb * BKV);
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int hq = hq0 + it % gpp;
        const int qb = qb0 + it / gpp;
        if (!mbar_wait(&ctl->stage_free[st], ph ^ 1, abort_flag, g.status, 530)) break;
        mbar_expect_tx(&ctl->qdo_full[st], 2 * QT_TILE);
        uint8_t* q_dst = sQ + st * QT_TILE;
        uint8_t* do_dst = sDO + st * QT_TILE;
        tma_load_4d(q_dst, &tq, &ctl->qdo_full[st], 0, hq, b, qb * BQT);
        tma_load_4d(q_dst + QT_HALF, &tq, &ctl->qdo_full[st], 64, hq, b, qb * BQT);
        tma_load_4d(do_dst, &tdo, &ctl->qdo_full[st], 0, hq, b, qb * BQT);
        tma_load_4d(do_dst + QT_HALF, &tdo, &ctl->qdo_full[st], 64, hq, b, qb * BQT);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t id_st = umma_idesc_bf16(128, BQT, 0, 0);    // S^T, dP^T: A = K / V (K-major), B = Q / dO (K-major), N = 64
      constexpr uint32_t id_acc = umma_idesc_bf16(128, 128, 0, 1);   // dV, dK: A = P^T / dS^T (K-major), B = dO / Q (MN-major)
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV);
      bool ok = mbar_wait(&ctl->kv_full, 0, abort_flag, g.status, 540);
      // S^T and dP^T of iteration j into TMEM buffer j & 1
      auto issue_scores = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&ctl->qdo_full[st], ph, abort_flag, g.status, 541)) return false;
        if (!mbar_wait(&ctl->sdp_empty[st], ph ^ 1, abort_flag, g.status, 542)) return false;
        tc_fence_after();
        const uint32_t q_base = smem_u32(sQ + st * QT_TILE), do_base = smem_u32(sDO + st * QT_TILE);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem + 64 * st, desc_kmajor(k_base, kk), umma_smem_desc(q_base + (kk >> 2) * QT_HALF + (kk & 3) * 32, 16, 1024), id_st,
                    kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem + 128 + 64 * st, desc_kmajor(v_base, kk), umma_smem_desc(do_base + (kk >> 2) * QT_HALF + (kk & 3) * 32, 16, 1024),
                    id_st, kk > 0);
        umma_commit(&ctl->sdp_full[st]);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (it + 1 < n_iter && !issue_scores(it + 1)) { ok = false; break; }
        if (!mbar_wait(&ctl->pds_ready[st], ph, abort_flag, g.status, 543)) { ok = false; break; }
        tc_fence_after();
        const uint32_t p_base = smem_u32(sP + st * PT_TILE), ds_base = smem_u32(sDS + st * PT_TILE);
        const uint32_t q_base = smem_u32(sQ + st * QT_TILE), do_base = smem_u32(sDO + st * QT_TILE);
#pragma unroll
        for (int kk = 0; kk < BQT / 16; ++kk)
          umma_bf16(tmem + 256, umma_smem_desc(p_base + kk * 32, 16, 1024), umma_smem_desc(do_base + kk * 2048, QT_HALF, 1024), id_acc,
                    (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < BQT / 16; ++kk)
          umma_bf16(tmem + 384, umma_smem_desc(ds_base + kk * 32, 16, 1024), umma_smem_desc(q_base + kk * 2048, QT_HALF, 1024), id_acc,
                    (it | kk) != 0);
        umma_commit(&ctl->stage_free[st]);      // Q, dO, P^T, dS^T of this stage are free once dV and dK have read them
      }
      if (ok) umma_commit(&ctl->acc_full);
    }
    __syncwarp();
  } else {
    // warps 2..5 take query columns [0, 32) of the 64-column buffers, warps 6..9 take [32, 64);
    // each warp covers the TMEM lane quarter (key rows) it is allowed to read
    const int quarter = warp & 3;
    const int c_half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;                 // key row inside the block
    const int kv_g = kb * BKV + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sl2 = g.scale * LOG2E;
    bool ok = n_iter > 0;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int hq = hq0 + it % gpp;
      const int qb = qb0 + it / gpp;
      // lane j holds the statistics of query column j of this warp's 32 columns
      const int q_mine = qb * BQT + c_half * 32 + lane;
      const bool q_ok = q_mine < g.Sq;
      const long long stat = ((long long)b * g.Hq + hq) * g.Sq + q_mine;
      const float L_mine = q_ok ? lse[stat] * LOG2E : INFINITY;     // +inf: exp2(x - inf) = 0 for rows past the end
      const float d_mine = q_ok ? delta[stat] : 0.f;
      if (!mbar_wait(&ctl->sdp_full[st], ph, abort_flag, g.status, 550)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[32], dpv[32];
      tmem_ld32(tmem + 64 * st + lane_base + c_half * 32, sv);
      tmem_ld32(tmem + 128 + 64 * st + lane_base + c_half * 32, dpv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->sdp_empty[st]);              // this TMEM buffer may take iteration it + 2
      uint32_t pk[16], dsk[16];
      const int q0 = qb * BQT + c_half * 32;
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float pe[2], de[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float Lq = __shfl_sync(0xffffffffu, L_mine, j + e);
          const float dq_ = __shfl_sync(0xffffffffu, d_mine, j + e);
          const bool valid = kv_g < g.Sk && (!g.causal || kv_g <= q0 + j + e + off);
          const float p = valid ? exp2f(__uint_as_float(sv[j + e]) * sl2 - Lq) : 0.f;
          pe[e] = p;
          de[e] = p * (__uint_as_float(dpv[j + e]) - dq_);
        }
        pk[j >> 1] = pack_bf16x2(pe[0], pe[1]);
        dsk[j >> 1] = pack_bf16x2(de[0], de[1]);
      }
      if (!mbar_wait(&ctl->stage_free[st], ph ^ 1, abort_flag, g.status, 551)) { ok = false; break; }
      uint8_t* prow = sP + st * PT_TILE + r * 128;
      uint8_t* drow = sDS + st * PT_TILE + r * 128;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t o = (uint32_t)(((c_half * 4 + t) ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(prow + o) = make_uint4(pk[4 * t], pk[4 * t + 1], pk[4 * t + 2], pk[4 * t + 3]);
        *reinterpret_cast<uint4*>(drow + o) = make_uint4(dsk[4 * t], dsk[4 * t + 1], dsk[4 * t + 2], dsk[4 * t + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->pds_ready[st]);
    }
    // epilogue: this thread's key row of dV and dK, columns [64 * c_half, 64 * c_half + 64)
    const int c_lo = c_half * 2;
    const int kj = kv_g;
    const long long part_elems = (long long)g.Sk * g.B * g.Hk * D;
    float* pdv = g.hs > 1 ? g.part + (long long)hpart * part_elems + (((long long)kj * g.B + b) * g.Hk + hk) * D : nullptr;
    float* pdk = g.hs > 1 ? pdv + (long long)g.hs * part_elems : nullptr;
    if (ok && n_iter > 0) {
      if (mbar_wait(&ctl->acc_full, 0, abort_flag, g.status, 552)) {
        tc_fence_after();
        __nv_bfloat16* dvr = dv + (long long)kj * g.dv_s + (long long)b * g.dv_b + (long long)hk * g.dv_h;
        __nv_bfloat16* dkr = dk + (long long)kj * g.dk_s + (long long)b * g.dk_b + (long long)hk * g.dk_h;
#pragma unroll 1
        for (int c = c_lo; c < c_lo + 2; ++c) {
          uint32_t a[32], bb[32];
          tmem_ld32(tmem + 256 + lane_base + c * 32, a);
          tmem_ld32(tmem + 384 + lane_base + c * 32, bb);
          tmem_ld_wait();
          if (kj >= g.Sk) continue;
          if (g.hs > 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              reinterpret_cast<float4*>(pdv + c * 32)[j] = make_float4(__uint_as_float(a[4 * j]), __uint_as_float(a[4 * j + 1]),
                                                                       __uint_as_float(a[4 * j + 2]), __uint_as_float(a[4 * j + 3]));
              reinterpret_cast<float4*>(pdk + c * 32)[j] =
                  make_float4(__uint_as_float(bb[4 * j]) * g.scale, __uint_as_float(bb[4 * j + 1]) * g.scale,
                              __uint_as_float(bb[4 * j + 2]) * g.scale, __uint_as_float(bb[4 * j + 3]) * g.scale);
            }
          } else {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u, w;
              const int i0 = q4 * 8;
              u.x = pack_bf16x2(__uint_as_float(a[i0]), __uint_as_float(a[i0 + 1]));
              u.y = pack_bf16x2(__uint_as_float(a[i0 + 2]), __uint_as_float(a[i0 + 3]));
              u.z = pack_bf16x2(__uint_as_float(a[i0 + 4]), __uint_as_float(a[i0 + 5]));
              u.w = pack_bf16x2(__uint_as_float(a[i0 + 6]), __uint_as_float(a[i0 + 7]));
              w.x = pack_bf16x2(__uint_as_float(bb[i0]) * g.scale, __uint_as_float(bb[i0 + 1]) * g.scale);
              w.y = pack_bf16x2(__uint_as_float(bb[i0 + 2]) * g.scale, __uint_as_float(bb[i0 + 3]) * g.scale);
              w.z = pack_bf16x2(__uint_as_float(bb[i0 + 4]) * g.scale, __uint_as_float(bb[i0 + 5]) * g.scale);
              w.w = pack_bf16x2(__uint_as_float(bb[i0 + 6]) * g.scale, __uint_as_float(bb[i0 + 7]) * g.scale);
              reinterpret_cast<uint4*>(dvr + c * 32)[q4] = u;
              reinterpret_cast<uint4*>(dkr + c * 32)[q4] = w;
            }
          }
        }
      }
    } else if (n_iter == 0 && kj < g.Sk) {
      // no query sees these keys: zero gradients (each warp half clears its own 64 columns)
      if (g.hs > 1) {
        for (int i = c_lo * 8; i < c_lo * 8 + 16; ++i) {
          reinterpret_cast<float4*>(pdv)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          reinterpret_cast<float4*>(pdk)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      } else {
        __nv_bfloat16* dvr = dv + (long long)kj * g.dv_s + (long long)b * g.dv_b + (long long)hk * g.dv_h;
        __nv_bfloat16* dkr = dk + (long long)kj * g.dk_s + (long long)b * g.dk_b + (long long)hk * g.dk_h;
        for (int i = c_lo * 4; i < c_lo * 4 + 8; ++i) {
          reinterpret_cast<uint4*>(dvr)[i] = make_uint4(0, 0, 0, 0);
          reinterpret_cast<uint4*>(dkr)[i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// Sums the `hs` fp32 partials of a head-split backward and writes bf16 dK / dV.
// One thread per 8 consecutive head-dim elements of one (key, batch, KV head) row of dV and of dK.
__global__ void __launch_bounds__(256) attn_dkv_reduce_kernel(const float* __restrict__ part, int hs, __nv_bfloat16* __restrict__ dk,
                                                              __nv_bfloat16* __restrict__ dv, int Sk, int B, int Hk, long long dk_s,
                                                              long long dk_b, long long dk_h, long long dv_s, long long dv_b,
                                                              long long dv_h) {
  const long long nvec = (long long)Sk * B * Hk * (D / 8);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * nvec) return;
  const int which = i >= nvec;                  // 0: dV, 1: dK
  const long long v = which ? i - nvec : i;
  const int c8 = (int)(v % (D / 8));
  const long long row = v / (D / 8);            // (kj * B + b) * Hk + hk
  const int hk = (int)(row % Hk), b = (int)((row / Hk) % B);
  const long long kj = row / ((long long)Hk * B);
  const long long part_elems = (long long)Sk * B * Hk * D;
  const float* src = part + (long long)which * hs * part_elems + row * D + c8 * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int h = 0; h < hs; ++h) {
    const float4 x = *reinterpret_cast<const float4*>(src + (long long)h * part_elems);
    const float4 y = *reinterpret_cast<const float4*>(src + (long long)h * part_elems + 4);
    acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w;
    acc[4] += y.x; acc[5] += y.y; acc[6] += y.z; acc[7] += y.w;
  }
  __nv_bfloat16* dst = which ? dk + kj * dk_s + b * dk_b + hk * dk_h : dv + kj * dv_s + b * dv_b + hk * dv_h;
  reinterpret_cast<uint4*>(dst)[c8] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                                                 pack_bf16x2(acc[6], acc[7]));
}

// ----------------------------------------------------------------------- backward, dQ
// One CTA per (128 query rows, batch, query head); it loops over the key blocks these
// queries see, recomputes S = Q K^T and dP = dO V^T, forms dS = P (dP - delta) and
// accumulates dQ += dS K in TMEM over the whole loop, so that no atomics and no fp32 scratch
// are needed for dQ (two extra MMAs per tile pair buy that).
struct DqCtl {
  uint64_t qdo_full;
  uint64_t kv_full[2], kv_empty[2];
  uint64_t sdp_full, ds_ready, dq_full;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int DQ_SMEM = TILE_BYTES * 7 + 1024 + 256;    // Q, dO, K x2, V x2, dS

struct DqGeometry {
  int B, Hq, Hk, Sq, Sk, causal;
  float scale;
  long long dq_s, dq_b, dq_h;
  DeviceStatus* status;
  int x0, p0, ny;                 // as in Geometry; ny = Hq
};

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                   const __grid_constant__ CUtensorMap tdo, const float* __restrict__ lse, const float* __restrict__ delta,
                   __nv_bfloat16* __restrict__ dq, const DqGeometry g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;
  uint8_t* sV = smem + 4 * TILE_BYTES;
  uint8_t* sDS = smem + 6 * TILE_BYTES;
  DqCtl* ctl = reinterpret_cast<DqCtl*>(smem + 7 * TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (g.Sq + BQ - 1) / BQ;
  const int qb = nqb - 1 - (g.x0 + (int)blockIdx.x);
  const int pyz = g.p0 + (int)blockIdx.y + (int)blockIdx.z * (int)gridDim.y;
  const int hq = pyz % g.ny, b = pyz / g.ny;
  const int hk = hq / (g.Hq / g.Hk);
  const int off = g.Sk - g.Sq;
  int nblk = (g.Sk + BKV - 1) / BKV;
  if (g.causal) {
    const int last_key = qb * BQ + BQ - 1 + off;
    nblk = last_key < 0 ? 0 : min(nblk, last_key / BKV + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(&ctl->qdo_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->kv_full[i], 1); mbar_init(&ctl->kv_empty[i], 1); }
    mbar_init(&ctl->sdp_full, 1); mbar_init(&ctl->ds_ready, 8); mbar_init(&ctl->dq_full, 1);
    ctl->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ctl->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  // TMEM columns: [0,128) S, [128,256) dP, [256,384) dQ

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv); tma_prefetch_desc(&tdo);
      mbar_expect_tx(&ctl->qdo_full, 2 * TILE_BYTES);
      tma_load_4d(sQ, &tq, &ctl->qdo_full, 0, hq, b, qb * BQ);
      tma_load_4d(sQ + HALF_BYTES, &tq, &ctl->qdo_full, 64, hq, b, qb * BQ);
      tma_load_4d(sDO, &tdo, &ctl->qdo_full, 0, hq, b, qb * BQ);
      tma_load_4d(sDO + HALF_BYTES, &tdo, &ctl->qdo_full, 64, hq, b, qb * BQ);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&ctl->kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, g.status, 800)) break;
        mbar_expect_tx(&ctl->kv_full[s], 2 * TILE_BYTES);
        tma_load_4d(sK + s * TILE_BYTES, &tk, &ctl->kv_full[s], 0, hk, b, j * BKV);
        tma_load_4d(sK + s * TILE_BYTES + HALF_BYTES, &tk, &ctl->kv_full[s], 64, hk, b, j * BKV);
        tma_load_4d(sV + s * TILE_BYTES, &tv, &ctl->kv_full[s], 0, hk, b, j * BKV);
        tma_load_4d(sV + s * TILE_BYTES + HALF_BYTES, &tv, &ctl->kv_full[s], 64, hk, b, j * BKV);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t id_kk = umma_idesc_bf16(128, 128, 0, 0);   // S, dP
      constexpr uint32_t id_km = umma_idesc_bf16(128, 128, 0, 1);   // dQ: dS K-major, K MN-major
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), ds_base = smem_u32(sDS);
      bool ok = mbar_wait(&ctl->qdo_full, 0, abort_flag, g.status, 810);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&ctl->kv_full[s], (j >> 1) & 1, abort_flag, g.status, 811)) break;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sK + s * TILE_BYTES), v_base = smem_u32(sV + s * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 0, desc_kmajor(q_base, kk), desc_kmajor(k_base, kk), id_kk, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 128, desc_kmajor(do_base, kk), desc_kmajor(v_base, kk), id_kk, kk > 0);
        umma_commit(&ctl->sdp_full);
        if (!mbar_wait(&ctl->ds_ready, j & 1, abort_flag, g.status, 812)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_bf16(tmem + 256, desc_kmajor(ds_base, kk), desc_mnmajor(k_base, kk), id_km, (j | kk) != 0);
        umma_commit(&ctl->kv_empty[s]);
      }
      if (ok) umma_commit(&ctl->dq_full);
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int c_lo = ((warp - 2) >> 2) * 2;
    const int r = quarter * 32 + lane;
    const int qi = qb * BQ + r;
    const bool row_ok = qi < g.Sq;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float sl2 = g.scale * LOG2E;
    const long long stat = ((long long)b * g.Hq + hq) * g.Sq + qi;
    const float L = row_ok ? lse[stat] * LOG2E : 0.f;
    const float dl = row_ok ? delta[stat] : 0.f;
    bool ok = nblk > 0;
    for (int j = 0; j < nblk && ok; ++j) {
      if (!mbar_wait(&ctl->sdp_full, j & 1, abort_flag, g.status, 820)) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * BKV;
      int limit = g.Sk - key0;
      if (g.causal) limit = min(limit, qi + off - key0 + 1);
      if (!row_ok) limit = 0;
#pragma unroll 1
      for (int c = c_lo; c < c_lo + 2; ++c) {
        uint32_t sv[32], dpv[32];
        tmem_ld32(tmem + 0 + lane_base + c * 32, sv);
        tmem_ld32(tmem + 128 + lane_base + c * 32, dpv);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float ds[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int col = c * 32 + q4 * 8 + i;
            float pe = exp2f(__uint_as_float(sv[q4 * 8 + i]) * sl2 - L);
            if (col >= limit) pe = 0.f;
            ds[i] = pe * (__uint_as_float(dpv[q4 * 8 + i]) - dl);
          }
          uint4 ud;
          ud.x = pack_bf16x2(ds[0], ds[1]); ud.y = pack_bf16x2(ds[2], ds[3]); ud.z = pack_bf16x2(ds[4], ds[5]); ud.w = pack_bf16x2(ds[6], ds[7]);
          *reinterpret_cast<uint4*>(sDS + swz_off(r, c * 4 + q4)) = ud;
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->ds_ready);
    }
    __nv_bfloat16* dqr = dq + (long long)qi * g.dq_s + (long long)b * g.dq_b + (long long)hq * g.dq_h;
    if (ok && nblk > 0) {
      if (mbar_wait(&ctl->dq_full, 0, abort_flag, g.status, 821)) {
        tc_fence_after();
#pragma unroll 1
        for (int c = c_lo; c < c_lo + 2; ++c) {
          uint32_t a[32];
          tmem_ld32(tmem + 256 + lane_base + c * 32, a);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 u;
              const int i0 = q4 * 8;
              u.x = pack_bf16x2(__uint_as_float(a[i0]) * g.scale, __uint_as_float(a[i0 + 1]) * g.scale);
              u.y = pack_bf16x2(__uint_as_float(a[i0 + 2]) * g.scale, __uint_as_float(a[i0 + 3]) * g.scale);
              u.z = pack_bf16x2(__uint_as_float(a[i0 + 4]) * g.scale, __uint_as_float(a[i0 + 5]) * g.scale);
              u.w = pack_bf16x2(__uint_as_float(a[i0 + 6]) * g.scale, __uint_as_float(a[i0 + 7]) * g.scale);
              reinterpret_cast<uint4*>(dqr + c * 32)[q4] = u;
            }
          }
        }
      }
    } else if (nblk == 0 && row_ok && c_lo == 0) {
      for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(dqr)[i] = make_uint4(0, 0, 0, 0);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}


static const CUtensorMap* tensor_map_sbhd(const void* p, int S, int B, int H, long long s_s, long long s_b, long long s_h,
                                          uint32_t box_rows = 128) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)B, (uint64_t)S};
  const uint64_t st[3] = {(uint64_t)s_h * 2, (uint64_t)s_b * 2, (uint64_t)s_s * 2};
  const uint32_t box[4] = {64, 1, 1, box_rows};
  return get_tmap_4d(p, 2, dims, st, box, true);
}

}  // namespace attn
}  // namespace dh

using namespace dh;
using namespace dh::attn;

// dK/dV kernel choice of dh_attn_bwd: -1 = read DHELLAM_ATTN_BWD_T on first use, 0 = attn_bwd_kernel, 1 = attn_bwd_t_kernel
static int g_bwd_mode = -1;

// SM budget for kernels whose grid is one CTA per tile (one CTA per SM by shared memory): the (X, Y, Z) grid is cut
// into launches of at most `budget` CTAs, which the stream runs one after the other, so at most `budget` SMs are in
// use at any time.  launch(grid, x0, p0) starts tile columns x0.. and flattened (y, z) pairs p0..
template <class F>
static void launch_in_waves(int X, int Y, int Z, int sm_budget, F&& launch) {
  const int sms = dh_sm_count();
  const int budget = (sm_budget <= 0 || sm_budget >= sms) ? 0 : sm_budget;
  const long long pairs = (long long)Y * Z;
  if (budget == 0 || (long long)X * pairs <= budget) {
    launch(dim3(X, Y, Z), 0, 0);
    return;
  }
  if (X >= budget) {
    for (long long p = 0; p < pairs; ++p)
      for (int x0 = 0; x0 < X; x0 += budget) launch(dim3(X - x0 < budget ? X - x0 : budget, 1, 1), x0, (int)p);
  } else {
    const int np = budget / X;
    for (long long p0 = 0; p0 < pairs; p0 += np) launch(dim3(X, (unsigned)(pairs - p0 < np ? pairs - p0 : np), 1), 0, (int)p0);
  }
}

extern "C" {

void dh_attn_set_bwd_mode(int mode) { g_bwd_mode = mode; }

int dh_attn_fwd(const void* q, const void* k, const void* v, void* out, void* lse, int64_t q_s, int64_t q_b, int64_t q_h, int64_t k_s,
                int64_t k_b, int64_t k_h, int64_t v_s, int64_t v_b, int64_t v_h, int B, int Hq, int Hk, int Sq, int Sk, int d, int causal,
                float scale, int sm_budget, cudaStream_t stream) {
  if (d != D) { set_last_error("dh_attn_fwd: head size %d is not supported (128 only)", d); return (int)cudaErrorInvalidValue; }
  if (Hq % Hk != 0) { set_last_error("dh_attn_fwd: query heads must be a multiple of KV heads"); return (int)cudaErrorInvalidValue; }
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  const CUtensorMap* tq = tensor_map_sbhd(q, Sq, B, Hq, q_s, q_b, q_h);
  const CUtensorMap* tk = tensor_map_sbhd(k, Sk, B, Hk, k_s, k_b, k_h);
  const CUtensorMap* tv = tensor_map_sbhd(v, Sk, B, Hk, v_s, v_b, v_h);
  if (!tq || !tk || !tv) return (int)cudaErrorInvalidValue;
  static PerDeviceFlags configured_on;
  bool& configured = device_flag(configured_on);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) { set_last_error("dh_attn_fwd: shared memory opt-in failed: %s", cudaGetErrorString(e)); return (int)e; }
    configured = true;
  }
  Geometry g;
  g.B = B; g.Hq = Hq; g.Hk = Hk; g.Sq = Sq; g.Sk = Sk; g.causal = causal; g.scale = scale;
  g.o_h = D; g.o_b = (long long)Hq * D; g.o_s = (long long)B * Hq * D;
  g.status = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  g.ny = Hq;
  launch_in_waves((Sq + BQ - 1) / BQ, Hq, B, sm_budget, [&](dim3 grid, int x0, int p0) {
    g.x0 = x0; g.p0 = p0;
    attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, stream>>>(*tq, *tk, *tv, (__nv_bfloat16*)out, (float*)lse, g);
  });
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_attn_fwd launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

// Number of CTAs that share the query heads of one KV head in the dK/dV kernel: 1 while
// KV blocks x batch x KV heads already give every SM a few CTAs, else the smallest power of
// two (dividing the group size) that does.
static int bwd_head_split(int B, int Hq, int Hk, int Sk) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("DHELLAM_ATTN_HEAD_SPLIT");
    enabled = e ? atoi(e) : 1;
  }
  if (!enabled) return 1;
  const int group = Hq / Hk;
  const long long ctas = (long long)((Sk + BKV - 1) / BKV) * B * Hk;
  int hs = 1;
  while (hs < group && group % (hs * 2) == 0 && ctas * hs < 4LL * dh_sm_count()) hs *= 2;
  return hs;
}

// Scratch: delta [B*Hq*Sq] fp32 (row dot products of dO and O), rounded up to 256 bytes, then, when
// the dK/dV kernel splits heads, the fp32 partials [2][hs][Sk][B][Hk][128].
int64_t dh_attn_bwd_scratch_bytes(int B, int Hq, int Hk, int Sq, int Sk) {
  int64_t n = ((int64_t)B * Hq * Sq * 4 + 255) / 256 * 256;
  if (Hk > 0 && Hq % Hk == 0) {
    const int hs = bwd_head_split(B, Hq, Hk, Sk);
    if (hs > 1) n += (int64_t)2 * hs * Sk * B * Hk * D * 4;
  }
  return n;
}

int dh_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out, const void* lse, void* dq, void* dk,
                void* dv, void* scratch, const int64_t* strides /* 8 tensors x (s,b,h): do,q,k,v,o,dq,dk,dv */, int B, int Hq, int Hk,
                int Sq, int Sk, int d, int causal, float scale, int sm_budget, cudaStream_t stream) {
  if (d != D) { set_last_error("dh_attn_bwd: head size %d is not supported (128 only)", d); return (int)cudaErrorInvalidValue; }
  if (Hq % Hk != 0) { set_last_error("dh_attn_bwd: query heads must be a multiple of KV heads"); return (int)cudaErrorInvalidValue; }
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  const int64_t* sdo = strides; const int64_t* sq = strides + 3; const int64_t* sk = strides + 6; const int64_t* sv = strides + 9;
  const int64_t* so = strides + 12; const int64_t* sdq = strides + 15; const int64_t* sdk = strides + 18; const int64_t* sdv = strides + 21;
  const CUtensorMap* tq = tensor_map_sbhd(q, Sq, B, Hq, sq[0], sq[1], sq[2]);
  const CUtensorMap* tk = tensor_map_sbhd(k, Sk, B, Hk, sk[0], sk[1], sk[2]);
  const CUtensorMap* tv = tensor_map_sbhd(v, Sk, B, Hk, sv[0], sv[1], sv[2]);
  const CUtensorMap* tdo = tensor_map_sbhd(dout, Sq, B, Hq, sdo[0], sdo[1], sdo[2]);
  if (!tq || !tk || !tv || !tdo) return (int)cudaErrorInvalidValue;
  static PerDeviceFlags configured_on;
  bool& configured = device_flag(configured_on);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM);
    if (e != cudaSuccess) { set_last_error("dh_attn_bwd: shared memory opt-in failed: %s", cudaGetErrorString(e)); return (int)e; }
    configured = true;
  }
  float* delta = reinterpret_cast<float*>(scratch);
  const long long rows_ll = (long long)B * Hq * Sq;
  if (rows_ll > (1ll << 26)) {     // the delta grid (one warp per row) and the int row index stay well inside 32 bits
    set_last_error("dh_attn_bwd: B*Hq*Sq = %lld rows exceed the supported 2^26", rows_ll);
    return (int)cudaErrorInvalidValue;
  }
  const int rows = (int)rows_ll;
  attn_delta_kernel<<<(unsigned)((rows_ll * 32 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, B, Hq, Sq,
                                                                 sdo[0], sdo[1], sdo[2], so[0], so[1], so[2]);
  DeviceStatus* st = reinterpret_cast<DeviceStatus*>(dh_status_device_ptr());
  BwdGeometry g;
  g.B = B; g.Hq = Hq; g.Hk = Hk; g.Sq = Sq; g.Sk = Sk; g.causal = causal; g.scale = scale;
  g.dk_s = sdk[0]; g.dk_b = sdk[1]; g.dk_h = sdk[2]; g.dv_s = sdv[0]; g.dv_b = sdv[1]; g.dv_h = sdv[2];
  g.status = st;
  g.hs = bwd_head_split(B, Hq, Hk, Sk);
  g.part = g.hs > 1 ? reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + ((int64_t)rows * 4 + 255) / 256 * 256) : nullptr;
  g.x0 = 0; g.p0 = 0; g.ny = Hk * g.hs;
  // DHELLAM_ATTN_BWD_T=1 (or dh_attn_set_bwd_mode(1)) selects the pipelined (transposed-score) form of the dK/dV kernel
  if (g_bwd_mode < 0) {
    const char* ev = getenv("DHELLAM_ATTN_BWD_T");
    g_bwd_mode = ev ? atoi(ev) : 0;
  }
  if (g_bwd_mode == 1) {
    const CUtensorMap* tq64 = tensor_map_sbhd(q, Sq, B, Hq, sq[0], sq[1], sq[2], BQT);
    const CUtensorMap* tdo64 = tensor_map_sbhd(dout, Sq, B, Hq, sdo[0], sdo[1], sdo[2], BQT);
    if (!tq64 || !tdo64) return (int)cudaErrorInvalidValue;
    static PerDeviceFlags configured_t_on;
    bool& configured_t = device_flag(configured_t_on);
    if (!configured_t) {
      cudaError_t e2 = cudaFuncSetAttribute(attn_bwd_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWDT_SMEM);
      if (e2 != cudaSuccess) { set_last_error("dh_attn_bwd: shared memory opt-in failed: %s", cudaGetErrorString(e2)); return (int)e2; }
      configured_t = true;
    }
    launch_in_waves((Sk + BKV - 1) / BKV, Hk * g.hs, B, sm_budget, [&](dim3 grid, int x0, int p0) {
      g.x0 = x0; g.p0 = p0;
      attn_bwd_t_kernel<<<grid, BWD_THREADS, BWDT_SMEM, stream>>>(*tq64, *tk, *tv, *tdo64, (const float*)lse, delta, (__nv_bfloat16*)dk,
                                                                  (__nv_bfloat16*)dv, g);
    });
  } else {
    launch_in_waves((Sk + BKV - 1) / BKV, Hk * g.hs, B, sm_budget, [&](dim3 grid, int x0, int p0) {
      g.x0 = x0; g.p0 = p0;
      attn_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, stream>>>(*tq, *tk, *tv, *tdo, (const float*)lse, delta, (__nv_bfloat16*)dk,
                                                               (__nv_bfloat16*)dv, g);
    });
  }
  if (g.hs > 1) {
    const long long n = 2LL * Sk * B * Hk * (D / 8);
    attn_dkv_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(g.part, g.hs, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, Sk, B, Hk,
                                                                           sdk[0], sdk[1], sdk[2], sdv[0], sdv[1], sdv[2]);
  }
  DqGeometry gq;
  gq.B = B; gq.Hq = Hq; gq.Hk = Hk; gq.Sq = Sq; gq.Sk = Sk; gq.causal = causal; gq.scale = scale;
  gq.dq_s = sdq[0]; gq.dq_b = sdq[1]; gq.dq_h = sdq[2];
  gq.status = st;
  gq.ny = Hq;
  launch_in_waves((Sq + BQ - 1) / BQ, Hq, B, sm_budget, [&](dim3 grid, int x0, int p0) {
    gq.x0 = x0; gq.p0 = p0;
    attn_bwd_dq_kernel<<<grid, BWD_THREADS, DQ_SMEM, stream>>>(*tq, *tk, *tv, *tdo, (const float*)lse, delta, (__nv_bfloat16*)dq, gq);
  });
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_attn_bwd launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}

}  // extern "C"

// =========================================================================== no-allocation entry
#include "attn_noalloc.h"

namespace dh {
bool encode_tmap_4d_into(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims[4], const uint64_t strides_bytes[3],
                         const uint32_t box[4], bool swizzle128);
namespace attn {

// Scratch of the no-allocation entry point.  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels receive the resolved device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[DH_ATTN_NOALLOC_SCRATCH_BYTES];

constexpr int kNoallocMaxDev = 32;
static void* g_noalloc_addr[kNoallocMaxDev] = {nullptr};
static bool g_noalloc_ready[kNoallocMaxDev] = {false};
static std::mutex g_noalloc_mutex;     // two host threads may make the first call on one device at the same time

static bool map_sbhd_into(CUtensorMap* m, const void* p, int S, int B, int H, const int64_t* st) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)B, (uint64_t)S};
  const uint64_t sb[3] = {(uint64_t)st[2] * 2, (uint64_t)st[1] * 2, (uint64_t)st[0] * 2};
  const uint32_t box[4] = {64, 1, 1, 128};
  return encode_tmap_4d_into(m, p, 2, dims, sb, box, true);
}

}  // namespace attn
}  // namespace dh

extern "C" int dh_attn_bwd_noalloc(const void* dout, const void* q, const void* k, const void* v, const void* out, const void* lse,
                                   void* dq, void* dk, void* dv, const int64_t* strides, int B, int Hq, int Hk, int Sq, int Sk, int d,
                                   int causal, float scale, cudaStream_t stream) {
  if (d != D) { set_last_error("dh_attn_bwd_noalloc: head size %d is not supported (128 only)", d); return (int)cudaErrorInvalidValue; }
  if (Hk <= 0 || Hq % Hk != 0) { set_last_error("dh_attn_bwd_noalloc: query heads must be a multiple of KV heads"); return (int)cudaErrorInvalidValue; }
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  const int64_t rows = (int64_t)B * Hq * Sq;
  const int64_t need = (rows * 4 + 255) / 256 * 256;
  if (need > (int64_t)DH_ATTN_NOALLOC_SCRATCH_BYTES) {
    set_last_error("dh_attn_bwd_noalloc: B*Hq*Sq = %lld rows need %lld bytes of scratch, the built-in array holds %u; "
                   "use dh_attn_bwd with a caller-provided buffer", (long long)rows, (long long)need, DH_ATTN_NOALLOC_SCRATCH_BYTES);
    return (int)cudaErrorInvalidValue;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kNoallocMaxDev) { set_last_error("dh_attn_bwd_noalloc: no usable current device"); return (int)cudaErrorInvalidDevice; }
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ready[dev]) {
    // once per device, with that device current: resolve the array's device address
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) { set_last_error("dh_attn_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e)); return (int)e; }
    e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM);
    if (e != cudaSuccess) { set_last_error("dh_attn_bwd_noalloc: shared memory opt-in failed: %s", cudaGetErrorString(e)); return (int)e; }
    g_noalloc_addr[dev] = ptr;
    g_noalloc_ready[dev] = true;
  }
  }
  const int64_t* sdo = strides; const int64_t* sq = strides + 3; const int64_t* sk = strides + 6; const int64_t* sv = strides + 9;
  const int64_t* so = strides + 12; const int64_t* sdq = strides + 15; const int64_t* sdk = strides + 18; const int64_t* sdv = strides + 21;
  CUtensorMap tq, tk, tv, tdo;
  if (!map_sbhd_into(&tq, q, Sq, B, Hq, sq) || !map_sbhd_into(&tk, k, Sk, B, Hk, sk) || !map_sbhd_into(&tv, v, Sk, B, Hk, sv) ||
      !map_sbhd_into(&tdo, dout, Sq, B, Hq, sdo))
    return (int)cudaErrorInvalidValue;
  // delta is fully rewritten by every call, so nothing in the shared array needs clearing
  float* delta = reinterpret_cast<float*>(g_noalloc_addr[dev]);
  attn_delta_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, B,
                                                                             Hq, Sq, sdo[0], sdo[1], sdo[2], so[0], so[1], so[2]);
  BwdGeometry g;
  g.B = B; g.Hq = Hq; g.Hk = Hk; g.Sq = Sq; g.Sk = Sk; g.causal = causal; g.scale = scale;
  g.dk_s = sdk[0]; g.dk_b = sdk[1]; g.dk_h = sdk[2]; g.dv_s = sdv[0]; g.dv_b = sdv[1]; g.dv_h = sdv[2];
  g.status = nullptr;
  g.hs = 1;              // the built-in scratch holds delta only: no head split here
  g.part = nullptr;
  g.x0 = 0; g.p0 = 0; g.ny = Hk;
  attn_bwd_kernel<<<dim3((Sk + BKV - 1) / BKV, Hk, B), BWD_THREADS, BWD_SMEM, stream>>>(tq, tk, tv, tdo, (const float*)lse, delta,
                                                                                      (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, g);
  DqGeometry gq;
  gq.B = B; gq.Hq = Hq; gq.Hk = Hk; gq.Sq = Sq; gq.Sk = Sk; gq.causal = causal; gq.scale = scale;
  gq.dq_s = sdq[0]; gq.dq_b = sdq[1]; gq.dq_h = sdq[2];
  gq.status = nullptr;
  gq.x0 = 0; gq.p0 = 0; gq.ny = Hq;
  attn_bwd_dq_kernel<<<dim3((Sq + BQ - 1) / BQ, Hq, B), BWD_THREADS, DQ_SMEM, stream>>>(tq, tk, tv, tdo, (const float*)lse, delta,
                                                                                      (__nv_bfloat16*)dq, gq);
  e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error("dh_attn_bwd_noalloc launch failed: %s", cudaGetErrorString(e));
  return (int)e;
}
