// Head-block and optimizer kernels for sm_100a: vocabulary-parallel embedding forward /
// backward, single-pass cross-entropy statistics and in-place logit gradient, the MoE
// router (logits + softmax + top-k + gate normalisation in one pass), fused Adam over flat
// buffers, and a sum-of-squares reduction for gradient clipping.
//
// Roles in the reference: dhellam/operators/embedding.py:16-49 (embedding),
// dhellam/operators/loss.py:15-127 (cross entropy with three all-reduces; here one pass
// produces the per-rank triple that a single exchange combines), Megatron's optimizer
// (script/run.sh:108-127).  The router has no counterpart in the reference.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

namespace dh {

constexpr int HT = 256;

__device__ __forceinline__ float hwarp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float hwarp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void h_unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 h_pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]); u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
static inline int h_grid(long long items, int per_sm, int sm_budget) {
  int sms = dh_sm_count();
  int budget = (sm_budget <= 0 || sm_budget > sms) ? sms : sm_budget;
  long long g = (long long)budget * per_sm;
  if (items < g) g = items;
  return g < 1 ? 1 : (int)g;
}
static inline int h_rc(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error_c(what, cudaGetErrorString(e));
  return (int)e;
}

// ============================================================================ embedding
__global__ void __launch_bounds__(HT) embedding_fwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ out, int T, int h, int Vl, int v0) {
  const int nvec = h >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const int loc = tok[t] - v0;
    uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * h);
    if (loc >= 0 && loc < Vl) {
      const uint4* src = reinterpret_cast<const uint4*>(w + (size_t)loc * h);
      for (int c = threadIdx.x; c < nvec; c += HT) o[c] = src[c];
    } else {
      for (int c = threadIdx.x; c < nvec; c += HT) o[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

__global__ void __launch_bounds__(HT) embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ tok,
                                                           float* __restrict__ grad, int T, int h, int Vl, int v0) {
  const int nvec = h >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const int loc = tok[t] - v0;
    if (loc < 0 || loc >= Vl) continue;
    const uint4* src = reinterpret_cast<const uint4*>(dout + (size_t)t * h);
    float* dst = grad + (size_t)loc * h;
    for (int c = threadIdx.x; c < nvec; c += HT) {
      float v[8];
      h_unpack8(ld_nc_v4(src + c), v);
      atomicAdd(reinterpret_cast<float4*>(dst + c * 8), make_float4(v[0], v[1], v[2], v[3]));
      atomicAdd(reinterpret_cast<float4*>(dst + c * 8 + 4), make_float4(v[4], v[5], v[6], v[7]));
    }
  }
}

// Reproducible form: `order` is a stable sort of the token positions by token id and `sorted_tok` the ids in that
// order; the CTA that meets the first position of a token adds all of that token's rows in sorted order and
// writes the row of the gradient once (no two CTAs touch the same row, nothing depends on timing).
__global__ void __launch_bounds__(HT) embedding_bwd_sorted_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ order,
                                                                  const int* __restrict__ sorted_tok, float* __restrict__ grad, int T, int h,
                                                                  int Vl, int v0) {
  const int nvec = h >> 3;
  for (int i = blockIdx.x; i < T; i += gridDim.x) {
    const int tk = sorted_tok[i];
    if (i > 0 && sorted_tok[i - 1] == tk) continue;          // not the first position of this token
    const int loc = tk - v0;
    if (loc < 0 || loc >= Vl) continue;
    float* dst = grad + (size_t)loc * h;
    for (int c = threadIdx.x; c < nvec; c += HT) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = i; j < T && sorted_tok[j] == tk; ++j) {
        float v[8];
        h_unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(dout + (size_t)order[j] * h) + c), v);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += v[q];
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) dst[c * 8 + q] += acc[q];
    }
  }
}

// ============================================================================ cross entropy
// One CTA per token row; online (max, sum-exp) in a single pass over the vocabulary shard.
template <bool F32>
__global__ void __launch_bounds__(HT) ce_stats_kernel(const void* __restrict__ logits, const int* __restrict__ labels,
                                                      float* __restrict__ stats, int T, int Vl, long long ld, int v0) {
  __shared__ float sm[32], ss[32], st[32];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    float m = -FLT_MAX, s = 0.f, tot = 0.f;      // tot: plain sum of the logits (label smoothing)
    if (F32) {
      const float* row = reinterpret_cast<const float*>(logits) + (size_t)t * ld;
      for (int c = threadIdx.x; c < Vl; c += HT) {
        const float v = row[c];
        tot += v;
        const float nm = fmaxf(m, v);
        s = s * __expf(m - nm) + __expf(v - nm);
        m = nm;
      }
    } else {
      const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(logits) + (size_t)t * ld;
      const int nvec = Vl >> 3;
      for (int c = threadIdx.x; c < nvec; c += HT) {
        float v[8];
        h_unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(row) + c), v);
        float lm = v[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) lm = fmaxf(lm, v[j]);
        const float nm = fmaxf(m, lm);
        float add = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { add += __expf(v[j] - nm); tot += v[j]; }
        s = s * __expf(m - nm) + add;
        m = nm;
      }
      for (int c = (nvec << 3) + threadIdx.x; c < Vl; c += HT) {
        const float v = __bfloat162float(row[c]);
        tot += v;
        const float nm = fmaxf(m, v);
        s = s * __expf(m - nm) + __expf(v - nm);
        m = nm;
      }
    }
    // combine (m, s, tot) over the CTA
    const float wm = hwarp_max(m);
    s = hwarp_sum(s * __expf(m - wm));
    tot = hwarp_sum(tot);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) { sm[w] = wm; ss[w] = s; st[w] = tot; }
    __syncthreads();
    if (w == 0) {
      float pm = l < (HT >> 5) ? sm[l] : -FLT_MAX;
      float ps = l < (HT >> 5) ? ss[l] : 0.f;
      const float pt = hwarp_sum(l < (HT >> 5) ? st[l] : 0.f);
      const float gm = hwarp_max(pm);
      ps = hwarp_sum(ps * __expf(pm - gm));
      if (l == 0) {
        const int loc = labels[t] - v0;
        float tgt = 0.f;
        if (loc >= 0 && loc < Vl) {
          tgt = F32 ? reinterpret_cast<const float*>(logits)[(size_t)t * ld + loc]
                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[(size_t)t * ld + loc]);
        }
        stats[t * 4 + 0] = gm;
        stats[t * 4 + 1] = ps;
        stats[t * 4 + 2] = tgt;
        stats[t * 4 + 3] = pt;
      }
    }
  }
}

template <bool F32>
__global__ void __launch_bounds__(HT) ce_grad_kernel(void* __restrict__ logits, const int* __restrict__ labels, const float* __restrict__ lse,
                                                     const float* __restrict__ gtok, int T, int Vl, long long ld, int v0,
                                                     float tcoef, float ucoef) {
  // d loss / d logit = softmax - tcoef * onehot(target) - ucoef; plain cross-entropy has tcoef = 1, ucoef = 0,
  // label smoothing s over V classes has tcoef = 1 - s', ucoef = s' / V with s' = s V / (V - 1).
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const float L = lse[t], g = gtok[t];
    const int loc = labels[t] - v0;
    if (F32) {
      float* row = reinterpret_cast<float*>(logits) + (size_t)t * ld;
      for (int c = threadIdx.x; c < Vl; c += HT) row[c] = (__expf(row[c] - L) - (c == loc ? tcoef : 0.f) - ucoef) * g;
    } else {
      __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(logits) + (size_t)t * ld;
      const int nvec = Vl >> 3;
      for (int c = threadIdx.x; c < nvec; c += HT) {
        float v[8];
        uint4* p = reinterpret_cast<uint4*>(row) + c;
        h_unpack8(*p, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (__expf(v[j] - L) - ((c * 8 + j) == loc ? tcoef : 0.f) - ucoef) * g;
        *p = h_pack8(v);
      }
      for (int c = (nvec << 3) + threadIdx.x; c < Vl; c += HT)
        row[c] = __float2bfloat16((__expf(__bfloat162float(row[c]) - L) - (c == loc ? tcoef : 0.f) - ucoef) * g);
    }
  }
}

// ============================================================================ router
// One warp per token: logits over E experts (E <= 64), softmax, top-k, normalised gates.
__global__ void __launch_bounds__(HT) router_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                    float* __restrict__ probs, int* __restrict__ topi, float* __restrict__ gates, int T,
                                                    int h, int E, int k) {
  __shared__ float slog[HT / 32][64];
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = h >> 3;
  for (int t = blockIdx.x * (HT / 32) + wid; t < T; t += gridDim.x * (HT / 32)) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)t * h);
    for (int e0 = 0; e0 < E; e0 += 8) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int c = lane; c < nvec; c += 32) {
        float xv[8];
        h_unpack8(xr[c], xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (e0 + j < E) {
            float wv[8];
            h_unpack8(reinterpret_cast<const uint4*>(w + (size_t)(e0 + j) * h)[c], wv);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[j] += xv[q] * wv[q];
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = hwarp_sum(acc[j]);
        if (lane == 0 && e0 + j < E) slog[wid][e0 + j] = v;
      }
    }
    __syncwarp();
    // softmax over E (lanes cover e and e+32)
    const float l0 = lane < E ? slog[wid][lane] : -FLT_MAX;
    const float l1 = lane + 32 < E ? slog[wid][lane + 32] : -FLT_MAX;
    const float mx = hwarp_max(fmaxf(l0, l1));
    const float e0v = lane < E ? __expf(l0 - mx) : 0.f;
    const float e1v = lane + 32 < E ? __expf(l1 - mx) : 0.f;
    const float den = hwarp_sum(e0v + e1v);
    const float p0 = e0v / den, p1 = e1v / den;
    if (lane < E) probs[(size_t)t * E + lane] = p0;
    if (lane + 32 < E) probs[(size_t)t * E + lane + 32] = p1;
    __syncwarp();
    if (lane < E) slog[wid][lane] = p0;
    if (lane + 32 < E) slog[wid][lane + 32] = p1;
    __syncwarp();
    if (lane == 0) {
      float sel[8];
      int idx[8];
      float tot = 0.f;
      for (int j = 0; j < k; ++j) {
        float best = -1.f;
        int bi = 0;
        for (int e = 0; e < E; ++e) {
          const float v = slog[wid][e];
          if (v > best) { best = v; bi = e; }      // ties resolve to the lowest index
        }
        sel[j] = best;
        idx[j] = bi;
        tot += best;
        slog[wid][bi] = -2.f;
      }
      for (int j = 0; j < k; ++j) {
        topi[(size_t)t * k + j] = idx[j];
        gates[(size_t)t * k + j] = sel[j] / tot;
      }
    }
    __syncwarp();
  }
}

// ============================================================================ optimizer
template <bool BF16>
__global__ void __launch_bounds__(HT) adam_kernel(void* __restrict__ param, float* __restrict__ master, float* __restrict__ m,
                                                  float* __restrict__ v, const float* __restrict__ grad, long long n, float lr, float b1,
                                                  float b2, float eps, float wd, float bc1, float bc2, float gscale) {
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * HT + threadIdx.x; i < n4; i += (long long)gridDim.x * HT) {
    float4 g = reinterpret_cast<const float4*>(grad)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float4 w = reinterpret_cast<float4*>(master)[i];
    float* gp = &g.x; float* mp = &mm.x; float* vp = &vv.x; float* wp = &w.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gp[j] * gscale;
      mp[j] = b1 * mp[j] + (1.f - b1) * gj;
      vp[j] = b2 * vp[j] + (1.f - b2) * gj * gj;
      const float upd = (mp[j] / bc1) / (sqrtf(vp[j] / bc2) + eps);
      wp[j] = wp[j] * (1.f - lr * wd) - lr * upd;
    }
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    reinterpret_cast<float4*>(master)[i] = w;
    if (BF16) {
      uint2 o;
      o.x = pack_bf16x2(w.x, w.y);
      o.y = pack_bf16x2(w.z, w.w);
      reinterpret_cast<uint2*>(param)[i] = o;
    } else {
      reinterpret_cast<float4*>(param)[i] = w;
    }
  }
  // tail (n not a multiple of 4)
  for (long long i = (n4 << 2) + (long long)blockIdx.x * HT + threadIdx.x; i < n; i += (long long)gridDim.x * HT) {
    const float gj = grad[i] * gscale;
    const float mj = b1 * m[i] + (1.f - b1) * gj;
    const float vj = b2 * v[i] + (1.f - b2) * gj * gj;
    const float wj = master[i] * (1.f - lr * wd) - lr * (mj / bc1) / (sqrtf(vj / bc2) + eps);
    m[i] = mj; v[i] = vj; master[i] = wj;
    if (BF16) reinterpret_cast<__nv_bfloat16*>(param)[i] = __float2bfloat16(wj);
    else reinterpret_cast<float*>(param)[i] = wj;
  }
}

__global__ void __launch_bounds__(HT) sumsq_kernel(const float* __restrict__ x, float* __restrict__ out, long long n) {
  __shared__ float red[32];
  float s = 0.f;
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * HT + threadIdx.x; i < n4; i += (long long)gridDim.x * HT) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * HT + threadIdx.x; i < n; i += (long long)gridDim.x * HT) s += x[i] * x[i];
  s = hwarp_sum(s);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = s;
  __syncthreads();
  if (w == 0) {
    float r = l < (HT >> 5) ? red[l] : 0.f;
    r = hwarp_sum(r);
    if (l == 0) atomicAdd(out, r);
  }
}

// Reproducible form of the sum of squares: CTA b stores its sum in scratch[b]; the last CTA to finish (a counter
// behind the partial sums) adds them in index order to *out and resets the counter for the next call.
__global__ void __launch_bounds__(HT) sumsq_det_kernel(const float* __restrict__ x, float* __restrict__ out, long long n,
                                                       float* __restrict__ scratch, unsigned int* __restrict__ counter) {
  __shared__ float red[32];
  __shared__ unsigned int last;
  float s = 0.f;
  const long long n4 = n >> 2;
  for (long long i = (long long)blockIdx.x * HT + threadIdx.x; i < n4; i += (long long)gridDim.x * HT) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * HT + threadIdx.x; i < n; i += (long long)gridDim.x * HT) s += x[i] * x[i];
  s = hwarp_sum(s);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = s;
  __syncthreads();
  if (w == 0) {
    float r = l < (HT >> 5) ? red[l] : 0.f;
    r = hwarp_sum(r);
    if (l == 0) {
      scratch[blockIdx.x] = r;
      __threadfence();
      last = atomicAdd(counter, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    float tot = 0.f;
    for (unsigned int b = 0; b < gridDim.x; ++b) tot += reinterpret_cast<volatile float*>(scratch)[b];
    *out += tot;
    *counter = 0u;
  }
}

}  // namespace dh

using namespace dh;

#define DH_REQ(cond, msg)                  \
  do {                                     \
    if (!(cond)) {                         \
      set_last_error_c(__func__, msg);     \
      return (int)cudaErrorInvalidValue;   \
    }                                      \
  } while (0)

extern "C" {

int dh_embedding_fwd(const void* tok, const void* w, void* out, int T, int h, int Vl, int v0, int sm_budget, cudaStream_t s) {
  DH_REQ(h % 8 == 0, "hidden size must be a multiple of 8");
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<h_grid(T, 8, sm_budget), HT, 0, s>>>((const int*)tok, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, h, Vl, v0);
  return h_rc("dh_embedding_fwd");
}
int dh_embedding_bwd(const void* dout, const void* tok, void* grad, int T, int h, int Vl, int v0, int sm_budget, cudaStream_t s) {
  DH_REQ(h % 8 == 0, "hidden size must be a multiple of 8");
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<h_grid(T, 8, sm_budget), HT, 0, s>>>((const __nv_bfloat16*)dout, (const int*)tok, (float*)grad, T, h, Vl, v0);
  return h_rc("dh_embedding_bwd");
}
// Reproducible embedding gradient.  order: int64 [T], a stable sort of the positions by token id; sorted_tok: int32 [T].
int dh_embedding_bwd_sorted(const void* dout, const void* order, const void* sorted_tok, void* grad, int T, int h, int Vl, int v0,
                            int sm_budget, cudaStream_t s) {
  DH_REQ(h % 8 == 0, "hidden size must be a multiple of 8");
  if (T <= 0) return 0;
  embedding_bwd_sorted_kernel<<<h_grid(T, 8, sm_budget), HT, 0, s>>>((const __nv_bfloat16*)dout, (const long long*)order, (const int*)sorted_tok,
                                                                     (float*)grad, T, h, Vl, v0);
  return h_rc("dh_embedding_bwd_sorted");
}
int dh_ce_stats(const void* logits, const void* labels, void* stats, int T, int Vl, int64_t ld, int v0, int is_f32, int sm_budget,
                cudaStream_t s) {
  DH_REQ(is_f32 || ld % 8 == 0, "bf16 logits need a row stride that is a multiple of 8");
  if (T <= 0) return 0;
  if (is_f32) ce_stats_kernel<true><<<h_grid(T, 8, sm_budget), HT, 0, s>>>(logits, (const int*)labels, (float*)stats, T, Vl, ld, v0);
  else ce_stats_kernel<false><<<h_grid(T, 8, sm_budget), HT, 0, s>>>(logits, (const int*)labels, (float*)stats, T, Vl, ld, v0);
  return h_rc("dh_ce_stats");
}
int dh_ce_grad_inplace(void* logits, const void* labels, const void* lse, const void* gtok, int T, int Vl, int64_t ld, int v0, int is_f32,
                       float tcoef, float ucoef,
                       int sm_budget, cudaStream_t s) {
  DH_REQ(is_f32 || ld % 8 == 0, "bf16 logits need a row stride that is a multiple of 8");
  if (T <= 0) return 0;
  if (is_f32) ce_grad_kernel<true><<<h_grid(T, 8, sm_budget), HT, 0, s>>>(logits, (const int*)labels, (const float*)lse, (const float*)gtok, T, Vl, ld, v0, tcoef, ucoef);
  else ce_grad_kernel<false><<<h_grid(T, 8, sm_budget), HT, 0, s>>>(logits, (const int*)labels, (const float*)lse, (const float*)gtok, T, Vl, ld, v0, tcoef, ucoef);
  return h_rc("dh_ce_grad_inplace");
}
int dh_router_topk(const void* x, const void* w, void* probs, void* topi, void* gates, int T, int h, int E, int k, cudaStream_t s) {
  DH_REQ(h % 8 == 0 && E <= 64 && k <= 8 && k <= E, "router supports h % 8 == 0, E <= 64, k <= 8");
  if (T <= 0) return 0;
  router_kernel<<<h_grid((T + 7) / 8, 4, 0), HT, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)probs, (int*)topi,
                                                         (float*)gates, T, h, E, k);
  return h_rc("dh_router_topk");
}
int dh_adam_step(void* param, void* master, void* m, void* v, const void* grad, int64_t n, int param_bf16, float lr, float b1, float b2,
                 float eps, float wd, float bc1, float bc2, float gscale, cudaStream_t s) {
  DH_REQ((reinterpret_cast<uintptr_t>(master) & 15) == 0 && (reinterpret_cast<uintptr_t>(grad) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(m) & 15) == 0 && (reinterpret_cast<uintptr_t>(v) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(param) & 7) == 0,
         "optimizer ranges must be 16-byte aligned");
  if (n <= 0) return 0;
  const int grid = h_grid((n / 4 + HT - 1) / HT, 16, 0);
  if (param_bf16) adam_kernel<true><<<grid, HT, 0, s>>>(param, (float*)master, (float*)m, (float*)v, (const float*)grad, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  else adam_kernel<false><<<grid, HT, 0, s>>>(param, (float*)master, (float*)m, (float*)v, (const float*)grad, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  return h_rc("dh_adam_step");
}
int dh_sum_squares(const void* x, void* out, int64_t n, cudaStream_t s) {
  DH_REQ((reinterpret_cast<uintptr_t>(x) & 15) == 0, "input must be 16-byte aligned");
  if (n <= 0) return 0;
  sumsq_kernel<<<h_grid((n / 4 + HT - 1) / HT, 8, 0), HT, 0, s>>>((const float*)x, (float*)out, n);
  return h_rc("dh_sum_squares");
}
// Reproducible form.  scratch: fp32 [dh_sum_squares_scratch()] whose LAST element is a counter that must be zero
// before the first call (the kernel leaves it zero); calls that share a scratch must be ordered on one stream.
int dh_sum_squares_scratch() { return dh_sm_count() * 8 + 1; }
int dh_sum_squares_det(const void* x, void* out, int64_t n, void* scratch, cudaStream_t s) {
  DH_REQ((reinterpret_cast<uintptr_t>(x) & 15) == 0, "input must be 16-byte aligned");
  DH_REQ(scratch != nullptr, "scratch buffer missing");
  if (n <= 0) return 0;
  const int grid = h_grid((n / 4 + HT - 1) / HT, 8, 0);
  float* sc = (float*)scratch;
  sumsq_det_kernel<<<grid, HT, 0, s>>>((const float*)x, (float*)out, n, sc, reinterpret_cast<unsigned int*>(sc + dh_sm_count() * 8));
  return h_rc("dh_sum_squares_det");
}

}  // extern "C"
