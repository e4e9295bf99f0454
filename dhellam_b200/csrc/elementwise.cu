// Memory-bound kernels of the transformer layer for sm_100a: RMSNorm / LayerNorm forward
// and backward (backward fuses the residual-gradient add and accumulates the affine
// gradients into fp32 main_grad), SwiGLU / GeLU forward and backward, bias-dropout-add
// with a recomputed keep-mask, and in-place rotary embedding on a packed QKV buffer.
//
// All kernels move 16 bytes per thread per access, keep a whole row in registers between
// the reduction and the normalisation (one DRAM read per element), and run as persistent
// grids sized by the caller's SM budget so that the dual-strand scheduler can co-run a
// kernel of the other strand on the remaining SMs.
//
// Roles in the reference: TransformerEngine tex.layernorm_fwd/bwd
// (dhellam/operators/layernorm.py:37-43, 82-89), torch.compile'd bda/swiglu
// (dhellam/operators/bda.py:3-12, dhellam/operators/swiglu.py:13-26), native gelu_cu and
// bda_cu (csrc/operators/gelu.cu:10-15, csrc/operators/bda.cu:10-16).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

namespace dh {

constexpr int NT = 256;          // threads per CTA in row kernels
constexpr int MAXV = 8;          // 16-byte vectors per thread  -> rows up to 256*8*8 = 16384 elements

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over the CTA; every thread gets the result.  `red` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) { red[w] = a; red[32 + w] = b; }
  __syncthreads();
  float ra = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  float rb = (l < (blockDim.x >> 5)) ? red[32 + l] : 0.f;
  a = warp_sum(ra);
  b = warp_sum(rb);
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]); u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

static inline int grid_for(long long work_items, int per_sm, int sm_budget) {
  int sms = dh_sm_count();
  int budget = (sm_budget <= 0 || sm_budget > sms) ? sms : sm_budget;
  long long g = (long long)budget * per_sm;
  if (work_items < g) g = work_items;
  return g < 1 ? 1 : (int)g;
}
static inline int launch_rc(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_last_error_c(what, cudaGetErrorString(e));
  return (int)e;
}

// ============================================================================ norms
// MODE 0: RMSNorm (mu unused), MODE 1: LayerNorm
template <int MODE, int VPT>
__global__ void __launch_bounds__(NT) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                      const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                      float* __restrict__ mu_out, float* __restrict__ rstd_out, int rows, int h,
                                                      float eps) {
  __shared__ float red[64];
  const int nvec = h >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    float v[VPT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        unpack8(ld_nc_v4(xr + c), v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) { s1 += v[i][j]; s2 += v[i][j] * v[i][j]; }
      }
    }
    block_sum2(s1, s2, red);
    float mu = 0.f, rstd;
    if (MODE == 1) {
      mu = s1 / h;
      rstd = rsqrtf(fmaxf(s2 / h - mu * mu, 0.f) + eps);
    } else {
      rstd = rsqrtf(s2 / h + eps);
    }
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (MODE == 1) mu_out[row] = mu;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * h);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float wv[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(w)[c], wv);
        if (MODE == 1 && b != nullptr) {
          float bv[8];
          unpack8(reinterpret_cast<const uint4*>(b)[c], bv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mu) * rstd * wv[j] + bv[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mu) * rstd * wv[j];
        }
        yr[c] = pack8(o);
      }
    }
  }
}

// 16-byte aligned fp32 x4 reduction into global memory (no return value).
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int MODE, int VPT>
__global__ void __launch_bounds__(NT) norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ mu_in,
                                                      const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ res,
                                                      __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, float* __restrict__ db,
                                                      int rows, int h, float* __restrict__ partial) {
  __shared__ float red[64];
  const int nvec = h >> 3;
  float accw[VPT][8], accb[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { accw[i][j] = 0.f; accb[i][j] = 0.f; }
  float wv[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * NT;
    if (c < nvec) unpack8(reinterpret_cast<const uint4*>(w)[c], wv[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * h);
    const float rstd = rstd_in[row];
    const float mu = MODE == 1 ? mu_in[row] : 0.f;
    float xh[VPT][8], g[VPT][8];
    float s1 = 0.f, s2 = 0.f;    // sum g, sum g*xhat
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float xv[8], dv[8];
        unpack8(ld_nc_v4(xr + c), xv);
        unpack8(ld_nc_v4(gr + c), dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mu) * rstd;
          g[i][j] = dv[j] * wv[i][j];
          accw[i][j] += dv[j] * xh[i][j];
          if (MODE == 1) accb[i][j] += dv[j];
          s1 += g[i][j];
          s2 += g[i][j] * xh[i][j];
        }
      }
    }
    block_sum2(s1, s2, red);
    const float m1 = MODE == 1 ? s1 / h : 0.f;
    const float m2 = s2 / h;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * h);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * h) : nullptr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - m1 - xh[i][j] * m2);
        if (rr) {
          float rv[8];
          unpack8(ld_nc_v4(rr + c), rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rv[j];
        }
        dxr[c] = pack8(o);
      }
    }
  }
  if (partial != nullptr) {
    // reproducible form: every CTA stores its partial sums (rows [0, grid) weight, rows [grid, 2 grid) bias);
    // norm_dw_finish_kernel adds them up in CTA order
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NT;
      if (c < nvec) {
        float4* pw = reinterpret_cast<float4*>(partial + (size_t)blockIdx.x * h + c * 8);
        pw[0] = make_float4(accw[i][0], accw[i][1], accw[i][2], accw[i][3]);
        pw[1] = make_float4(accw[i][4], accw[i][5], accw[i][6], accw[i][7]);
        if (MODE == 1 && db != nullptr) {
          float4* pb = reinterpret_cast<float4*>(partial + ((size_t)gridDim.x + blockIdx.x) * h + c * 8);
          pb[0] = make_float4(accb[i][0], accb[i][1], accb[i][2], accb[i][3]);
          pb[1] = make_float4(accb[i][4], accb[i][5], accb[i][6], accb[i][7]);
        }
      }
    }
    return;
  }
  // gradient buffers are views into one flat buffer: 16-byte alignment is usual, not guaranteed
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(dw) | (MODE == 1 && db != nullptr ? reinterpret_cast<uintptr_t>(db) : 0)) & 15) == 0;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * NT;
    if (c < nvec) {
      // every CTA adds its partial sums to the same h addresses: the 4-wide reduction
      // quarters the number of L2 atomic operations
      if (vec_ok) {
        red_add_v4(dw + c * 8, accw[i][0], accw[i][1], accw[i][2], accw[i][3]);
        red_add_v4(dw + c * 8 + 4, accw[i][4], accw[i][5], accw[i][6], accw[i][7]);
        if (MODE == 1 && db != nullptr) {
          red_add_v4(db + c * 8, accb[i][0], accb[i][1], accb[i][2], accb[i][3]);
          red_add_v4(db + c * 8 + 4, accb[i][4], accb[i][5], accb[i][6], accb[i][7]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          atomicAdd(dw + c * 8 + j, accw[i][j]);
          if (MODE == 1 && db != nullptr) atomicAdd(db + c * 8 + j, accb[i][j]);
        }
      }
    }
  }
}

// Adds `parts` partial rows of length h, in row order, to the gradient (same result for every run).
__global__ void __launch_bounds__(NT) norm_dw_finish_kernel(const float* __restrict__ partial, int parts, int h, float* __restrict__ dw,
                                                            float* __restrict__ db) {
  const int c = blockIdx.x * NT + threadIdx.x;
  if (c >= h) return;
  float a = 0.f, b = 0.f;
  for (int p = 0; p < parts; ++p) a += partial[(size_t)p * h + c];
  dw[c] += a;
  if (db != nullptr) {
    for (int p = 0; p < parts; ++p) b += partial[((size_t)parts + p) * h + c];
    db[c] += b;
  }
}

// ============================================================================ activations
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// `rows_dev` (nullable): the number of rows in use lives in device memory (ragged expert batches); rows is then the capacity.
__global__ void __launch_bounds__(NT) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ out,
                                                        long long rows, int f, const int* __restrict__ rows_dev) {
  const int fv = f >> 3;
  if (rows_dev != nullptr) rows = min(rows, (long long)*rows_dev);
  const long long total = rows * fv;
  for (long long i = (long long)blockIdx.x * NT + threadIdx.x; i < total; i += (long long)gridDim.x * NT) {
    const long long r = i / fv;
    const int c = (int)(i - r * fv);
    const uint4* row = reinterpret_cast<const uint4*>(y + r * 2 * (long long)f);
    float g[8], u[8], o[8];
    unpack8(ld_nc_v4(row + c), g);
    unpack8(ld_nc_v4(row + fv + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j];
    reinterpret_cast<uint4*>(out + r * (long long)f)[c] = pack8(o);
  }
}

__global__ void __launch_bounds__(NT) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                                        __nv_bfloat16* __restrict__ dy, long long rows, int f,
                                                        const int* __restrict__ rows_dev) {
  const int fv = f >> 3;
  if (rows_dev != nullptr) rows = min(rows, (long long)*rows_dev);
  const long long total = rows * fv;
  for (long long i = (long long)blockIdx.x * NT + threadIdx.x; i < total; i += (long long)gridDim.x * NT) {
    const long long r = i / fv;
    const int c = (int)(i - r * fv);
    const uint4* row = reinterpret_cast<const uint4*>(y + r * 2 * (long long)f);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld_nc_v4(row + c), g);
    unpack8(ld_nc_v4(row + fv + c), u);
    unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(dout + r * (long long)f) + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_(g[j]);
      dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    uint4* orow = reinterpret_cast<uint4*>(dy + r * 2 * (long long)f);
    orow[c] = pack8(dg);
    orow[fv + c] = pack8(du);
  }
}

__global__ void __launch_bounds__(NT) gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = (long long)blockIdx.x * NT + threadIdx.x; i < nvec; i += (long long)gridDim.x * NT) {
    float v[8], o[8];
    unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(x) + i), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = tanhf(0.7978845608028654f * (v[j] + 0.044715f * v[j] * v[j] * v[j]));
      o[j] = 0.5f * v[j] * (1.f + t);
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(o);
  }
}

__global__ void __launch_bounds__(NT) gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ x,
                                                      __nv_bfloat16* __restrict__ dx, long long nvec) {
  for (long long i = (long long)blockIdx.x * NT + threadIdx.x; i < nvec; i += (long long)gridDim.x * NT) {
    float v[8], d[8], o[8];
    unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(x) + i), v);
    unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(dout) + i), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x2 = v[j] * v[j];
      const float t = tanhf(0.7978845608028654f * (v[j] + 0.044715f * v[j] * x2));
      const float dt = (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
      o[j] = d[j] * (0.5f * (1.f + t) + 0.5f * v[j] * dt);
    }
    reinterpret_cast<uint4*>(dx)[i] = pack8(o);
  }
}

// ============================================================================ bias-dropout-add
// Counter-based keep decision for element `idx` under `seed` (same integer hash as the
// Python model in ops/bda.py).
__device__ __forceinline__ bool keep_element(unsigned long long idx, unsigned long long seed, float p) {
  uint32_t x = (uint32_t)idx ^ (uint32_t)seed;
  x += (uint32_t)(idx >> 32) * 0x9E3779B1u + (uint32_t)(seed >> 32);
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  const float u = (float)(x >> 8) * (1.0f / 16777216.0f);
  return u >= p;
}

__global__ void __launch_bounds__(NT) bda_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                                                     const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ out,
                                                     long long nvec, int hvec, float p, unsigned long long seed) {
  const float scale = p > 0.f ? 1.f / (1.f - p) : 1.f;
  for (long long i = (long long)blockIdx.x * NT + threadIdx.x; i < nvec; i += (long long)gridDim.x * NT) {
    float v[8], r[8], o[8];
    unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(x) + i), v);
    unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(res) + i), r);
    if (bias != nullptr) {
      float bv[8];
      unpack8(reinterpret_cast<const uint4*>(bias)[i % hvec], bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += bv[j];
    }
    if (p > 0.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = keep_element((unsigned long long)i * 8 + j, seed, p) ? v[j] * scale : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = v[j] + r[j];
    reinterpret_cast<uint4*>(out)[i] = pack8(o);
  }
}

__global__ void __launch_bounds__(NT) bda_bwd_kernel(const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dx, long long nvec,
                                                     float p, unsigned long long seed) {
  const float scale = 1.f / (1.f - p);
  for (long long i = (long long)blockIdx.x * NT + threadIdx.x; i < nvec; i += (long long)gridDim.x * NT) {
    float v[8];
    unpack8(ld_nc_v4(reinterpret_cast<const uint4*>(dout) + i), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = keep_element((unsigned long long)i * 8 + j, seed, p) ? v[j] * scale : 0.f;
    reinterpret_cast<uint4*>(dx)[i] = pack8(v);
  }
}

// ============================================================================ RoPE
// One thread rotates 8 pairs (i, i + d/2) of one head of one row.
__global__ void __launch_bounds__(NT) rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos, const float* __restrict__ cosT,
                                                  const float* __restrict__ sinT, int rows, long long row_stride, int heads, int d,
                                                  int inverse) {
  const int hv = d >> 4;                   // vectors per half head
  const long long per_row = (long long)heads * hv;
  const long long total = (long long)rows * per_row;
  for (long long i = (long long)blockIdx.x * NT + threadIdx.x; i < total; i += (long long)gridDim.x * NT) {
    const long long r = i / per_row;
    const int rem = (int)(i - r * per_row);
    const int hd = rem / hv, c = rem - hd * hv;
    __nv_bfloat16* base = qkv + r * row_stride + (long long)hd * d;
    uint4* p1 = reinterpret_cast<uint4*>(base) + c;
    uint4* p2 = reinterpret_cast<uint4*>(base + (d >> 1)) + c;
    float a[8], b[8], o1[8], o2[8];
    unpack8(*p1, a);
    unpack8(*p2, b);
    const float* cr = cosT + (long long)pos[r] * (d >> 1) + c * 8;
    const float* sr = sinT + (long long)pos[r] * (d >> 1) + c * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cs = cr[j];
      const float sn = inverse ? -sr[j] : sr[j];
      o1[j] = a[j] * cs - b[j] * sn;
      o2[j] = b[j] * cs + a[j] * sn;
    }
    *p1 = pack8(o1);
    *p2 = pack8(o2);
  }
}

}  // namespace dh

// ============================================================================ C API
using namespace dh;

#define DH_REQUIRE(cond, msg)                      \
  do {                                             \
    if (!(cond)) {                                 \
      set_last_error_c(__func__, msg);             \
      return (int)cudaErrorInvalidValue;           \
    }                                              \
  } while (0)

// picks the number of 16-byte vectors per thread from the row length
#define DH_VPT_DISPATCH(h, KERNEL, MODE, GRID, ...)                                   \
  do {                                                                                \
    const int vpt_ = ((h) / 8 + NT - 1) / NT;                                         \
    if (vpt_ <= 1) KERNEL<MODE, 1><<<GRID, NT, 0, s>>>(__VA_ARGS__);                  \
    else if (vpt_ <= 2) KERNEL<MODE, 2><<<GRID, NT, 0, s>>>(__VA_ARGS__);             \
    else if (vpt_ <= 4) KERNEL<MODE, 4><<<GRID, NT, 0, s>>>(__VA_ARGS__);             \
    else KERNEL<MODE, 8><<<GRID, NT, 0, s>>>(__VA_ARGS__);                            \
  } while (0)

extern "C" {

int dh_rmsnorm_fwd(const void* x, const void* w, void* y, void* rstd, int rows, int h, float eps, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(h % 8 == 0 && h <= NT * MAXV * 8, "hidden size must be a multiple of 8 and at most 16384");
  if (rows <= 0) return 0;
  DH_VPT_DISPATCH(h, norm_fwd_kernel, 0, grid_for(rows, 8, sm_budget), (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, nullptr,
                  (__nv_bfloat16*)y, nullptr, (float*)rstd, rows, h, eps);
  return launch_rc("dh_rmsnorm_fwd");
}
int dh_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* res, void* dx, void* dw, int rows, int h,
                   int sm_budget, cudaStream_t s) {
  DH_REQUIRE(h % 8 == 0 && h <= NT * MAXV * 8, "hidden size must be a multiple of 8 and at most 16384");
  if (rows <= 0) return 0;
  DH_VPT_DISPATCH(h, norm_bwd_kernel, 0, grid_for(rows, 2, sm_budget), (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                  (const __nv_bfloat16*)w, nullptr, (const float*)rstd, (const __nv_bfloat16*)res, (__nv_bfloat16*)dx, (float*)dw, nullptr,
                  rows, h, nullptr);
  return launch_rc("dh_rmsnorm_bwd");
}
// Number of CTAs the norm backward launches = rows of fp32 partial sums (x h, x 2 with a bias) its reproducible form needs.
int dh_norm_bwd_grid(int rows, int sm_budget) { return grid_for(rows, 2, sm_budget); }
// Reproducible forms: the weight (and bias) gradient is summed over CTAs in a fixed order through `partial`
// (fp32 [grid, h], [2 grid, h] for layer norm) instead of order-dependent reductions into memory.
int dh_rmsnorm_bwd_det(const void* dy, const void* x, const void* w, const void* rstd, const void* res, void* dx, void* dw, void* partial,
                       int rows, int h, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(h % 8 == 0 && h <= NT * MAXV * 8, "hidden size must be a multiple of 8 and at most 16384");
  DH_REQUIRE(partial != nullptr && (reinterpret_cast<uintptr_t>(partial) & 15) == 0, "partial sums need a 16-byte aligned buffer");
  if (rows <= 0) return 0;
  const int grid = grid_for(rows, 2, sm_budget);
  DH_VPT_DISPATCH(h, norm_bwd_kernel, 0, grid, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, nullptr,
                  (const float*)rstd, (const __nv_bfloat16*)res, (__nv_bfloat16*)dx, (float*)dw, nullptr, rows, h, (float*)partial);
  norm_dw_finish_kernel<<<(h + NT - 1) / NT, NT, 0, s>>>((const float*)partial, grid, h, (float*)dw, nullptr);
  return launch_rc("dh_rmsnorm_bwd_det");
}
int dh_layernorm_bwd_det(const void* dy, const void* x, const void* w, const void* mu, const void* rstd, const void* res, void* dx, void* dw,
                         void* db, void* partial, int rows, int h, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(h % 8 == 0 && h <= NT * MAXV * 8, "hidden size must be a multiple of 8 and at most 16384");
  DH_REQUIRE(partial != nullptr && (reinterpret_cast<uintptr_t>(partial) & 15) == 0, "partial sums need a 16-byte aligned buffer");
  if (rows <= 0) return 0;
  const int grid = grid_for(rows, 2, sm_budget);
  DH_VPT_DISPATCH(h, norm_bwd_kernel, 1, grid, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const float*)mu,
                  (const float*)rstd, (const __nv_bfloat16*)res, (__nv_bfloat16*)dx, (float*)dw, (float*)db, rows, h, (float*)partial);
  norm_dw_finish_kernel<<<(h + NT - 1) / NT, NT, 0, s>>>((const float*)partial, grid, h, (float*)dw, (float*)db);
  return launch_rc("dh_layernorm_bwd_det");
}
int dh_layernorm_fwd(const void* x, const void* w, const void* b, void* y, void* mu, void* rstd, int rows, int h, float eps, int sm_budget,
                     cudaStream_t s) {
  DH_REQUIRE(h % 8 == 0 && h <= NT * MAXV * 8, "hidden size must be a multiple of 8 and at most 16384");
  if (rows <= 0) return 0;
  DH_VPT_DISPATCH(h, norm_fwd_kernel, 1, grid_for(rows, 8, sm_budget), (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                  (const __nv_bfloat16*)b, (__nv_bfloat16*)y, (float*)mu, (float*)rstd, rows, h, eps);
  return launch_rc("dh_layernorm_fwd");
}
int dh_layernorm_bwd(const void* dy, const void* x, const void* w, const void* mu, const void* rstd, const void* res, void* dx, void* dw,
                     void* db, int rows, int h, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(h % 8 == 0 && h <= NT * MAXV * 8, "hidden size must be a multiple of 8 and at most 16384");
  if (rows <= 0) return 0;
  DH_VPT_DISPATCH(h, norm_bwd_kernel, 1, grid_for(rows, 2, sm_budget), (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                  (const __nv_bfloat16*)w, (const float*)mu, (const float*)rstd, (const __nv_bfloat16*)res, (__nv_bfloat16*)dx, (float*)dw,
                  (float*)db, rows, h, nullptr);
  return launch_rc("dh_layernorm_bwd");
}
int dh_swiglu_fwd(const void* y, void* out, int64_t rows, int f, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(f % 8 == 0, "ffn width must be a multiple of 8");
  if (rows <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for((rows * (f / 8) + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)y, (__nv_bfloat16*)out, rows, f, nullptr);
  return launch_rc("dh_swiglu_fwd");
}
// Ragged form: `rows` is the capacity, the number of rows in use is read from device memory (*rows_dev).
int dh_swiglu_fwd_n(const void* y, void* out, int64_t rows, const void* rows_dev, int f, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(f % 8 == 0, "ffn width must be a multiple of 8");
  if (rows <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for((rows * (f / 8) + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)y, (__nv_bfloat16*)out, rows, f,
                                                                                         (const int*)rows_dev);
  return launch_rc("dh_swiglu_fwd_n");
}
int dh_swiglu_bwd_n(const void* dout, const void* y, void* dy, int64_t rows, const void* rows_dev, int f, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(f % 8 == 0, "ffn width must be a multiple of 8");
  if (rows <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for((rows * (f / 8) + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y,
                                                                                         (__nv_bfloat16*)dy, rows, f, (const int*)rows_dev);
  return launch_rc("dh_swiglu_bwd_n");
}
int dh_swiglu_bwd(const void* dout, const void* y, void* dy, int64_t rows, int f, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(f % 8 == 0, "ffn width must be a multiple of 8");
  if (rows <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for((rows * (f / 8) + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y,
                                                                                         (__nv_bfloat16*)dy, rows, f, nullptr);
  return launch_rc("dh_swiglu_bwd");
}
int dh_gelu_fwd(const void* x, void* out, int64_t n, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(n % 8 == 0, "element count must be a multiple of 8");
  if (n <= 0) return 0;
  gelu_fwd_kernel<<<grid_for((n / 8 + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n / 8);
  return launch_rc("dh_gelu_fwd");
}
int dh_gelu_bwd(const void* dout, const void* x, void* dx, int64_t n, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(n % 8 == 0, "element count must be a multiple of 8");
  if (n <= 0) return 0;
  gelu_bwd_kernel<<<grid_for((n / 8 + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)x,
                                                                              (__nv_bfloat16*)dx, n / 8);
  return launch_rc("dh_gelu_bwd");
}
int dh_bda_fwd(const void* x, const void* bias, const void* res, void* out, int64_t n, int h, float p, uint64_t seed, int sm_budget,
               cudaStream_t s) {
  DH_REQUIRE(n % 8 == 0 && h % 8 == 0, "sizes must be multiples of 8");
  if (n <= 0) return 0;
  bda_fwd_kernel<<<grid_for((n / 8 + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)bias,
                                                                             (const __nv_bfloat16*)res, (__nv_bfloat16*)out, n / 8, h / 8, p,
                                                                             seed);
  return launch_rc("dh_bda_fwd");
}
int dh_bda_bwd(const void* dout, void* dx, int64_t n, float p, uint64_t seed, int sm_budget, cudaStream_t s) {
  DH_REQUIRE(n % 8 == 0, "element count must be a multiple of 8");
  if (n <= 0) return 0;
  bda_bwd_kernel<<<grid_for((n / 8 + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((const __nv_bfloat16*)dout, (__nv_bfloat16*)dx, n / 8, p, seed);
  return launch_rc("dh_bda_bwd");
}
int dh_rope_inplace(void* qkv, const void* pos, const void* cosT, const void* sinT, int rows, int row_stride, int heads, int d, int inverse,
                    int sm_budget, cudaStream_t s) {
  DH_REQUIRE(d % 16 == 0 && row_stride % 8 == 0, "head size must be a multiple of 16 and the row stride of 8");
  if (rows <= 0) return 0;
  const long long total = (long long)rows * heads * (d / 16);
  rope_kernel<<<grid_for((total + NT - 1) / NT, 8, sm_budget), NT, 0, s>>>((__nv_bfloat16*)qkv, (const int*)pos, (const float*)cosT,
                                                                          (const float*)sinT, rows, row_stride, heads, d, inverse);
  return launch_rc("dh_rope_inplace");
}

}  // extern "C"
