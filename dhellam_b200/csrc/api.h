// C-level launch API of the sm_100a kernel library.  Every function takes raw device
// pointers and a stream, launches asynchronously and returns a cudaError_t-style int
// (0 = success).  The torch binding in bindings.cpp is a thin shim over these.
//
// Capability parity with the reference's native module (csrc/torchapi.cpp:2-9,
// csrc/operators/ops.h:18-81): GEMM, GELU, bias-dropout-add, attention fwd/bwd, and an
// SM-budget argument on every persistent kernel in place of TPC masking
// (csrc/operators/smctrl.h:76-81).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- status ---------------------------------------------------------------
struct dh_status_t {
  int code, where, block, extra;
};
// Device address of this device's status word (allocated on first use).
void* dh_status_device_ptr();
// Copies the status word to the host (synchronises the device) and optionally clears it.
int dh_status_read(dh_status_t* out, int clear);
const char* dh_last_error_string();
int dh_sm_count();

// ---- GEMM (tcgen05 / TMEM / TMA) --------------------------------------------
// D[M,N] (row-major, leading dimension ldd) = opA[M,K] * opB[N,K]^T  (+ D when accumulate)
//   a_mn_major = 0: A is stored [M][K] (K contiguous, row stride lda elements)
//   a_mn_major = 1: A is stored [K][M] (M contiguous, row stride lda elements)
//   b_mn_major = 0: B is stored [N][K]; 1: B is stored [K][N]
//   d_fp32: output type is fp32 (else bf16); accumulate needs d_fp32.
//   epilogue: 0 none, 1 = SwiGLU over interleaved (gate, up) column pairs: D has N/2 columns
//   sm_budget: number of persistent CTAs (<=0: all SMs)
int dh_gemm_bf16(const void* a, int64_t lda, int a_mn_major, const void* b, int64_t ldb, int b_mn_major, void* d,
                 int64_t ldd, int d_fp32, int accumulate, int M, int N, int K, int epilogue, int sm_budget,
                 cudaStream_t stream);
// dK/dV kernel of dh_attn_bwd: 0 = one 128-query tile per iteration (default), 1 = pipelined transposed-score form
// (64 queries per iteration, double-buffered); -1 = take DHELLAM_ATTN_BWD_T from the environment at the next call.
void dh_attn_set_bwd_mode(int mode);
// Kernel choice for dh_gemm_bf16: 0 = per problem (default; also DHELLAM_GEMM_MODE), 1 = single-CTA tiles
// (128 x 256) only, 2 = CTA-pair tiles (256 x 256, tcgen05 cta_group::2) whenever M > 128.
void dh_gemm_set_mode(int mode);
// Split of an accumulating (fp32, add-in-place) GEMM along K into n atomic-add work items per tile:
// -1 = heuristic (fill the last wave), 0 / 1 = off, n = forced.
void dh_gemm_set_splitk(int n);
// dh_gemm_bf16 with the tensor-parallel collective hooks of the CTA-pair kernel (see gemm_sm100.cu).
int dh_gemm_bf16_sync(const void* a, int64_t lda, int a_mn_major, const void* b, int64_t ldb, int b_mn_major, void* d, int64_t ldd,
                      int d_fp32, int accumulate, int M, int N, int K, int sm_budget, const void* wait_count, unsigned wait_target,
                      void* const* sig_ptrs, int sig_bpr, int perm_mode, int world, int rank, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
