// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation.
//
// Who needs it.  The regular backward (dh_attn_bwd) takes a scratch buffer from its caller,
// and the Python layer gets that buffer from an allocator.  Some callers have no allocator
// they are allowed to use at the point of the call: a host application that reserved all
// device memory up front and forbids cudaMalloc from libraries it loads; a C or Fortran
// program that links this library without any tensor framework; a training process whose
// caching allocator already holds nearly all of the GPU's memory, so that a raw cudaMalloc
// from inside the library would fail.  For them the scratch lives inside the library image.
//
// What it does.  Same maths and same kernels as dh_attn_bwd (head size 128, bf16, strided
// [S, B, heads, d] operands, causal or full, grouped KV heads).  The scratch (one fp32 per
// query row and head: the dot product of dO and O that both backward kernels read) is a
// file-scope
//     static __device__ __align__(256) unsigned char[DH_ATTN_NOALLOC_SCRATCH_BYTES]
// in attention_sm100.cu.  Every GPU that loads the library holds those bytes until the
// process exits, which is why the limit is modest.
//
// Limits and rules.
//   * B * Hq * Sq rows need  rows*4 bytes (rounded up to 256); a call that needs more than
//     DH_ATTN_NOALLOC_SCRATCH_BYTES is rejected with cudaErrorInvalidValue and a message in
//     dh_last_error_string().  1 MiB covers 262144 rows, for example Sq = 4096, B = 8, Hq = 8.
//   * The first call on each device resolves the scratch's device address
//     (cudaGetSymbolAddress, with that device current) and opts the kernels into their
//     shared-memory size.  Make that first call before any stream capture begins.  The set-up
//     is done under a host mutex, so threads that make their first calls on one device at the
//     same time are safe; the calls themselves still share the scratch (next rule).
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine; the TMA
//     descriptors are built on the caller's stack.
//   * All calls on a device share the one array and it keeps the last call's contents.
//     Nothing in it has to start at zero: every call rewrites all the rows it reads.  Two calls whose
//     GPU work overlaps (different streams, no ordering between them) race on the array:
//     order them on one stream or with events.
//   * Timed-out device waits are not reported through the status word by this entry point
//     (the status word is allocated memory); the kernels still bound every wait.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define DH_ATTN_NOALLOC_SCRATCH_BYTES (1u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

// strides: 8 tensors x (sequence, batch, head) element strides, in the order
// dout, q, k, v, out, dq, dk, dv.  Returns 0 on success, else a cudaError_t value.
int dh_attn_bwd_noalloc(const void* dout, const void* q, const void* k, const void* v, const void* out, const void* lse, void* dq,
                        void* dk, void* dv, const int64_t* strides, int B, int Hq, int Hk, int Sq, int Sk, int d, int causal,
                        float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
