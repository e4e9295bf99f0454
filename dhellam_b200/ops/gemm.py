"""Linear-layer products on the tcgen05 GEMM.

* ``gemm_nt(x, w)``          Y  = X Wᵀ        forward          (``gemm_fwd`` in the reference,
  dhellam/operators/layernorm_column.py:7-62)
* ``gemm_nn(dy, w)``         dX = dY W        data gradient    (``dgrad_bwd``, :209-263)
* ``gemm_tn_acc(dy, x, g)``  G += dYᵀ X       weight gradient accumulated into an fp32
  ``main_grad`` buffer (``wgrad_bwd``, :265-323)

On CUDA tensors the products run on the hand-written sm_100a kernel; on CPU tensors the
same functions run an fp32 PyTorch reference so that the engine is testable without a GPU.
Every function takes ``sm_budget`` (number of persistent CTAs) which is the co-execution
knob the dual-strand scheduler uses in place of the reference's TPC masks
(csrc/operators/smctrl.h:76-81).
"""
from __future__ import annotations

from ctypes import c_int, c_int64, c_uint, c_void_p

import ctypes

import torch

from .. import kernels as K

_GEMM_ARGS = [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
              c_int, c_int, c_void_p]
_GEMM_SYNC_ARGS = [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                   c_int, c_void_p, c_uint, c_void_p, c_int, c_int, c_int, c_int, c_void_p]


class GemmSync:
    """Collective hooks of the CTA-pair GEMM (``dh_gemm_bf16_sync``), built by ``ops.fused_comm.FusedTP``.

    ``wait_count`` / ``wait_target``: the A operand is an all-gather staging buffer; the kernel
    waits per 128-row block for that block's arrival counter.  ``sig_ptrs`` / ``sig_bpr``: the
    output is this rank's partial product of a reduce-scatter; after every stored row block the
    kernel bumps the block's counter on the owning rank.  ``perm_mode``: row visiting order
    (1 = own shard first then the others block by block, 2 = block by block over all owners)."""

    def __init__(self, wait_count: int = 0, wait_target: int = 0, sig_ptrs=None, sig_bpr: int = 0, perm_mode: int = 0,
                 world: int = 1, rank: int = 0):
        self.wait_count, self.wait_target = wait_count, wait_target
        self.sig_ptrs, self.sig_bpr = sig_ptrs, sig_bpr
        self.perm_mode, self.world, self.rank = perm_mode, world, rank
        self.start_id = 0          # set by the launch: id under which the kernel announces "all CTAs resident"


def _native(*ts) -> bool:
    return all(K.use_native(t) for t in ts)


def _library(*ts) -> bool:
    return all(K.use_library(t) for t in ts)


def _check2d(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D tensor with unit inner stride, got shape {tuple(t.shape)} strides {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16, got {t.dtype}")


def _launch(a, a_mn, b, b_mn, d, accumulate, M, N, Kdim, sm_budget, stream, sync: "GemmSync | None" = None):
    if sync is not None:
        fn = K.proto("dh_gemm_bf16_sync", _GEMM_SYNC_ARGS)
        rc = fn(a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn), d.data_ptr(), d.stride(0),
                int(d.dtype == torch.float32), int(accumulate), M, N, Kdim, int(sm_budget), sync.wait_count or None,
                int(sync.wait_target), sync.sig_ptrs, int(sync.sig_bpr), int(sync.perm_mode), int(sync.world), int(sync.rank),
                K.stream_ptr(stream))
        K.check(rc, "dh_gemm_bf16_sync")
        if sync.sig_ptrs is not None:
            sync.start_id = K.proto("dh_gemm_last_start_id", [], ctypes.c_uint)()
        return
    fn = K.proto("dh_gemm_bf16", _GEMM_ARGS)
    rc = fn(a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn), d.data_ptr(), d.stride(0),
            int(d.dtype == torch.float32), int(accumulate), M, N, Kdim, 0, int(sm_budget), K.stream_ptr(stream))
    K.check(rc, "dh_gemm_bf16")


def set_gemm_mode(mode: int):
    """Kernel choice on the GPU: 0 per problem (default), 1 single-CTA 128x256 tiles only,
    2 CTA-pair 256x256 tiles (``tcgen05`` ``cta_group::2``) whenever M > 128."""
    K.proto("dh_gemm_set_mode", [c_int], None)(int(mode))


def set_gemm_splitk(n: int):
    """K split of accumulating GEMMs (weight gradients): -1 heuristic (default), 0/1 off, n forced."""
    K.proto("dh_gemm_set_splitk", [c_int], None)(int(n))


def gemm_nt(x, w, out=None, sm_budget: int = 0, stream=None, out_dtype=None, sync: "GemmSync | None" = None):
    """``x [M,K] @ w[N,K]ᵀ -> [M,N]``.  ``sync`` adds the collective hooks (GPU only)."""
    M, Kd = x.shape
    N = w.shape[0]
    assert w.shape[1] == Kd, (x.shape, w.shape)
    if _library(x, w):
        from . import library as LIB
        return LIB.gemm_nt(x, w, out, out_dtype)
    if not _native(x, w):
        y = (x.float() @ w.float().t()).to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check2d(x, "x"), _check2d(w, "w")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
    _launch(x, False, w, False, out, False, M, N, Kd, sm_budget, stream, sync)
    return out


def gemm_nn(dy, w, out=None, sm_budget: int = 0, stream=None, sync: "GemmSync | None" = None):
    """``dy [M,N] @ w[N,K] -> [M,K]``.  ``sync`` adds the collective hooks (GPU only)."""
    M, N = dy.shape
    Kd = w.shape[1]
    assert w.shape[0] == N, (dy.shape, w.shape)
    if _library(dy, w):
        from . import library as LIB
        return LIB.gemm_nn(dy, w, out)
    if not _native(dy, w):
        y = (dy.float() @ w.float()).to(dy.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check2d(dy, "dy"), _check2d(w, "w")
    if out is None:
        out = torch.empty((M, Kd), dtype=torch.bfloat16, device=dy.device)
    # contraction over N: A = dy (K-major in the kernel's terms), B = w stored [N][K] = MN-major
    _launch(dy, False, w, True, out, False, M, Kd, N, sm_budget, stream, sync)
    return out


def gemm_tn_acc(dy, x, main_grad, accumulate: bool = True, sm_budget: int = 0, stream=None):
    """``main_grad [N,K] (+)= dy[M,N]ᵀ @ x[M,K]`` with fp32 accumulation in place."""
    M, N = dy.shape
    Kd = x.shape[1]
    assert x.shape[0] == M and tuple(main_grad.shape) == (N, Kd), (dy.shape, x.shape, main_grad.shape)
    if _library(dy, x, main_grad):
        from . import library as LIB
        return LIB.gemm_tn_acc(dy, x, main_grad, accumulate)
    if not _native(dy, x, main_grad):
        g = dy.float().t() @ x.float()
        if accumulate:
            main_grad.add_(g.to(main_grad.dtype))
        else:
            main_grad.copy_(g)
        return main_grad
    _check2d(dy, "dy"), _check2d(x, "x")
    if main_grad.dtype != torch.float32 or main_grad.stride(1) != 1:
        raise ValueError("main_grad must be fp32 with unit inner stride")
    # contraction over M: A = dyᵀ stored [M][N] (MN-major), B = xᵀ stored [M][K] (MN-major)
    _launch(dy, True, x, True, main_grad, accumulate, N, Kd, M, sm_budget, stream)
    return main_grad


# ----------------------------------------------------------------------------- reference-style wrappers
def _timed(fn, profiling, stream):
    """Runs ``fn`` on ``stream``; returns ``(result, elapsed ms or 0)`` timed with CUDA events
    on that stream (the reference wraps its calls in host timers, layernorm_column.py:28-35)."""
    if not torch.cuda.is_available():
        return fn(), 0.0
    stream = stream if stream is not None else torch.cuda.current_stream()
    with torch.cuda.stream(stream):
        if not profiling:
            return fn(), 0.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        out = fn()
        e1.record(stream)
        e1.synchronize()
        return out, e0.elapsed_time(e1)


def gemm_fwd(args, input, weight, output=None, layout: str = "TN", profiling: bool = False, math_sm_count: int = 0,
             is_matmul: bool = False, stream=None):
    """``output = input @ weightᵀ`` for a ``[N, K]`` weight (layout "TN"), or ``input @ weight``
    for layout "NN".  Signature of the reference's ``gemm_fwd`` (layernorm_column.py:7-62);
    ``math_sm_count`` becomes the CTA budget, ``is_matmul`` is ignored (one kernel serves both)."""
    x2 = input.reshape(-1, input.shape[-1])
    fn = (lambda: gemm_nt(x2, weight, out=output, sm_budget=abs(math_sm_count))) if layout[0] == "T" else \
         (lambda: gemm_nn(x2, weight, out=output, sm_budget=abs(math_sm_count)))
    out, ms = _timed(fn, profiling, stream)
    return out.view(*input.shape[:-1], out.shape[-1]), ms


gemm_fwd_event = gemm_fwd


def dgrad_bwd(args, input_grad, weight, dgrad_output=None, layout: str = "NN", profiling: bool = False, math_sm_count: int = 0,
              is_matmul: bool = False, stream=None):
    """``dgrad = input_grad @ weight`` (layernorm_column.py:209-263)."""
    g2 = input_grad.reshape(-1, input_grad.shape[-1])
    out, ms = _timed(lambda: gemm_nn(g2, weight, out=dgrad_output, sm_budget=abs(math_sm_count)), profiling, stream)
    return out, ms


def wgrad_bwd(args, input_grad, input_data, wgrad_output, grad_accumulate: bool = False, layout: str = "NT", profiling: bool = False,
              math_sm_count: int = 0, is_matmul: bool = False, stream=None):
    """``wgrad (+)= input_gradᵀ @ input_data`` into ``wgrad_output`` (fp32 ``main_grad`` in
    training; layernorm_column.py:265-323)."""
    g2 = input_grad.reshape(-1, input_grad.shape[-1])
    x2 = input_data.reshape(-1, input_data.shape[-1])

    def run():
        if wgrad_output.dtype == torch.float32:
            return gemm_tn_acc(g2, x2, wgrad_output, accumulate=grad_accumulate, sm_budget=abs(math_sm_count))
        tmp = torch.zeros(wgrad_output.shape, dtype=torch.float32, device=wgrad_output.device)
        gemm_tn_acc(g2, x2, tmp, accumulate=False, sm_budget=abs(math_sm_count))
        if grad_accumulate:
            wgrad_output.add_(tmp.to(wgrad_output.dtype))
        else:
            wgrad_output.copy_(tmp)
        return wgrad_output
    return _timed(run, profiling, stream)


def gemm_bwd(args, input_grad, weight, input_data, dgrad_output, wgrad_output, grad_accumulate: bool = False, layout: str = "NNNT",
             profiling: bool = False, math_sm_count: int = 0, is_matmul: bool = False):
    """dgrad + wgrad pair (layernorm_column.py:121-207).  Returns
    ``(dgrad, wgrad, dgrad ms, wgrad ms)``."""
    d, t1 = dgrad_bwd(args, input_grad, weight, dgrad_output, layout[:2], profiling, math_sm_count)
    w, t2 = wgrad_bwd(args, input_grad, input_data, wgrad_output, grad_accumulate, layout[2:], profiling, math_sm_count)
    return d, w, t1, t2


def pygemm(a, b, d, transa: bool = False, transb: bool = False, grad_accumulate: bool = False, math_sm_count: int = 0, stream=None,
           profiling: bool = False):
    """General entry of the native GEMM (``pygemm``, csrc/operators/gemm.cu:144-170):
    ``d (+)= op(a) @ op(b)`` with row-major operands; ``trans*`` mean "use the transpose"."""
    M = a.shape[1] if transa else a.shape[0]
    Kd = a.shape[0] if transa else a.shape[1]
    N = b.shape[0] if transb else b.shape[1]
    if not _native(a, b, d):
        r = (a.float().t() if transa else a.float()) @ (b.float().t() if transb else b.float())
        d.copy_(d.float() + r if grad_accumulate else r)
        return 0.0

    def run():
        # kernel form: D = opA[M,K] * opB[N,K]^T ; A stored [K][M] when transa; B stored [K][N] when not transb
        _launch(a, transa, b, not transb, d, grad_accumulate, M, N, Kd, abs(math_sm_count), stream)
    _, ms = _timed(run, profiling, stream)
    return ms
