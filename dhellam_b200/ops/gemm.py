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

from ctypes import c_int, c_int64, c_void_p

import torch

from .. import kernels as K

_GEMM_ARGS = [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
              c_int, c_int, c_void_p]


def _native(*ts) -> bool:
    return all(t.is_cuda for t in ts)


def _check2d(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D tensor with unit inner stride, got shape {tuple(t.shape)} strides {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16, got {t.dtype}")


def _launch(a, a_mn, b, b_mn, d, accumulate, M, N, Kdim, sm_budget, stream):
    fn = K.proto("dh_gemm_bf16", _GEMM_ARGS)
    rc = fn(a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn), d.data_ptr(), d.stride(0),
            int(d.dtype == torch.float32), int(accumulate), M, N, Kdim, 0, int(sm_budget), K.stream_ptr(stream))
    K.check(rc, "dh_gemm_bf16")


def gemm_nt(x, w, out=None, sm_budget: int = 0, stream=None, out_dtype=None):
    """``x [M,K] @ w[N,K]ᵀ -> [M,N]``."""
    M, Kd = x.shape
    N = w.shape[0]
    assert w.shape[1] == Kd, (x.shape, w.shape)
    if not _native(x, w):
        y = (x.float() @ w.float().t()).to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check2d(x, "x"), _check2d(w, "w")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
    _launch(x, False, w, False, out, False, M, N, Kd, sm_budget, stream)
    return out


def gemm_nn(dy, w, out=None, sm_budget: int = 0, stream=None):
    """``dy [M,N] @ w[N,K] -> [M,K]``."""
    M, N = dy.shape
    Kd = w.shape[1]
    assert w.shape[0] == N, (dy.shape, w.shape)
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
    _launch(dy, False, w, True, out, False, M, Kd, N, sm_budget, stream)
    return out


def gemm_tn_acc(dy, x, main_grad, accumulate: bool = True, sm_budget: int = 0, stream=None):
    """``main_grad [N,K] (+)= dy[M,N]ᵀ @ x[M,K]`` with fp32 accumulation in place."""
    M, N = dy.shape
    Kd = x.shape[1]
    assert x.shape[0] == M and tuple(main_grad.shape) == (N, Kd), (dy.shape, x.shape, main_grad.shape)
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
