"""SwiGLU and GeLU with explicit backward.

``swiglu_fwd/bwd`` take the fused FC1 output ``[.., 2f]`` whose first half is the gate
and second half the up projection (dhellam/operators/swiglu.py:13-26).  ``gelu_fwd`` is
the tanh form of the reference's native kernel (csrc/operators/gelu.cu:10-15); its
backward has no counterpart there and is added for the GPT family.
"""
from __future__ import annotations

from ctypes import c_int, c_int64, c_void_p

import torch

from .. import kernels as K

_K0 = 0.7978845608028654
_K1 = 0.044715


def swiglu_fwd(y, sm_budget: int = 0, stream=None):
    f = y.shape[-1] // 2
    if not K.use_native(y):
        g, u = y[..., :f].float(), y[..., f:].float()
        return (torch.nn.functional.silu(g) * u).to(y.dtype)
    out = torch.empty(y.shape[:-1] + (f,), dtype=y.dtype, device=y.device)
    fn = K.proto("dh_swiglu_fwd", [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    K.check(fn(y.data_ptr(), out.data_ptr(), y.numel() // (2 * f), f, sm_budget, K.stream_ptr(stream)), "dh_swiglu_fwd")
    return out


def swiglu_bwd(dout, y, sm_budget: int = 0, stream=None):
    f = y.shape[-1] // 2
    if not K.use_native(y):
        g, u, d = y[..., :f].float(), y[..., f:].float(), dout.float()
        s = torch.sigmoid(g)
        dg = d * u * s * (1 + g * (1 - s))
        du = d * g * s
        return torch.cat([dg, du], dim=-1).to(y.dtype)
    dy = torch.empty_like(y)
    fn = K.proto("dh_swiglu_bwd", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    K.check(fn(dout.data_ptr(), y.data_ptr(), dy.data_ptr(), y.numel() // (2 * f), f, sm_budget, K.stream_ptr(stream)),
            "dh_swiglu_bwd")
    return dy


def gelu_fwd(x, sm_budget: int = 0, stream=None):
    if not K.use_native(x):
        xf = x.float()
        return (0.5 * xf * (1 + torch.tanh(_K0 * (xf + _K1 * xf ** 3)))).to(x.dtype)
    out = torch.empty_like(x)
    fn = K.proto("dh_gelu_fwd", [c_void_p, c_void_p, c_int64, c_int, c_void_p])
    K.check(fn(x.data_ptr(), out.data_ptr(), x.numel(), sm_budget, K.stream_ptr(stream)), "dh_gelu_fwd")
    return out


def gelu_bwd(dout, x, sm_budget: int = 0, stream=None):
    if not K.use_native(x):
        xf, d = x.float(), dout.float()
        t = torch.tanh(_K0 * (xf + _K1 * xf ** 3))
        dt = (1 - t * t) * _K0 * (1 + 3 * _K1 * xf * xf)
        return (d * (0.5 * (1 + t) + 0.5 * xf * dt)).to(x.dtype)
    dx = torch.empty_like(x)
    fn = K.proto("dh_gelu_bwd", [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p])
    K.check(fn(dout.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), sm_budget, K.stream_ptr(stream)), "dh_gelu_bwd")
    return dx


# Name kept for users of the reference's native module (csrc/torchapi.cpp:4).
def pygelu(x, stream=None, profiling=False):
    return gelu_fwd(x, stream=stream)
