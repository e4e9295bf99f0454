"""Bias + dropout + residual add, forward and backward.

Same role as the reference's ``bda_fwd_`` / ``bda_bwd_`` (dhellam/operators/bda.py:3-12) and
its native ``bda_cu`` (csrc/operators/bda.cu:10-16), with two differences: the keep-mask is
recomputed from ``(seed, element index)`` by a counter-based hash instead of being stored
as an int8 tensor, and kept values are scaled by ``1/(1-p)`` (the reference hard-codes
0.9 for p = 0.1).
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_uint64, c_void_p

import torch

from .. import kernels as K

_M32 = 0xFFFFFFFF


def keep_mask_reference(numel: int, seed: int, p: float, device="cpu"):
    """Bit-exact CPU model of the device hash: element i is kept iff u(seed, i) >= p."""
    i = torch.arange(numel, dtype=torch.int64, device=device)
    x = (i ^ (seed & _M32)) & _M32
    x = (x + ((i >> 32) * 0x9E3779B1 & _M32) + ((seed >> 32) & _M32)) & _M32
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & _M32
    x = x ^ (x >> 16)
    u = (x >> 8).to(torch.float32) * (1.0 / 16777216.0)
    return u >= p


def bda_fwd(x, residual, bias=None, p: float = 0.0, seed: int = 0, training: bool = True, sm_budget: int = 0, stream=None):
    """``out = residual + dropout(x + bias)``."""
    p_eff = p if training else 0.0
    if not K.use_native(x):
        v = x.float()
        if bias is not None:
            v = v + bias.float()
        if p_eff > 0:
            keep = keep_mask_reference(x.numel(), seed, p_eff, x.device).view(x.shape)
            v = v * keep * (1.0 / (1.0 - p_eff))
        return (v + residual.float()).to(x.dtype)
    out = torch.empty_like(x)
    fn = K.proto("dh_bda_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_uint64, c_int, c_void_p])
    K.check(fn(x.data_ptr(), K.ptr(bias), residual.data_ptr(), out.data_ptr(), x.numel(), x.shape[-1], p_eff, seed,
               sm_budget, K.stream_ptr(stream)), "dh_bda_fwd")
    return out


def bda_bwd(dout, p: float = 0.0, seed: int = 0, training: bool = True, sm_budget: int = 0, stream=None):
    """Returns ``dx`` (gradient of the dropout branch).  The residual gradient is ``dout`` itself."""
    p_eff = p if training else 0.0
    if p_eff == 0.0:
        return dout
    if not K.use_native(dout):
        keep = keep_mask_reference(dout.numel(), seed, p_eff, dout.device).view(dout.shape)
        return (dout.float() * keep * (1.0 / (1.0 - p_eff))).to(dout.dtype)
    dx = torch.empty_like(dout)
    fn = K.proto("dh_bda_bwd", [c_void_p, c_void_p, c_int64, c_float, c_uint64, c_int, c_void_p])
    K.check(fn(dout.data_ptr(), dx.data_ptr(), dout.numel(), p_eff, seed, sm_budget, K.stream_ptr(stream)), "dh_bda_bwd")
    return dx


# Name kept for users of the reference's native module (csrc/torchapi.cpp:5).
def pybda(x, bias, residual, p=0.1, seed=0, stream=None, profiling=False):
    return bda_fwd(x, residual, bias, p, seed, stream=stream)
