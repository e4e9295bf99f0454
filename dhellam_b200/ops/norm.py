"""RMSNorm / LayerNorm with explicit forward and backward.

Role of the reference's ``pylayernorm_fwd`` / ``pylayernorm_bwd`` (TransformerEngine
``tex.layernorm_fwd/bwd``; dhellam/operators/layernorm.py:6-91) and of the LN-backward op
that also adds the residual gradient and accumulates the affine gradients into
``main_grad`` (dhellam/core/dstb.py:387-405).  RMSNorm is added for the Llama family.

CUDA tensors run the sm_100a kernels (csrc/norm.cu); CPU tensors run the fp32 reference.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from .. import kernels as K


def _rows(x):
    return x.numel() // x.shape[-1], x.shape[-1]


# ----------------------------------------------------------------------------- reference
def _rms_fwd_ref(x, w, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * w.float()).to(x.dtype)
    return y, rstd.squeeze(-1)


def _rms_bwd_ref(dy, x, w, rstd):
    xf, dyf, wf = x.float(), dy.float(), w.float()
    r = rstd.unsqueeze(-1)
    xhat = xf * r
    g = dyf * wf
    dx = r * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
    return dx, dw


def _ln_fwd_ref(x, w, b, eps):
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = ((xf - mu) * rstd * w.float() + (b.float() if b is not None else 0.0)).to(x.dtype)
    return y, mu.squeeze(-1), rstd.squeeze(-1)


def _ln_bwd_ref(dy, x, w, mu, rstd):
    xf, dyf, wf = x.float(), dy.float(), w.float()
    r = rstd.unsqueeze(-1)
    xhat = (xf - mu.unsqueeze(-1)) * r
    g = dyf * wf
    dx = r * (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True))
    dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
    db = dyf.reshape(-1, x.shape[-1]).sum(0)
    return dx, dw, db


# ----------------------------------------------------------------------------- public
def rmsnorm_fwd(x, weight, eps: float = 1e-5, sm_budget: int = 0, stream=None):
    """Returns ``(y, rstd)``; ``rstd`` is fp32 per row."""
    if not K.use_native(x):
        return _rms_fwd_ref(x, weight, eps)
    rows, h = _rows(x)
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    fn = K.proto("dh_rmsnorm_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    K.check(fn(x.data_ptr(), weight.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, h, eps, sm_budget, K.stream_ptr(stream)),
            "dh_rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy, x, weight, rstd, weight_main_grad=None, residual_grad=None, sm_budget: int = 0, stream=None):
    """``dx = rmsnorm'(dy) (+ residual_grad)``; the weight gradient is added into
    ``weight_main_grad`` (fp32) when given, else returned."""
    if not K.use_native(x):
        dx, dw = _rms_bwd_ref(dy, x, weight, rstd)
        if residual_grad is not None:
            dx = dx + residual_grad.float()
        dx = dx.to(x.dtype)
        if weight_main_grad is not None:
            weight_main_grad.add_(dw.to(weight_main_grad.dtype))
            return dx, None
        return dx, dw
    rows, h = _rows(x)
    dx = torch.empty_like(x)
    ret = None
    if weight_main_grad is None:
        weight_main_grad = torch.zeros(h, dtype=torch.float32, device=x.device)
        ret = weight_main_grad
    if K.deterministic():
        grid = K.proto("dh_norm_bwd_grid", [c_int, c_int])(rows, sm_budget)
        partial = K.det_scratch(x.device, grid * h)
        fn = K.proto("dh_rmsnorm_bwd_det", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_void_p])
        K.check(fn(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), rstd.data_ptr(), K.ptr(residual_grad), dx.data_ptr(),
                   weight_main_grad.data_ptr(), partial.data_ptr(), rows, h, sm_budget, K.stream_ptr(stream)), "dh_rmsnorm_bwd_det")
        return dx, ret
    fn = K.proto("dh_rmsnorm_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                    c_int, c_void_p])
    K.check(fn(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), rstd.data_ptr(), K.ptr(residual_grad), dx.data_ptr(),
               weight_main_grad.data_ptr(), rows, h, sm_budget, K.stream_ptr(stream)), "dh_rmsnorm_bwd")
    return dx, ret


def layernorm_fwd(x, weight, bias, eps: float = 1e-5, sm_budget: int = 0, stream=None):
    """Returns ``(y, mu, rstd)`` like the reference's ``pylayernorm_fwd``."""
    if not K.use_native(x):
        return _ln_fwd_ref(x, weight, bias, eps)
    rows, h = _rows(x)
    y = torch.empty_like(x)
    mu = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mu)
    fn = K.proto("dh_layernorm_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                      c_int, c_void_p])
    K.check(fn(x.data_ptr(), weight.data_ptr(), K.ptr(bias), y.data_ptr(), mu.data_ptr(), rstd.data_ptr(), rows, h, eps,
               sm_budget, K.stream_ptr(stream)), "dh_layernorm_fwd")
    return y, mu, rstd


def layernorm_bwd(dy, x, weight, mu, rstd, weight_main_grad=None, bias_main_grad=None, residual_grad=None,
                  sm_budget: int = 0, stream=None):
    """Returns ``(dx, dw, db)``; ``dw``/``db`` are None when accumulated into the given buffers."""
    if not K.use_native(x):
        dx, dw, db = _ln_bwd_ref(dy, x, weight, mu, rstd)
        if residual_grad is not None:
            dx = dx + residual_grad.float()
        dx = dx.to(x.dtype)
        if weight_main_grad is not None:
            weight_main_grad.add_(dw.to(weight_main_grad.dtype))
            dw = None
        if bias_main_grad is not None:
            bias_main_grad.add_(db.to(bias_main_grad.dtype))
            db = None
        return dx, dw, db
    rows, h = _rows(x)
    dx = torch.empty_like(x)
    rw = rb = None
    if weight_main_grad is None:
        weight_main_grad = rw = torch.zeros(h, dtype=torch.float32, device=x.device)
    if bias_main_grad is None:
        bias_main_grad = rb = torch.zeros(h, dtype=torch.float32, device=x.device)
    if K.deterministic():
        grid = K.proto("dh_norm_bwd_grid", [c_int, c_int])(rows, sm_budget)
        partial = K.det_scratch(x.device, 2 * grid * h)
        fn = K.proto("dh_layernorm_bwd_det", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        K.check(fn(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), mu.data_ptr(), rstd.data_ptr(), K.ptr(residual_grad),
                   dx.data_ptr(), weight_main_grad.data_ptr(), bias_main_grad.data_ptr(), partial.data_ptr(), rows, h, sm_budget,
                   K.stream_ptr(stream)), "dh_layernorm_bwd_det")
        return dx, rw, rb
    fn = K.proto("dh_layernorm_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_void_p])
    K.check(fn(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), mu.data_ptr(), rstd.data_ptr(), K.ptr(residual_grad),
               dx.data_ptr(), weight_main_grad.data_ptr(), bias_main_grad.data_ptr(), rows, h, sm_budget,
               K.stream_ptr(stream)), "dh_layernorm_bwd")
    return dx, rw, rb


# Names kept for users of the reference package (dhellam/__init__.py:1-5).
def pylayernorm_fwd(x, weight, bias, eps, sm_margin=0, zero_centered_gamma=False, stream=None, profiling=False):
    w = weight + 1 if zero_centered_gamma else weight
    y, mu, rstd = layernorm_fwd(x, w, bias, eps, stream=stream)
    return y, mu, rstd, 0.0


def pylayernorm_bwd(dy, x, mu, rstd, weight, sm_margin=0, zero_centered_gamma=False, stream=None, profiling=False):
    w = weight + 1 if zero_centered_gamma else weight
    dx, dw, db = layernorm_bwd(dy, x, w, mu, rstd, stream=stream)
    return dx, dw, db, 0.0
