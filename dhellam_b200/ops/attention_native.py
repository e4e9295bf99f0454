"""ctypes glue for the sm_100a attention backward (csrc/attention_sm100.cu).

The backward needs scratch memory beyond its inputs and outputs: ``delta = rowsum(dO * O)``,
one fp32 per query row and head, which both backward kernels read, and, when the dK/dV kernel
splits the query heads of a KV head over several CTAs (few KV heads per GPU), their fp32
partial sums.  The scratch is taken from a small per-device cache here so that the hot path
does not allocate.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .. import kernels as K

_scratch = {}


def _scratch_for(device, nbytes: int):
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def attn_bwd_native(dout, q, k, v, out, lse, dq, dk, dv, causal, scale, sm_budget=0, stream=None):
    Sq, B, Hq, d = q.shape
    Sk, Hk = k.shape[0], k.shape[2]
    for t in (dout, q, k, v, out, dq, dk, dv):
        assert t.stride(3) == 1 and t.dtype == torch.bfloat16
    nbytes_fn = K.proto("dh_attn_bwd_scratch_bytes", [c_int, c_int, c_int, c_int, c_int], c_int64)
    scratch = _scratch_for(q.device, nbytes_fn(B, Hq, Hk, Sq, Sk))
    strides = []
    for t in (dout, q, k, v, out, dq, dk, dv):
        strides += [t.stride(0), t.stride(1), t.stride(2)]
    arr = (c_int64 * 24)(*strides)
    fn = K.proto("dh_attn_bwd", [c_void_p] * 10 + [ctypes.POINTER(c_int64), c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_float, c_int, c_void_p])
    K.check(fn(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), dq.data_ptr(),
               dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(), arr, B, Hq, Hk, Sq, Sk, d, 1 if causal else 0, scale,
               sm_budget, K.stream_ptr(stream)), "dh_attn_bwd")
