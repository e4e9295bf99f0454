"""Rotary position embedding applied in place to the Q and K heads of a packed QKV buffer.

The reference uses learned absolute positions (dhellam/core/dshb.py:250-255); RoPE is
needed for the Llama family.  Layout of one row of ``qkv``:
``[nq heads x d | nkv heads x d | nkv heads x d]``; pairs are ``(i, i + d/2)``.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from functools import lru_cache

import torch

from .. import kernels as K


def rope_table(max_pos: int, d: int, theta: float, device="cpu"):
    """Returns ``(cos, sin)``, each ``[max_pos, d/2]`` fp32."""
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope_apply_(qkv, positions, cos, sin, nq: int, nkv: int, d: int, inverse: bool = False, sm_budget: int = 0, stream=None):
    """Rotates the first ``nq + nkv`` heads of every row of ``qkv [T, (nq+2nkv)*d]`` in place.

    ``positions [T]`` int32 gives the sequence position of each row.  ``inverse`` applies
    the transposed rotation, which is the backward of the forward rotation.
    """
    T = qkv.shape[0]
    assert qkv.shape[1] == (nq + 2 * nkv) * d
    if not K.use_native(qkv):
        v = qkv[:, : (nq + nkv) * d].float().view(T, nq + nkv, d)
        c = cos[positions.long()][:, None, :]
        s = sin[positions.long()][:, None, :]
        if inverse:
            s = -s
        x1, x2 = v[..., : d // 2], v[..., d // 2:]
        r = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        qkv[:, : (nq + nkv) * d] = r.view(T, -1).to(qkv.dtype)
        return qkv
    fn = K.proto("dh_rope_inplace", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p])
    K.check(fn(qkv.data_ptr(), positions.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, qkv.stride(0), nq + nkv, d,
               1 if inverse else 0, sm_budget, K.stream_ptr(stream)), "dh_rope_inplace")
    return qkv
