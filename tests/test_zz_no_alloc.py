"""The attention backward for callers that cannot allocate device memory
(``dh_attn_bwd_noalloc``, declared in dhellam_b200/csrc/attn_noalloc.h).

Such a caller is, for instance, a program that reserved the whole GPU for its own pools and
forbids ``cudaMalloc`` in the libraries it loads, or one that links the kernel library from
C without any tensor framework.  The entry point keeps its scratch in an array inside the
library and is called here the way such a program would call it: through the exported C
symbol, with raw pointers.  Its results must equal those of the regular entry point, whose
scratch comes from an allocator, and a second call must not be disturbed by what the first
one left in the shared array.

This file sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _call_noalloc(lib, dout, q, k, v, out, lse, causal, scale):
    Sq, B, Hq, d = q.shape
    Sk, Hk = k.shape[0], k.shape[2]
    dq = torch.empty((Sq, B, Hq, d), dtype=q.dtype, device=q.device)
    dk = torch.empty((Sk, B, Hk, d), dtype=q.dtype, device=q.device)
    dv = torch.empty((Sk, B, Hk, d), dtype=q.dtype, device=q.device)
    strides = []
    for t in (dout, q, k, v, out, dq, dk, dv):
        strides += [t.stride(0), t.stride(1), t.stride(2)]
    arr = (c_int64 * 24)(*strides)
    fn = lib.dh_attn_bwd_noalloc
    fn.argtypes = [c_void_p] * 9 + [ctypes.POINTER(c_int64), c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    fn.restype = c_int
    rc = fn(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), dq.data_ptr(), dk.data_ptr(),
            dv.data_ptr(), arr, B, Hq, Hk, Sq, Sk, d, 1 if causal else 0, scale, torch.cuda.current_stream().cuda_stream)
    return rc, dq, dk, dv


def test_noalloc_attention_backward_matches_regular_entry_point_twice():
    from dhellam_b200 import kernels as K
    from dhellam_b200.ops.attention import attn_bwd, attn_fwd
    lib = K.lib()
    torch.manual_seed(7)
    d = 128
    scale = 1.0 / math.sqrt(d)
    # different problems back to back: none must see its predecessor's leftovers
    # the third problem fills the built-in scratch exactly (4 x 16 x 4096 rows) and makes the regular
    # entry point split the 16 query heads of its one KV head over 8 CTAs, two heads each
    for (Sq, B, Hq, Hk, causal) in ((384, 2, 4, 2, True), (256, 1, 2, 1, False), (4096, 4, 16, 1, True)):
        qkv = torch.randn(Sq, B, Hq + 2 * Hk, d, device="cuda").to(torch.bfloat16)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hk], qkv[:, :, Hq + Hk:]
        out, lse = attn_fwd(q, k, v, causal, scale)
        dout = torch.randn(Sq, B, Hq, d, device="cuda").to(torch.bfloat16)
        ref_dq, ref_dk, ref_dv = attn_bwd(dout, q, k, v, out, lse, causal, scale)
        rc, dq, dk, dv = _call_noalloc(lib, dout, q, k, v, out, lse, causal, scale)
        assert rc == 0, lib.dh_last_error_string().decode()
        torch.cuda.synchronize()
        # dQ: same kernel, same inputs, no atomics: bitwise equal.  dK / dV: the regular entry
        # point may split the query heads of a KV head over several CTAs and add their fp32
        # partial sums afterwards (it has the scratch for that), so only the rounding can differ.
        assert torch.equal(dq, ref_dq)
        assert _rel(dk, ref_dk) < 5e-3
        assert _rel(dv, ref_dv) < 5e-3


def test_noalloc_attention_backward_rejects_oversized_problem():
    from dhellam_b200 import kernels as K
    lib = K.lib()
    d = 128
    # 8192 x 8 x 8 = 524288 rows need twice the built-in 1 MiB; nothing is launched,
    # so small placeholder tensors are enough for the pointer arguments
    Sq, B, Hq, Hk = 8192, 8, 8, 8
    t = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    fn = lib.dh_attn_bwd_noalloc
    fn.argtypes = [c_void_p] * 9 + [ctypes.POINTER(c_int64), c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    fn.restype = c_int
    arr = (c_int64 * 24)(*([B * Hq * d, Hq * d, d] * 8))
    rc = fn(*([t.data_ptr()] * 9), arr, B, Hq, Hk, Sq, Sq, d, 1, 0.088, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert "scratch" in lib.dh_last_error_string().decode()


def test_noalloc_attention_backward_against_fp32_reference_at_1024():
    """The same entry point against a plain fp32 attention backward (autograd over an explicit softmax),
    1024 positions, causal, four query heads per KV head."""
    from dhellam_b200 import kernels as K
    from dhellam_b200.ops.attention import attn_fwd
    lib = K.lib()
    torch.manual_seed(11)
    Sq, B, Hq, Hk, d = 1024, 2, 8, 2, 128
    scale = 1.0 / math.sqrt(d)
    q = torch.randn(Sq, B, Hq, d, device="cuda").to(torch.bfloat16)
    k = torch.randn(Sq, B, Hk, d, device="cuda").to(torch.bfloat16)
    v = torch.randn(Sq, B, Hk, d, device="cuda").to(torch.bfloat16)
    dout = torch.randn(Sq, B, Hq, d, device="cuda").to(torch.bfloat16)
    out, lse = attn_fwd(q, k, v, True, scale)
    rc, dq, dk, dv = _call_noalloc(lib, dout, q, k, v, out, lse, True, scale)
    assert rc == 0, lib.dh_last_error_string().decode()
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    g = Hq // Hk
    kk = kf.repeat_interleave(g, dim=2)
    vv = vf.repeat_interleave(g, dim=2)
    s = torch.einsum("sbhd,tbhd->bhst", qf, kk) * scale
    mask = torch.ones(Sq, Sq, device="cuda", dtype=torch.bool).tril()
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
    o = torch.einsum("bhst,tbhd->sbhd", p, vv)
    o.backward(dout.float())
    assert _rel(out, o.detach()) < 1e-2
    assert _rel(dq, qf.grad) < 1.5e-2
    assert _rel(dk, kf.grad) < 1.5e-2
    assert _rel(dv, vf.grad) < 1.5e-2
