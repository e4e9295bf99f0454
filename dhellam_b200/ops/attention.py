"""Causal / full multi-head attention with grouped KV heads, explicit forward and backward.

Role of the reference's ``pymha_varlen_fwd`` / ``pymha_varlen_bwd`` (flash-attention 2
wrappers, csrc/operators/flash_atten.cu:220-434, 479-757) and of the per-ring-step calls in
dhellam/operators/ring_attn.py:97-144, 315-381.  Operands are strided 4-D views
``[S, B, heads, d]`` (sequence-first, so a packed QKV buffer is used without copies); the
softmax statistics are returned as ``lse [B, heads, S]`` in fp32 (natural log).

CUDA tensors run the tcgen05 flash-attention kernels (csrc/attention_sm100.cu); CPU tensors
run the fp32 reference below.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .. import kernels as K


def _ref_fwd(q, k, v, causal, scale):
    Sq, B, Hq, d = q.shape
    Sk, Hk = k.shape[0], k.shape[2]
    g = Hq // Hk
    qf = q.float().permute(1, 2, 0, 3)                      # B Hq Sq d
    kf = k.float().permute(1, 2, 0, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(1, 2, 0, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale       # B Hq Sq Sk
    if causal:
        # bottom-right aligned: query i sees keys j <= i + (Sk - Sq)
        i = torch.arange(Sq, device=q.device)[:, None]
        j = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(j > i + (Sk - Sq), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                         # B Hq Sq
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf)                                  # B Hq Sq d
    return o.permute(2, 0, 1, 3).contiguous(), lse, p


def attn_fwd(q, k, v, causal: bool = True, scale: float | None = None, sm_budget: int = 0, stream=None, out=None):
    """Returns ``(out [Sq,B,Hq,d], lse [B,Hq,Sq] fp32)``.  ``out`` may name a contiguous destination of
    that shape (for example a slice along the sequence of a larger output)."""
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if K.use_library(q):
        from . import library as LIB
        o, lse = LIB.attn_fwd(q, k, v, causal, scale)
        if out is not None:
            out.copy_(o)
            return out, lse
        return o, lse
    if not q.is_cuda:
        o, lse, _ = _ref_fwd(q, k, v, causal, scale)
        if out is not None:
            out.copy_(o.to(q.dtype))
            return out, lse
        return o.to(q.dtype), lse
    Sq, B, Hq, _ = q.shape
    Sk, Hk = k.shape[0], k.shape[2]
    assert q.stride(3) == 1 and k.stride(3) == 1 and v.stride(3) == 1
    if out is None:
        out = torch.empty((Sq, B, Hq, d), dtype=q.dtype, device=q.device)
    else:
        assert tuple(out.shape) == (Sq, B, Hq, d) and out.is_contiguous() and out.dtype == q.dtype
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    fn = K.proto("dh_attn_fwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    K.check(fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
               q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
               v.stride(0), v.stride(1), v.stride(2),
               B, Hq, Hk, Sq, Sk, d, 1 if causal else 0, scale, sm_budget, K.stream_ptr(stream)), "dh_attn_fwd")
    return out, lse


def attn_bwd(dout, q, k, v, out, lse, causal: bool = True, scale: float | None = None, dq=None, dk=None, dv=None,
             sm_budget: int = 0, stream=None):
    """Returns ``(dq, dk, dv)`` shaped like ``q, k, v``.  ``dq/dk/dv`` may be given as strided
    views (for example into a packed dQKV buffer) and are then written in place, which
    removes the reference's ``cat(dq, dk, dv)`` (dhellam/core/dstb.py:379-384)."""
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if K.use_library(q):
        from . import library as LIB
        if dq is None:
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        return LIB.attn_bwd(dout, q, k, v, out, lse, dq, dk, dv, causal, scale)
    if not q.is_cuda:
        Sq, B, Hq, _ = q.shape
        Sk, Hk = k.shape[0], k.shape[2]
        g = Hq // Hk
        do = dout.float().permute(1, 2, 0, 3)                # B Hq Sq d
        of = out.float().permute(1, 2, 0, 3)
        qf = q.float().permute(1, 2, 0, 3)
        kf = k.float().permute(1, 2, 0, 3).repeat_interleave(g, dim=1)
        vf = v.float().permute(1, 2, 0, 3).repeat_interleave(g, dim=1)
        # probabilities are rebuilt from the GIVEN statistics, which for a ring step are
        # those of the whole key set, not of this block alone
        s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        if causal:
            i = torch.arange(Sq, device=q.device)[:, None]
            j = torch.arange(Sk, device=q.device)[None, :]
            s = s.masked_fill(j > i + (Sk - Sq), float("-inf"))
        p = torch.exp(s - lse.unsqueeze(-1))
        dvf = torch.matmul(p.transpose(-1, -2), do)          # B Hq Sk d
        dp = torch.matmul(do, vf.transpose(-1, -2))
        delta = (do * of).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dqf = torch.matmul(ds, kf)
        dkf = torch.matmul(ds.transpose(-1, -2), qf)
        dkf = dkf.view(B, Hk, g, Sk, d).sum(2)
        dvf = dvf.view(B, Hk, g, Sk, d).sum(2)
        rq = dqf.permute(2, 0, 1, 3).to(q.dtype)
        rk = dkf.permute(2, 0, 1, 3).to(k.dtype)
        rv = dvf.permute(2, 0, 1, 3).to(v.dtype)
        if dq is not None:
            dq.copy_(rq), dk.copy_(rk), dv.copy_(rv)
            return dq, dk, dv
        return rq.contiguous(), rk.contiguous(), rv.contiguous()
    Sq, B, Hq, _ = q.shape
    Sk, Hk = k.shape[0], k.shape[2]
    if dq is None:
        dq = torch.empty((Sq, B, Hq, d), dtype=q.dtype, device=q.device)
        dk = torch.empty((Sk, B, Hk, d), dtype=q.dtype, device=q.device)
        dv = torch.empty((Sk, B, Hk, d), dtype=q.dtype, device=q.device)
    from .attention_native import attn_bwd_native
    attn_bwd_native(dout, q, k, v, out, lse, dq, dk, dv, causal, scale, sm_budget, stream)
    return dq, dk, dv


def merge_attention_partials(o_a, lse_a, o_b, lse_b):
    """Combines two attention partial results over disjoint key sets (fp32 math; the
    reference does this step in fp64, dhellam/operators/ring_attn.py:26-40)."""
    lse = torch.logaddexp(lse_a, lse_b)                      # B H S
    wa = torch.exp(lse_a - lse).permute(2, 0, 1).unsqueeze(-1)
    wb = torch.exp(lse_b - lse).permute(2, 0, 1).unsqueeze(-1)
    o = o_a.float() * wa + o_b.float() * wb
    return o.to(o_a.dtype), lse


# ----------------------------------------------------------------------------- variable-length API
def set_attn_bwd_mode(mode: int):
    """dK/dV kernel on the GPU: 0 = one 128-query tile per iteration (default), 1 = the pipelined
    transposed-score form, -1 = re-read ``DHELLAM_ATTN_BWD_T`` at the next call."""
    K.proto("dh_attn_set_bwd_mode", [c_int], None)(int(mode))


def _offsets(cu):
    """``cu_seqlens`` as a Python list.  A CUDA tensor costs a device synchronisation here; pass a CPU tensor or a
    list (the offsets are known on the host in every caller of this package) to avoid it."""
    return [int(x) for x in (cu.tolist() if torch.is_tensor(cu) else cu)]


def _uniform_length(cu):
    """Common length of the sequences described by cumulative offsets ``cu`` (starting at 0), or 0 if they differ."""
    if len(cu) < 2 or cu[0] != 0:
        return 0
    n = cu[1] - cu[0]
    return n if n > 0 and all(cu[i + 1] - cu[i] == n for i in range(len(cu) - 1)) else 0


def _as_sbhd(t, b, s):
    """Packed ``[b * s, h, d]`` seen as ``[s, b, h, d]`` (a view; the kernels take strides)."""
    return t.view(b, s, t.shape[1], t.shape[2]).permute(1, 0, 2, 3)


def pymha_varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout: float = 0.0,
                     softmax_scale: float | None = None, is_causal: bool = True, return_softmax: bool = False,
                     math_sm_count: int = 0, profiling: bool = False):
    """Packed variable-length attention with the reference's signature
    (csrc/operators/ops.h:18-32): ``q [total_q, h, d]``, ``k, v [total_k, h_k, d]`` and
    cumulative sequence offsets.  Returns ``(out [total_q, h, d], softmax_lse [b, h, max_q])``.
    A batch of equal-length sequences runs as ONE launch over strided views of the packed tensors; sequences
    of different lengths run one strided call each, so no padding copy is made.  Attention dropout is not supported by the sm_100a kernel (``p_dropout`` must be 0)."""
    assert p_dropout == 0.0, "attention dropout is not implemented"
    cq = _offsets(cu_seqlens_q)
    ck = _offsets(cu_seqlens_k)
    b = len(cq) - 1
    sq, sk = _uniform_length(cq), _uniform_length(ck)
    if sq and sk and sq == max_seqlen_q:
        # every sequence has the same length (the reference's own use: a micro-batch of fixed-length samples):
        # the packed [b * s, h, d] tensors are [s, b, h, d] tensors with other strides, one launch does it all
        o, lse = attn_fwd(_as_sbhd(q, b, sq), _as_sbhd(k, b, sk), _as_sbhd(v, b, sk), is_causal, softmax_scale,
                          sm_budget=abs(math_sm_count))
        return o.permute(1, 0, 2, 3).reshape(q.shape), lse
    out = torch.empty_like(q)
    lse = torch.full((b, q.shape[1], max_seqlen_q), float("-inf"), dtype=torch.float32, device=q.device)
    for i in range(b):
        qi, ki, vi = q[cq[i]:cq[i + 1]].unsqueeze(1), k[ck[i]:ck[i + 1]].unsqueeze(1), v[ck[i]:ck[i + 1]].unsqueeze(1)
        o, l = attn_fwd(qi, ki, vi, is_causal, softmax_scale, sm_budget=abs(math_sm_count))
        out[cq[i]:cq[i + 1]] = o.squeeze(1)
        lse[i, :, : cq[i + 1] - cq[i]] = l[0]
    return out, lse


def pymha_varlen_bwd(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, p_dropout: float = 0.0,
                     softmax_scale: float | None = None, is_causal: bool = True, rng_state=None, deterministic: bool = False,
                     math_sm_count: int = 0, profiling: bool = False, stream_ptr: int = 0):
    """Backward of ``pymha_varlen_fwd`` (csrc/operators/ops.h:34-52).  Returns ``(dq, dk, dv)``."""
    cq = _offsets(cu_seqlens_q)
    ck = _offsets(cu_seqlens_k)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    b = len(cq) - 1
    sq, sk = _uniform_length(cq), _uniform_length(ck)
    if sq and sk and sq == max_seqlen_q and softmax_lse.shape[-1] == sq:
        a, b_, c = attn_bwd(_as_sbhd(dout, b, sq), _as_sbhd(q, b, sq), _as_sbhd(k, b, sk), _as_sbhd(v, b, sk), _as_sbhd(out, b, sq),
                            softmax_lse, is_causal, softmax_scale, sm_budget=abs(math_sm_count))
        dq.copy_(a.permute(1, 0, 2, 3).reshape(q.shape))
        dk.copy_(b_.permute(1, 0, 2, 3).reshape(k.shape))
        dv.copy_(c.permute(1, 0, 2, 3).reshape(v.shape))
        return dq, dk, dv
    for i in range(len(cq) - 1):
        sl_q, sl_k = slice(cq[i], cq[i + 1]), slice(ck[i], ck[i + 1])
        lse_i = softmax_lse[i:i + 1, :, : cq[i + 1] - cq[i]].contiguous()
        a, b_, c = attn_bwd(dout[sl_q].unsqueeze(1), q[sl_q].unsqueeze(1), k[sl_k].unsqueeze(1), v[sl_k].unsqueeze(1),
                            out[sl_q].unsqueeze(1), lse_i, is_causal, softmax_scale, sm_budget=abs(math_sm_count))
        dq[sl_q], dk[sl_k], dv[sl_k] = a.squeeze(1), b_.squeeze(1), c.squeeze(1)
    return dq, dk, dv
