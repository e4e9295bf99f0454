"""PyTorch / vendor-library implementations of the heavy ops, for the composition arm only.

The reference trains through ``torch.matmul`` / ``torch.addmm`` (cuBLAS;
dhellam/operators/layernorm_column.py:32,239,290-292), the flash-attention 2 package
(dhellam/operators/ring_attn.py:20-23, csrc/operators/flash_atten.cu), NCCL collectives
(dhellam/operators/comm.py:13-58) and eager / jit-fused PyTorch elementwise ops.  It cannot be
installed on this machine, so the benchmark carries a labelled *composition* of the same
recipe: with ``kernels.set_backend("library")`` every op of the ops layer runs either its
PyTorch restatement (norm, activation, bias-dropout-add, RoPE, embedding, cross-entropy: the
fp32 reference paths in those modules, which are plain PyTorch and run on CUDA tensors too) or
one of the functions below, and ``libdhellam_b200.so`` is never loaded.

Nothing here is used by the product path.
"""
from __future__ import annotations

import math

import torch

_FLASH = None            # None = not probed, False = unusable here, else the extension module
ATTENTION_IMPL = "unprobed"


# ----------------------------------------------------------------------------- GEMM (cuBLAS through torch.matmul)
def gemm_nt(x, w, out=None, out_dtype=None):
    if out is not None:
        return torch.matmul(x, w.t(), out=out)
    y = torch.matmul(x, w.t())
    return y if out_dtype in (None, y.dtype) else y.to(out_dtype)


def gemm_nn(dy, w, out=None):
    return torch.matmul(dy, w, out=out) if out is not None else torch.matmul(dy, w)


def gemm_tn_acc(dy, x, main_grad, accumulate=True):
    """Weight gradient in the parameters' dtype, then added into the fp32 ``main_grad`` (what a
    Megatron run without a fused accumulate kernel does)."""
    g = torch.matmul(dy.t(), x)
    if accumulate:
        main_grad.add_(g)
    else:
        main_grad.copy_(g)
    return main_grad


# ----------------------------------------------------------------------------- attention (flash-attn 2 package, else SDPA)
class AttnCtx:
    """Opaque stand-in for the softmax statistics when attention runs through autograd (SDPA
    fall-back): carries the graph from the forward to the backward op."""
    is_cuda = False

    def __init__(self, q, k, v, o):
        self.q, self.k, self.v, self.o = q, k, v, o


def _flash_module():
    global _FLASH, ATTENTION_IMPL
    if _FLASH is None:
        try:
            import flash_attn_2_cuda as m          # the compiled extension of the flash_attn 2.x wheel
            import flash_attn
            _FLASH = m
            ATTENTION_IMPL = f"flash_attn {flash_attn.__version__}"
        except Exception as e:                      # wheel absent or not loadable here
            _FLASH = False
            ATTENTION_IMPL = f"torch SDPA (flash_attn unusable: {type(e).__name__})"
    return _FLASH


def _bshd(t):
    """``[S, B, H, d]`` (sequence-first, as the engine keeps it) viewed as ``[B, S, H, d]``."""
    return t.permute(1, 0, 2, 3)


def attn_fwd(q, k, v, causal, scale):
    """Returns ``(out [Sq,B,Hq,d], lse [B,Hq,Sq] fp32)`` (or an ``AttnCtx`` in place of lse)."""
    global _FLASH, ATTENTION_IMPL
    Sq, B, Hq, d = q.shape
    out = torch.empty((Sq, B, Hq, d), dtype=q.dtype, device=q.device)
    fa = _flash_module()
    if fa:
        try:
            res = fa.fwd(_bshd(q), _bshd(k), _bshd(v), _bshd(out), None, 0.0, float(scale), bool(causal), -1, -1, 0.0, False, None)
            return out, res[1]
        except Exception as e:                      # e.g. no kernel image for this GPU in the wheel
            _FLASH = False
            ATTENTION_IMPL = f"torch SDPA (flash_attn failed: {str(e)[:80]})"
    qa = q.detach().permute(1, 2, 0, 3).requires_grad_(True)       # B H S d
    ka = k.detach().permute(1, 2, 0, 3).requires_grad_(True)
    va = v.detach().permute(1, 2, 0, 3).requires_grad_(True)
    with torch.enable_grad():
        o = torch.nn.functional.scaled_dot_product_attention(qa, ka, va, is_causal=bool(causal), scale=float(scale),
                                                             enable_gqa=(k.shape[2] != Hq))
    out.copy_(o.detach().permute(2, 0, 1, 3))
    return out, AttnCtx(qa, ka, va, o)


def attn_bwd(dout, q, k, v, out, lse, dq, dk, dv, causal, scale):
    if isinstance(lse, AttnCtx):
        gq, gk, gv = torch.autograd.grad(lse.o, (lse.q, lse.k, lse.v), dout.permute(1, 2, 0, 3))
        dq.copy_(gq.permute(2, 0, 1, 3)), dk.copy_(gk.permute(2, 0, 1, 3)), dv.copy_(gv.permute(2, 0, 1, 3))
        return dq, dk, dv
    fa = _flash_module()
    fa.bwd(_bshd(dout), _bshd(q), _bshd(k), _bshd(v), _bshd(out), lse, _bshd(dq), _bshd(dk), _bshd(dv), None, 0.0, float(scale),
           bool(causal), -1, -1, 0.0, False, None, None)
    return dq, dk, dv


# ----------------------------------------------------------------------------- optimizer pieces
def sum_squares(t):
    return (torch.linalg.vector_norm(t.reshape(-1), 2.0, dtype=torch.float32) ** 2).reshape(1)


def adam_update(param, master, m, v, grad, lr, b1, b2, eps, wd, step, grad_scale=1.0, chunk: int = 1 << 28):
    """AdamW on fp32 master weights through PyTorch's fused multi-tensor kernel, in chunks so
    that no temporary of the model's size appears; then the low-precision copy."""
    n = master.numel()
    step_t = torch.full((), float(step), dtype=torch.float32, device=master.device)
    inv = torch.full((), 1.0 / grad_scale if grad_scale != 0 else 1.0, dtype=torch.float32, device=master.device)
    for a in range(0, n, chunk):
        b = min(a + chunk, n)
        g = grad[a:b]
        if grad_scale == 0:
            g = torch.zeros_like(g)
        torch._fused_adamw_([master[a:b]], [g], [m[a:b]], [v[a:b]], [], [step_t], lr=float(lr), beta1=float(b1), beta2=float(b2),
                            weight_decay=float(wd), eps=float(eps), amsgrad=False, maximize=False, grad_scale=inv, found_inf=None)
        param[a:b].copy_(master[a:b])
