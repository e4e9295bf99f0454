"""Vocabulary-parallel cross-entropy and loss scaling.

The reference computes the loss with three tensor-parallel all-reduces (max, target
logit, sum of exponentials; dhellam/operators/loss.py:15-98, or Megatron's
``vocab_parallel_cross_entropy`` from dhellam/core/dshb.py:106).  Here every rank reduces
its vocabulary shard to three numbers per token ``(local max, sum exp(logit - local max),
target logit or 0)`` in one pass, the ranks exchange those triples in ONE all-gather, and
each rank combines them locally.  The backward overwrites the logits buffer with
``(softmax - onehot) * grad`` in place.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p

import torch
import torch.distributed as dist

from .. import kernels as K
from .comm import group_size


def ce_local_stats(logits, labels, vocab_start: int, sm_budget: int = 0, stream=None):
    """``stats [T,3] fp32 = (max, sumexp relative to max, target logit if owned else 0)``."""
    T, Vl = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        m = lf.max(dim=-1).values
        se = torch.exp(lf - m[:, None]).sum(-1)
        loc = labels.long() - vocab_start
        own = (loc >= 0) & (loc < Vl)
        tgt = torch.where(own, lf.gather(1, loc.clamp(0, Vl - 1)[:, None]).squeeze(1), torch.zeros_like(m))
        return torch.stack([m, se, tgt], dim=1)
    stats = torch.empty((T, 3), dtype=torch.float32, device=logits.device)
    fn = K.proto("dh_ce_stats", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_void_p])
    K.check(fn(logits.data_ptr(), labels.data_ptr(), stats.data_ptr(), T, Vl, logits.stride(0), vocab_start,
               int(logits.dtype == torch.float32), sm_budget, K.stream_ptr(stream)), "dh_ce_stats")
    return stats


def ce_combine_stats(all_stats):
    """``all_stats [R,T,3]`` -> ``(loss [T], lse [T])``."""
    m = all_stats[..., 0]
    gmax = m.max(dim=0).values
    se = (all_stats[..., 1] * torch.exp(m - gmax[None])).sum(0)
    tgt = all_stats[..., 2].sum(0)
    lse = torch.log(se) + gmax
    return lse - tgt, lse


def vocab_parallel_ce_fwd(logits, labels, vocab_start: int = 0, group=None, stream=None):
    """Returns ``(loss_per_token [T] fp32, lse [T] fp32)``."""
    stats = ce_local_stats(logits, labels, vocab_start, stream=stream)
    ws = group_size(group)
    if ws > 1:
        T = stats.shape[0]
        flat = torch.empty((ws * T, 3), dtype=stats.dtype, device=stats.device)
        dist.all_gather_into_tensor(flat, stats, group=group)
        gathered = flat.view(ws, T, 3)
    else:
        gathered = stats.unsqueeze(0)
    return ce_combine_stats(gathered)


def vocab_parallel_ce_bwd_(logits, labels, lse, grad_per_token, vocab_start: int = 0, sm_budget: int = 0, stream=None):
    """Overwrites ``logits`` with ``d loss / d logits`` and returns it."""
    T, Vl = logits.shape
    if not logits.is_cuda:
        p = torch.exp(logits.float() - lse[:, None])
        loc = labels.long() - vocab_start
        own = (loc >= 0) & (loc < Vl)
        rows = torch.nonzero(own).squeeze(1)
        p[rows, loc[rows]] -= 1.0
        logits.copy_((p * grad_per_token[:, None]).to(logits.dtype))
        return logits
    fn = K.proto("dh_ce_grad_inplace", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int,
                                        c_void_p])
    K.check(fn(logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), grad_per_token.data_ptr(), T, Vl, logits.stride(0),
               vocab_start, int(logits.dtype == torch.float32), sm_budget, K.stream_ptr(stream)), "dh_ce_grad_inplace")
    return logits


def mask_scale_loss_fwd(loss_per_token, loss_mask, scale_func=None):
    """Masked mean with an optional loss-scaling hook (``optimizer.scale_loss`` in the
    reference: dhellam/operators/loss.py:131-164).  Returns ``(scaled_loss, sum, count)``."""
    m = loss_mask.reshape(-1).float()
    s = (loss_per_token.reshape(-1).float() * m).sum()
    n = m.sum()
    loss = s / n.clamp_min(1.0)
    return (scale_func(loss) if scale_func is not None else loss), s, n


def mask_scale_loss_bwd(loss_mask, count, grad_scale: float = 1.0):
    """Gradient of the masked mean with respect to each token's loss."""
    return loss_mask.reshape(-1).float() * (grad_scale / count.clamp_min(1.0))
