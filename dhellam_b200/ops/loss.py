"""Vocabulary-parallel cross-entropy and loss scaling.

The reference computes the loss with three tensor-parallel all-reduces (max, target
logit, sum of exponentials; dhellam/operators/loss.py:15-98, or Megatron's
``vocab_parallel_cross_entropy`` from dhellam/core/dshb.py:106).  Here every rank reduces
its vocabulary shard to four numbers per token ``(local max, sum exp(logit - local max),
target logit or 0, sum of logits)`` in one pass, the ranks exchange those in ONE all-gather,
and each rank combines them locally.  The backward overwrites the logits buffer with
``(softmax - onehot) * grad`` in place.

Label smoothing follows the reference's definition (loss.py:66-88): with ``s' = s V / (V - 1)``
the loss is ``(1 - s') * ce - s' * mean_v(log p_v)``.  The mean runs over the WHOLE vocabulary
here (``mean_v log p_v = sum_v logit_v / V - lse``, which only needs the sum of the logits as a
fourth statistic); the reference takes it over the local partition only, which makes its loss
depend on the tensor-parallel size.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p

import torch
import torch.distributed as dist

from .. import kernels as K
from .comm import group_size


def ce_local_stats(logits, labels, vocab_start: int, sm_budget: int = 0, stream=None):
    """``stats [T,4] fp32 = (max, sumexp relative to max, target logit if owned else 0, sum of logits)``."""
    T, Vl = logits.shape
    if not K.use_native(logits):
        lf = logits.float()
        m = lf.max(dim=-1).values
        se = torch.exp(lf - m[:, None]).sum(-1)
        loc = labels.long() - vocab_start
        own = (loc >= 0) & (loc < Vl)
        tgt = torch.where(own, lf.gather(1, loc.clamp(0, Vl - 1)[:, None]).squeeze(1), torch.zeros_like(m))
        return torch.stack([m, se, tgt, lf.sum(-1)], dim=1)
    stats = torch.empty((T, 4), dtype=torch.float32, device=logits.device)
    fn = K.proto("dh_ce_stats", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_void_p])
    K.check(fn(logits.data_ptr(), labels.data_ptr(), stats.data_ptr(), T, Vl, logits.stride(0), vocab_start,
               int(logits.dtype == torch.float32), sm_budget, K.stream_ptr(stream)), "dh_ce_stats")
    return stats


def _smoothing(label_smoothing: float, vocab: int) -> float:
    if not label_smoothing:
        return 0.0
    assert 0.0 < label_smoothing < 1.0 and vocab > 1
    return label_smoothing * vocab / (vocab - 1)


def ce_combine_stats(all_stats, label_smoothing: float = 0.0, vocab: int = 0):
    """``all_stats [R,T,4]`` -> ``(loss [T], lse [T])``; ``vocab`` = full vocabulary size (needed
    only with label smoothing)."""
    m = all_stats[..., 0]
    gmax = m.max(dim=0).values
    se = (all_stats[..., 1] * torch.exp(m - gmax[None])).sum(0)
    tgt = all_stats[..., 2].sum(0)
    lse = torch.log(se) + gmax
    loss = lse - tgt
    s = _smoothing(label_smoothing, vocab)
    if s:
        mean_log_p = all_stats[..., 3].sum(0) / vocab - lse
        loss = (1.0 - s) * loss - s * mean_log_p
    return loss, lse


def vocab_parallel_ce_fwd(logits, labels, vocab_start: int = 0, group=None, stream=None, label_smoothing: float = 0.0):
    """Returns ``(loss_per_token [T] fp32, lse [T] fp32)``."""
    stats = ce_local_stats(logits, labels, vocab_start, stream=stream)
    ws = group_size(group)
    if ws > 1:
        T = stats.shape[0]
        flat = torch.empty((ws * T, 4), dtype=stats.dtype, device=stats.device)
        dist.all_gather_into_tensor(flat, stats, group=group)
        gathered = flat.view(ws, T, 4)
    else:
        gathered = stats.unsqueeze(0)
    return ce_combine_stats(gathered, label_smoothing, logits.shape[1] * ws)


def vocab_parallel_ce_bwd_(logits, labels, lse, grad_per_token, vocab_start: int = 0, sm_budget: int = 0, stream=None,
                           label_smoothing: float = 0.0, vocab: int = 0):
    """Overwrites ``logits`` with ``d loss / d logits`` and returns it.  With label smoothing pass
    the full vocabulary size as ``vocab``: the gradient is ``softmax - (1 - s') onehot - s' / V``."""
    T, Vl = logits.shape
    s = _smoothing(label_smoothing, vocab)
    tcoef, ucoef = 1.0 - s, (s / vocab if s else 0.0)
    if not K.use_native(logits):
        p = torch.exp(logits.float() - lse[:, None])
        loc = labels.long() - vocab_start
        own = (loc >= 0) & (loc < Vl)
        rows = torch.nonzero(own).squeeze(1)
        p[rows, loc[rows]] -= tcoef
        if ucoef:
            p -= ucoef
        logits.copy_((p * grad_per_token[:, None]).to(logits.dtype))
        return logits
    fn = K.proto("dh_ce_grad_inplace", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_float,
                                        c_float, c_int, c_void_p])
    K.check(fn(logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), grad_per_token.data_ptr(), T, Vl, logits.stride(0),
               vocab_start, int(logits.dtype == torch.float32), tcoef, ucoef, sm_budget, K.stream_ptr(stream)), "dh_ce_grad_inplace")
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


# ----------------------------------------------------------------------------- reference-style wrappers
def cross_entropy_fwd(inputs: dict, label_smoothing: float = 0.0, group=None, vocab_start: int = None):
    """Dictionary protocol of the reference's ``cross_entropy_fwd`` (dhellam/operators/loss.py:15-98):
    ``inputs = {"vocab_parallel_logits": [..., V/t], "target": [...]}``; returns a context with
    ``loss`` (shape of ``target``) and what the backward needs.  The tensor-parallel group and
    rank come from ``adaptor.parallel_state`` unless given."""
    from ..adaptor import parallel_state as TPS
    logits, target = inputs["vocab_parallel_logits"], inputs["target"]
    if group is None:
        try:
            group = TPS.get_tensor_model_parallel_group()
        except RuntimeError:            # no model-parallel state: a single rank holding the whole vocabulary
            group = None
    Vl = logits.shape[-1]
    if vocab_start is None:
        vocab_start = dist.get_rank(group=group) * Vl if group_size(group) > 1 else 0
    l2 = logits.reshape(-1, Vl)
    loss, lse = vocab_parallel_ce_fwd(l2, target.reshape(-1).to(torch.int32), vocab_start, group, label_smoothing=label_smoothing)
    return {"loss": loss.view(target.shape), "lse": lse, "label_smoothing": label_smoothing, "vocab_size": Vl * group_size(group),
            "logits": logits, "target": target, "vocab_start": vocab_start}


def cross_entropy_bwd(context: dict, dout):
    """``d logits`` for ``dout = d L / d loss`` (shape of ``target``); overwrites the logits buffer
    (dhellam/operators/loss.py:100-127)."""
    logits = context["logits"]
    Vl = logits.shape[-1]
    g = vocab_parallel_ce_bwd_(logits.reshape(-1, Vl), context["target"].reshape(-1).to(torch.int32), context["lse"],
                               dout.reshape(-1).float(), context["vocab_start"], label_smoothing=context["label_smoothing"],
                               vocab=context["vocab_size"])
    return g.view(logits.shape)
