"""Head block: embedding at the bottom of the model and final norm -> LM head -> loss at
the top, both living on the first pipeline stage of the folded model.

Capability parity with the reference's ``DSHB`` (dhellam/core/dshb.py:98-242): embedding
forward of micro-batch k runs beside the loss-head backward of micro-batch k-1, and the
loss-head forward of k beside the embedding backward of k-1; the LM-head weight is tied to
the word embedding (dshb.py:256-262).  Unlike the reference, which differentiates the head
through autograd (``template_bwd_new``), every piece has an explicit backward that
accumulates into ``main_grad``, and the loss uses one fused statistics exchange instead of
three all-reduces.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import comm as C
from ..ops import embedding as E
from ..ops import gemm as G
from ..ops import loss as L
from ..ops import norm as N
from .transformer import _norm_bwd, _norm_fwd


class HeadParams:
    """``word_embeddings [V/t, h]``, optional ``output_weight [V/t, h]`` (untied), final norm."""

    def __init__(self, tensors: dict):
        self.__dict__.update(tensors)
        self._names = list(tensors.keys())

    def named(self):
        return [(n, getattr(self, n)) for n in self._names]

    def get(self, name, default=None):
        return self.__dict__.get(name, default)

    @property
    def lm_weight(self):
        return self.get("output_weight") if self.get("output_weight") is not None else self.word_embeddings


def _use(env, t):
    s = getattr(env, "cur_stream", None)
    if s is not None and t is not None and t.is_cuda:
        t.record_stream(s)
    return t


def _span(env):
    """Timing bracket for a collective that the current (compute) stream has to sit through."""
    t = getattr(env, "exposed", None)
    if t is None or not t.enabled:
        import contextlib
        return contextlib.nullcontext()
    return t.span(getattr(env, "cur_stream", None))


def _symmetric(env, rows_full: int, width: int) -> bool:
    """True when the head block's collective of this shape can use the symmetric-memory kernels
    (same row count and width as the layers' collectives)."""
    return bool(getattr(env, "fused_tp", False)) and rows_full == env.fused.rows and width == env.fused.width


def tp_gather_rows(env, shard, tag: str):
    """Sequence all-gather of ``shard [T/t, h]`` inside the tensor-parallel group: multimem / peer
    push + arrival counters when the symmetric buffers fit the shape, else the library collective."""
    if env.ps.tp <= 1:
        return shard
    with _span(env):
        if _symmetric(env, shard.shape[0] * env.ps.tp, shard.shape[1]) and shard.dtype == torch.bfloat16:
            return env.fused.all_gather(shard.contiguous(), tag)
        full, _ = C.gather_along_first_dim(shard, env.ps.tp_group)
        return full


def vocab_range(env):
    vl = env.cfg.vocab_size // env.ps.tp
    return env.ps.tp_rank * vl, vl


def embed_fwd(env, hp: HeadParams, mb):
    """tokens -> hidden ``[T/t, h]`` (sequence-parallel rows)."""
    v0, _ = vocab_range(env)
    T, h = mb.tokens.numel(), hp.word_embeddings.shape[1]
    if env.ps.tp > 1 and _symmetric(env, T, h) and hp.word_embeddings.dtype == torch.bfloat16:
        # partial rows straight into symmetric memory, summed inside the switch (no library collective)
        E.embedding_fwd(mb.tokens, hp.word_embeddings, v0, out=env.fused.partial_buffer("embed", T, h))
        with _span(env):
            x = env.fused.rs_reduce("embed")
    else:
        partial = E.embedding_fwd(mb.tokens, hp.word_embeddings, v0)
        if env.ps.tp > 1:
            with _span(env):
                x, _ = C.reduce_scatter_along_first_dim(partial, env.ps.tp_group)
        else:
            x = partial
    if env.cfg.position == "learned":
        pos = hp.position_embeddings[mb.positions_local.long()]
        x = x + pos
    return x


def embed_bwd(env, hp: HeadParams, mb, dx):
    v0, _ = vocab_range(env)
    dx = _use(env, dx)
    if env.cfg.position == "learned":
        hp.position_embeddings.main_grad.index_add_(0, mb.positions_local.long(), dx.float())
    full = tp_gather_rows(env, dx, "embed_bwd")
    E.embedding_bwd(full, mb.tokens, hp.word_embeddings.main_grad, v0)


def loss_fwd(env, hp: HeadParams, mb, x):
    """final norm -> gather -> logits -> vocab-parallel CE -> masked mean.
    Returns ``(loss scalar tensor, saved)``."""
    x = _use(env, x)
    y, stat = _norm_fwd(env, x, hp.final_ln_weight, hp.get("final_ln_bias"), 0)
    y_full = tp_gather_rows(env, y, "head")        # a staging-buffer view: valid until the second next head gather
    logits = G.gemm_nt(y_full, hp.lm_weight)
    v0, _ = vocab_range(env)
    loss_tok, lse = L.vocab_parallel_ce_fwd(logits, mb.labels, v0, env.ps.tp_group, label_smoothing=env.train.label_smoothing)
    mask = mb.loss_mask.reshape(-1).float()
    sums = torch.stack([(loss_tok * mask).sum(), mask.sum()])
    if env.ps.cp > 1:
        dist.all_reduce(sums, group=env.ps.cp_group)
    loss = sums[0] / sums[1].clamp_min(1.0)
    saved = dict(x=x, stat=stat, y_full=y_full, logits=logits, lse=lse, count=sums[1])
    return loss, saved


def loss_bwd(env, hp: HeadParams, mb, saved, grad_scale: float):
    """Returns ``dx [T/t, h]``; accumulates the LM-head and final-norm gradients."""
    v0, _ = vocab_range(env)
    g_tok = L.mask_scale_loss_bwd(mb.loss_mask, saved["count"], grad_scale)
    logits = _use(env, saved.pop("logits"))
    dlogits = L.vocab_parallel_ce_bwd_(logits, mb.labels, _use(env, saved.pop("lse")), g_tok, v0,
                                       label_smoothing=env.train.label_smoothing, vocab=env.cfg.vocab_size)
    if dlogits.dtype != hp.lm_weight.dtype:
        dlogits = dlogits.to(hp.lm_weight.dtype)
    y_full = _use(env, saved.pop("y_full"))
    T, h = dlogits.shape[0], hp.lm_weight.shape[1]
    if env.ps.tp > 1 and _symmetric(env, T, h) and dlogits.dtype == torch.bfloat16:
        G.gemm_nn(dlogits, hp.lm_weight, out=env.fused.partial_buffer("head_bwd", T, h))
        G.gemm_tn_acc(dlogits, y_full, hp.lm_weight.main_grad)      # runs while the peers finish their partial products
        with _span(env):
            d_y = env.fused.rs_reduce("head_bwd")
    else:
        d_y_full = G.gemm_nn(dlogits, hp.lm_weight)
        G.gemm_tn_acc(dlogits, y_full, hp.lm_weight.main_grad)
        if env.ps.tp > 1:
            with _span(env):
                d_y, _ = C.reduce_scatter_along_first_dim(d_y_full, env.ps.tp_group)
        else:
            d_y = d_y_full
    dx = _norm_bwd(env, d_y, _use(env, saved.pop("x")), hp.final_ln_weight, hp.get("final_ln_bias"), saved.pop("stat"), None, 0)
    return dx
