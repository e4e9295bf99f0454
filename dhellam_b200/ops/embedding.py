"""Vocabulary-parallel word embedding, forward and backward.

Same contract as the reference's ``word_embedding_fwd`` / ``word_embedding_bwd``
(dhellam/operators/embedding.py:16-49): tokens outside this rank's vocabulary range
contribute zero rows, and the caller sums the partial results over the tensor-parallel
group (a reduce-scatter when the activations are sequence-parallel).  The backward adds
rows of the output gradient into the fp32 ``main_grad`` of the embedding table.
"""
from __future__ import annotations

from ctypes import c_int, c_int64, c_void_p

import torch

from .. import kernels as K


def embedding_fwd(tokens, weight, vocab_start: int = 0, sm_budget: int = 0, stream=None, out=None):
    """``tokens [T]`` integer -> ``[T, h]``; rows of foreign tokens are zero.  ``out`` may name
    the destination (for example a symmetric-memory buffer that a reduce-scatter reads next)."""
    T = tokens.numel()
    Vl, h = weight.shape
    if not K.use_native(weight):
        loc = tokens.reshape(-1).long() - vocab_start
        own = (loc >= 0) & (loc < Vl)
        res = weight[loc.clamp(0, Vl - 1)] * own[:, None].to(weight.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        out = torch.empty((T, h), dtype=weight.dtype, device=weight.device)
    fn = K.proto("dh_embedding_fwd", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    K.check(fn(tokens.data_ptr(), weight.data_ptr(), out.data_ptr(), T, h, Vl, vocab_start, sm_budget,
               K.stream_ptr(stream)), "dh_embedding_fwd")
    return out


def embedding_bwd(dout, tokens, main_grad, vocab_start: int = 0, sm_budget: int = 0, stream=None):
    """``main_grad[token - vocab_start] += dout[row]`` for owned tokens (fp32 accumulate)."""
    T = tokens.numel()
    Vl, h = main_grad.shape
    if not K.use_native(main_grad):
        loc = tokens.reshape(-1).long() - vocab_start
        own = (loc >= 0) & (loc < Vl)
        rows = torch.nonzero(own).squeeze(1)
        main_grad.index_add_(0, loc[rows], dout.reshape(T, h)[rows].to(main_grad.dtype))
        return main_grad
    if K.deterministic():
        # fixed summation order: positions sorted by token id (stable), one CTA per distinct token
        flat = tokens.reshape(-1)
        sorted_tok, order = torch.sort(flat, stable=True)
        sorted_tok = sorted_tok.to(torch.int32).contiguous()
        fn = K.proto("dh_embedding_bwd_sorted", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
        K.check(fn(dout.data_ptr(), order.contiguous().data_ptr(), sorted_tok.data_ptr(), main_grad.data_ptr(), T, h, Vl, vocab_start,
                   sm_budget, K.stream_ptr(stream)), "dh_embedding_bwd_sorted")
        return main_grad
    fn = K.proto("dh_embedding_bwd", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    K.check(fn(dout.data_ptr(), tokens.data_ptr(), main_grad.data_ptr(), T, h, Vl, vocab_start, sm_budget,
               K.stream_ptr(stream)), "dh_embedding_bwd")
    return main_grad


# Names kept for users of the reference package.
word_embedding_fwd = embedding_fwd
word_embedding_bwd = embedding_bwd
