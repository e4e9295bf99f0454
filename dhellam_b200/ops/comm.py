"""Library collectives (NCCL on GPUs, gloo on CPU ranks) along the first dimension.

These are the baseline transport for tensor/sequence parallelism and the oracle for the
fused kernels in ``ops/fused_comm.py``.  Same contracts as the reference's
``gather_along_first_dim`` / ``reduce_scatter_along_first_dim`` / ``split_along_first_dim``
(dhellam/operators/comm.py:13-80): each returns ``(tensor, handle)`` where ``handle`` is a
work object to ``wait()`` on when ``async_op`` is set, else ``None``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def group_size(group) -> int:
    """Size of ``group``.  In this framework ``None`` means "no group" (a parallel axis of
    size one), never the world group; pass ``dist.group.WORLD`` for that."""
    if group is None:
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None:
        return 0
    return dist.get_rank(group)


def gather_along_first_dim(x, group=None, async_op: bool = False, out=None):
    ws = group_size(group)
    if ws == 1:
        return x, None
    shape = (x.shape[0] * ws,) + tuple(x.shape[1:])
    if out is None:
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    h = dist.all_gather_into_tensor(out, x.contiguous(), group=group, async_op=async_op)
    return out, (h if async_op else None)


def reduce_scatter_along_first_dim(x, group=None, async_op: bool = False, out=None):
    ws = group_size(group)
    if ws == 1:
        return x, None
    assert x.shape[0] % ws == 0, "first dimension must divide by the group size"
    shape = (x.shape[0] // ws,) + tuple(x.shape[1:])
    if out is None:
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    h = dist.reduce_scatter_tensor(out, x.contiguous(), group=group, async_op=async_op)
    return out, (h if async_op else None)


def split_along_first_dim(x, group=None):
    ws = group_size(group)
    if ws == 1:
        return x
    n = x.shape[0] // ws
    r = group_rank(group)
    return x[r * n:(r + 1) * n].contiguous()


def all_reduce(x, group=None, op=None, async_op: bool = False):
    if group_size(group) == 1:
        return x, None
    h = dist.all_reduce(x, op=op or dist.ReduceOp.SUM, group=group, async_op=async_op)
    return x, (h if async_op else None)


def all_to_all_rows(x, send_counts, recv_counts, group=None):
    """Variable-size row exchange (expert-parallel dispatch/combine baseline)."""
    ws = group_size(group)
    if ws == 1:
        return x
    out = torch.empty((int(sum(recv_counts)),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x.contiguous(), output_split_sizes=[int(c) for c in recv_counts],
                           input_split_sizes=[int(c) for c in send_counts], group=group)
    return out


class ReqList(list):
    """List of p2p requests with a collective ``wait`` (dhellam/operators/comm.py:82-87)."""

    def wait(self):
        for r in self:
            r.wait()


def ring_exchange(send, recv, group, global_ranks, reverse: bool = False):
    """Posts send→next / recv←prev on the ring (or the reverse direction) and returns the
    request list.  Even ranks post the send first and odd ranks the receive first, as in
    the reference's ``flash_attn_p2p_communicate`` (dhellam/operators/comm.py:144-205)."""
    ws = len(global_ranks)
    me = dist.get_rank(group)
    nxt = global_ranks[(me + 1) % ws]
    prv = global_ranks[(me - 1) % ws]
    dst, src = (prv, nxt) if reverse else (nxt, prv)
    ops = [dist.P2POp(dist.isend, send, dst, group), dist.P2POp(dist.irecv, recv, src, group)]
    if me % 2 == 1:
        ops.reverse()
    return ReqList(dist.batch_isend_irecv(ops))
