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


def get_distributed_world_size(group=None) -> int:
    """Name kept from the reference (dhellam/operators/comm.py:7-11)."""
    return group_size(group)


# --------------------------------------------------------------------------- host-level chunked overlap
# The reference carries two prototypes that overlap a TP collective with its GEMM from the
# host, chunk by chunk (dhellam/operators/comm.py:89-143).  The kernels of
# ``ops/fused_comm.py`` do the same thing inside one launch; these functions keep the
# prototypes' contracts on any backend (they are also the only overlapped form on CPU ranks).
def chunk_allgather_gemm(gemm_weight, comm_input, tp_size: int, tp_rank: int, tp_group, tp_ranks=None):
    """``all_gather(comm_input) @ gemm_weight.T`` with the gather done as ``tp_size - 1`` ring
    steps; the GEMM on the shard that has already arrived runs while the next shard is in
    flight.  ``comm_input [m, k]``, ``gemm_weight [n, k]``.  Returns ``(out [m * tp, n],
    gathered [m * tp, k])``, rows in rank order."""
    from .gemm import gemm_nt
    if tp_size == 1:
        return gemm_nt(comm_input, gemm_weight), comm_input
    m = comm_input.shape[0]
    ranks = tp_ranks if tp_ranks is not None else dist.get_process_group_ranks(tp_group)
    gathered = torch.empty((m * tp_size,) + tuple(comm_input.shape[1:]), dtype=comm_input.dtype, device=comm_input.device)
    out = torch.empty((m * tp_size, gemm_weight.shape[0]), dtype=comm_input.dtype, device=comm_input.device)
    gathered[tp_rank * m:(tp_rank + 1) * m].copy_(comm_input)
    have = tp_rank                                  # index of the shard this rank holds and forwards
    for step in range(tp_size):
        cur = gathered[have * m:(have + 1) * m]
        reqs = None
        if step + 1 < tp_size:
            nxt = (have - 1) % tp_size              # the previous rank forwards the shard it held one step ago
            reqs = ring_exchange(cur, gathered[nxt * m:(nxt + 1) * m], tp_group, ranks)
        gemm_nt(cur, gemm_weight, out=out[have * m:(have + 1) * m])
        if reqs is not None:
            reqs.wait()
            have = nxt
    return out, gathered


def chunk_gemm_reduce_scatter(gemm_input, gemm_weight, tp_size: int, tp_rank: int, tp_group, chunks: int = 4):
    """``reduce_scatter(gemm_input @ gemm_weight.T)`` along the rows, computed in ``chunks``
    blocks of output columns: the reduce-scatter of one block runs (asynchronously) while the
    GEMM of the next block computes.  ``gemm_input [M, k]``, ``gemm_weight [n, k]``.  Returns
    this rank's ``[M / tp, n]`` rows of the sum."""
    from .gemm import gemm_nt
    if tp_size == 1:
        return gemm_nt(gemm_input, gemm_weight)
    M, n = gemm_input.shape[0], gemm_weight.shape[0]
    chunks = max(1, min(chunks, n // 8))
    bounds = [(n * i // chunks) // 8 * 8 for i in range(chunks)] + [n]
    parts, handles = [], ReqList()
    for i in range(chunks):
        lo, hi = bounds[i], bounds[i + 1]
        if hi <= lo:
            continue
        partial = gemm_nt(gemm_input, gemm_weight[lo:hi])
        shard = torch.empty((M // tp_size, hi - lo), dtype=partial.dtype, device=partial.device)
        handles.append(dist.reduce_scatter_tensor(shard, partial, group=tp_group, async_op=True))
        parts.append(shard)
    handles.wait()
    return torch.cat(parts, dim=1)


def flash_attn_p2p_communicate(rank, send_tensor, send_dst, recv_tensor, recv_src, cp_group, batch_p2p_comm: bool = True):
    """One ring-attention exchange with the reference's signature
    (dhellam/operators/comm.py:144-205): even ranks post the send first, odd ranks the receive
    first; returns the list of requests to wait on."""
    ops = [dist.P2POp(dist.isend, send_tensor, send_dst, cp_group), dist.P2POp(dist.irecv, recv_tensor, recv_src, cp_group)]
    if rank % 2 == 1:
        ops.reverse()
    if batch_p2p_comm:
        return ReqList(dist.batch_isend_irecv(ops))
    return ReqList([op.op(op.tensor, op.peer, group=op.group) for op in ops])
