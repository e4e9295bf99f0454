"""Pipeline-parallel neighbour exchange for the folded model.

Each hop of the folded pipeline carries a *pair* of tensors in the same direction, the
forward strand's activation and the backward strand's gradient, each ``(rows/t, h)``
(the reference patches Megatron for this: megatron.patch:207-349,
``send_forward_recv_backward_dhellam`` / ``send_backward_recv_forward_dhellam``).  Here one
``batch_isend_irecv`` per tick moves whatever is valid in both directions on the
communication stream, ordered against the compute streams with events instead of the
reference's 1-element handshake plus device synchronisation (megatron.patch:75-99).
Transport stays on the library's point-to-point calls (NCCL on GPUs, gloo on CPU ranks).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def exchange(ps, send_next: Sequence[Optional[torch.Tensor]], send_prev: Sequence[Optional[torch.Tensor]],
             recv_next: Sequence[bool], recv_prev: Sequence[bool], shape, dtype, device, slots: Sequence[int] = (0, 1)):
    """Posts the sends/receives of one tick boundary for the strands in ``slots`` (0 = forward
    activation, 1 = backward gradient) as ONE group and waits for them (on GPUs the wait only
    orders the current stream).

    ``send_*`` are lists (forward activation, backward gradient) with ``None`` for an
    absent strand; ``recv_*`` say which of the two to expect from that neighbour.
    Returns ``(from_next, from_prev)`` lists with tensors or ``None``.  The engine calls this
    once per strand: the forward strand's tensor leaves as soon as it exists, while the (longer)
    backward strand of the same tick is still computing, and each strand of the next tick waits
    for its own tensor only.
    """
    ops = []
    from_next: List[Optional[torch.Tensor]] = [None, None]
    from_prev: List[Optional[torch.Tensor]] = [None, None]
    nxt, prv = ps.pp_next(), ps.pp_prev()
    # A fixed global order (slot 0 then slot 1; prev-direction then next-direction) keeps
    # the pairing of sends and receives identical on both sides.
    for i in slots:
        if send_prev[i] is not None:
            ops.append(dist.P2POp(dist.isend, send_prev[i].contiguous(), prv, ps.pp_group))
        if recv_next[i]:
            from_next[i] = torch.empty(shape, dtype=dtype, device=device)
            ops.append(dist.P2POp(dist.irecv, from_next[i], nxt, ps.pp_group))
    for i in slots:
        if send_next[i] is not None:
            ops.append(dist.P2POp(dist.isend, send_next[i].contiguous(), nxt, ps.pp_group))
        if recv_prev[i]:
            from_prev[i] = torch.empty(shape, dtype=dtype, device=device)
            ops.append(dist.P2POp(dist.irecv, from_prev[i], prv, ps.pp_group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return from_next, from_prev


def tick_plan(t: int, p: int, P: int, N: int):
    """What stage ``p`` of ``P`` does at tick ``t`` with ``N`` micro-batches.

    Returns ``(down, a, b, fa, fb)``: sweep direction, forward-strand micro-batch ``a``,
    backward-strand micro-batch ``b = a - P`` and whether each is live.  A micro-batch
    enters every second tick; stage ``p`` sweeps down (its first layer chunk forward, its
    second chunk backward) on ticks of parity ``p`` and up on the others, so every stage is
    busy on every tick of the steady state.
    """
    down = (t - p) % 2 == 0
    if down:
        a = (t - p) // 2
    else:
        a = (t - 2 * P + 1 + p) // 2
    b = a - P
    return down, a, b, 0 <= a < N, 0 <= b < N


def total_ticks(P: int, N: int) -> int:
    return 2 * N + 4 * P - 2
