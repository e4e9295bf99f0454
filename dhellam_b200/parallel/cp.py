"""Context parallelism: causal ring attention with the load-balanced two-chunk split.

Each rank holds sequence chunks ``r`` and ``2c-1-r`` of ``2c``.  KV blocks travel
rank -> rank+1; at step ``i`` a rank holds the block of rank ``r-i`` and computes one of
three cases (step 0: causal over the local block; ``i <= r``: all queries against the first
half of the block; ``i > r``: second-half queries against the whole block), then merges
the partial result through the log-sum-exp.  In the backward the block's dKV accumulator
travels with it and needs one more hop to return home, hence ``c`` forward and ``c+1``
backward steps, each a schedulable op (``cp_attn_block_fwd_k`` / ``cp_attn_block_bwd_k``)
so that the pairing search can put the other strand's compute beside each transfer.

Capability parity: dhellam/operators/ring_attn.py:43-411 (``fa_cp_block_fwd/bwd``) and the
unrolled ring ops of dhellam/core/dstb.py:715-722, 806-818, generalised from c = 2 to any c.

Two transports.  The ring above over library point-to-point calls (NCCL / gloo) is the CPU path
and the fall-back.  On GPUs with peer memory (``env.fused_cp``, see ``ops.fused_comm.FusedCP``) the
same schedulable ops run a gather form instead: the first forward op pushes this rank's two K|V
chunks to their global places in every peer's buffer, the last one runs one causal attention call
per query chunk over the keys that chunk may see (chunk ``j`` sees keys ``[0, (j+1) L)``, which is
exactly the kernel's bottom-right aligned causal mask), so there are no per-step partial outputs,
no log-sum-exp merges and no concatenations; the backward re-gathers K|V the same way, writes this
rank's dK|dV contributions for all keys into its symmetric buffer and reduces its own two chunks
over the ranks inside the switch.
"""
from __future__ import annotations

import torch

from ..ops import attention as ATT
from ..ops import comm as C


def _use(run, t):
    s = getattr(run.env, "cur_stream", None)
    if s is not None and t is not None and t.is_cuda:
        t.record_stream(s)
    return t


def _views(run, qkv):
    from ..models.transformer import _qkv_views
    return _qkv_views(run.env, qkv, run.mb.batch)


def _post(run, send, reverse=False):
    ps = run.env.ps
    recv = torch.empty_like(send)
    reqs = C.ring_exchange(send, recv, ps.cp_group, ps.cp_ranks, reverse=reverse)
    return recv, reqs


def _kv_rows(run, qkv):
    """The K|V columns of the packed QKV rows: ``[T, 2 * nkv * d]`` strided view."""
    from ..models.transformer import _heads
    nq, nkv, d = _heads(run.env)
    return qkv[:, nq * d:]


def _kv_heads_view(env, rows, B):
    """``[S * B, 2 * nkv * d]`` gathered rows -> ``(k, v)`` as ``[S, B, nkv, d]`` strided views."""
    from ..models.transformer import _heads
    nq, nkv, d = _heads(env)
    v4 = rows.view(rows.shape[0] // B, B, 2 * nkv, d)
    return v4[:, :, :nkv], v4[:, :, nkv:]


def _gather_fwd_step(run, i: int, c: int):
    from ..models.transformer import _apply_rope
    env = run.env
    cp = env.fused_cp
    st = run.v.setdefault("ring", {})
    if i == 0:
        qkv = _use(run, run.v.pop("qkv"))
        _apply_rope(run, qkv)
        run.acts["qkv"] = qkv
        st["qkv"] = qkv
        st["slot"], st["target"] = cp.push_kv(_kv_rows(run, qkv), "kv_fwd")
    if i < c - 1:
        return
    qkv = st["qkv"]
    B = run.mb.batch
    q, _, _ = _views(run, qkv)
    r, L = cp.rank, q.shape[0] // 2
    a_id, b_id = cp.chunk_ids()
    rows = cp.wait_kv("kv_fwd", st["slot"], st["target"], b_id + 1)
    k, v = _kv_heads_view(env, rows, B)
    o = torch.empty((q.shape[0], B, q.shape[2], q.shape[3]), dtype=q.dtype, device=q.device)
    lses = []
    for half, chunk in ((1, b_id), (0, a_id)):                 # the heavier chunk first
        n = (chunk + 1) * L
        _, lse = ATT.attn_fwd(q[half * L:(half + 1) * L], k[:n], v[:n], causal=True, scale=env.softmax_scale,
                              out=o[half * L:(half + 1) * L])
        lses.append(lse)
    run.acts["attn_out"], run.acts["lse"] = o, (lses[1], lses[0])
    run.v["attn_out"] = o.view(o.shape[0] * o.shape[1], -1)
    run.v.pop("ring")


def _gather_bwd_step(run, i: int, c: int):
    from ..models.transformer import _apply_rope, _heads
    env = run.env
    cp = env.fused_cp
    st = run.v.setdefault("ring_b", {})
    if i == 0:
        qkv = _use(run, run.acts.pop("qkv"))
        st["qkv"] = qkv
        st["slot"], st["target"] = cp.push_kv(_kv_rows(run, qkv), "kv_bwd")      # re-gather instead of keeping 2c chunks per layer
    if i < c:
        return
    qkv = st["qkv"]
    B = run.mb.batch
    nq, nkv, d = _heads(env)
    q, _, _ = _views(run, qkv)
    L = q.shape[0] // 2
    a_id, b_id = cp.chunk_ids()
    rows = cp.wait_kv("kv_bwd", st["slot"], st["target"], b_id + 1)
    k, v = _kv_heads_view(env, rows, B)
    o = _use(run, run.acts["attn_out"])
    lse_a, lse_b = run.acts.pop("lse")
    do = _use(run, run.v.pop("d_attn_out")).view(o.shape)
    dqkv = torch.empty_like(qkv)
    dq, _, _ = _views(run, dqkv)
    part, pslot = cp.dkv_buffer()
    pk, pv = _kv_heads_view(env, part, B)
    nb = (b_id + 1) * L
    # the later chunk sees the longer key range: its dK|dV go straight into the symmetric buffer, rows it cannot see are zero
    ATT.attn_bwd(do[L:], q[L:], k[:nb], v[:nb], o[L:], _use(run, lse_b), causal=True, scale=env.softmax_scale,
                 dq=dq[L:], dk=pk[:nb], dv=pv[:nb])
    if nb * B < part.shape[0]:
        part[nb * B:].zero_()
    na = (a_id + 1) * L
    tmp = torch.empty((na * B, part.shape[1]), dtype=part.dtype, device=part.device)
    tk, tv = _kv_heads_view(env, tmp, B)
    ATT.attn_bwd(do[:L], q[:L], k[:na], v[:na], o[:L], _use(run, lse_a), causal=True, scale=env.softmax_scale,
                 dq=dq[:L], dk=tk, dv=tv)
    part[:na * B] += tmp
    cp.reduce_dkv(pslot, dqkv[:, nq * d:])
    _apply_rope(run, dqkv, inverse=True)
    run.v["d_qkv"] = dqkv
    run.v.pop("ring_b")


def make_ring_fwd_step(i: int, c: int):
    def step(run):
        from ..models.transformer import _apply_rope
        if getattr(run.env, "fused_cp", None) is not None:
            return _gather_fwd_step(run, i, c)
        env, ps = run.env, run.env.ps
        r = ps.cp_rank
        st = run.v.setdefault("ring", {})
        if i == 0:
            qkv = _use(run, run.v.pop("qkv"))
            _apply_rope(run, qkv)
            q, k, v = _views(run, qkv)
            st["q"] = q
            st["kv"] = torch.stack([k, v]).contiguous()          # [2, S, B, Hk, d]
            run.acts["qkv"] = qkv
        else:
            st["reqs"].wait()
            st["kv"] = st.pop("kv_next")
        kv = st["kv"]
        if i < c - 1:
            st["kv_next"], st["reqs"] = _post(run, kv)
        q = st["q"]
        S = q.shape[0]
        half = S // 2
        scale = env.softmax_scale
        if i == 0:
            o, lse = ATT.attn_fwd(q, kv[0], kv[1], causal=True, scale=scale)
            st["o"], st["lse"] = o, lse
        elif i <= r:
            o, lse = ATT.attn_fwd(q, kv[0][:half], kv[1][:half], causal=False, scale=scale)
            st["o"], st["lse"] = ATT.merge_attention_partials(st["o"], st["lse"], o, lse)
        else:
            o, lse = ATT.attn_fwd(q[half:], kv[0], kv[1], causal=False, scale=scale)
            o2, lse2 = ATT.merge_attention_partials(st["o"][half:], st["lse"][:, :, half:], o, lse)
            st["o"] = torch.cat([st["o"][:half], o2], dim=0)
            st["lse"] = torch.cat([st["lse"][:, :, :half], lse2], dim=2)
        if i == c - 1:
            o = st["o"].contiguous()
            run.acts["attn_out"], run.acts["lse"] = o, st["lse"].contiguous()
            run.v["attn_out"] = o.view(o.shape[0] * o.shape[1], -1)
            run.v.pop("ring")
    return step


def make_ring_bwd_step(i: int, c: int):
    def step(run):
        from ..models.transformer import _apply_rope
        if getattr(run.env, "fused_cp", None) is not None:
            return _gather_bwd_step(run, i, c)
        env, ps = run.env, run.env.ps
        r = ps.cp_rank
        st = run.v.setdefault("ring_b", {})
        scale = env.softmax_scale
        if i == 0:
            qkv = _use(run, run.acts.pop("qkv"))
            q, k, v = _views(run, qkv)
            o = _use(run, run.acts["attn_out"])
            st["q"], st["o"], st["lse"] = q, o, _use(run, run.acts.pop("lse"))
            st["do"] = _use(run, run.v.pop("d_attn_out")).view(o.shape)
            st["dq"] = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
            kv = torch.stack([k, v]).contiguous()
            st["pack"] = torch.stack([kv.float(), torch.zeros_like(kv, dtype=torch.float32)])   # [2(kv,dkv), 2, S,B,H,d]
            st["shape"] = qkv.shape
        else:
            st["reqs"].wait()
            st["pack"] = st.pop("pack_next")
        if i == c:
            # the block is home again: its accumulator is this rank's dK, dV
            from ..models.transformer import _heads
            nq, nkv, d = _heads(env)
            dkv = st["pack"][1]
            S, B = st["q"].shape[0], st["q"].shape[1]
            dqkv = torch.empty((S, B, nq + 2 * nkv, d), dtype=run.env.dtype, device=dkv.device)
            dqkv[:, :, :nq] = st["dq"].to(dqkv.dtype)
            dqkv[:, :, nq:nq + nkv] = dkv[0].to(dqkv.dtype)
            dqkv[:, :, nq + nkv:] = dkv[1].to(dqkv.dtype)
            dqkv = dqkv.view(st["shape"])
            _apply_rope(run, dqkv, inverse=True)
            run.v["d_qkv"] = dqkv
            run.v.pop("ring_b")
            return
        pack = st["pack"]
        kv = pack[0].to(run.env.dtype)
        q, o, lse, do = st["q"], st["o"], st["lse"], st["do"]
        S = q.shape[0]
        half = S // 2
        if i == 0:
            dq, dk, dv = ATT.attn_bwd(do, q, kv[0], kv[1], o, lse, causal=True, scale=scale)
            st["dq"] += dq.float()
            pack[1][0] += dk.float()
            pack[1][1] += dv.float()
        elif i <= r:
            dq, dk, dv = ATT.attn_bwd(do, q, kv[0][:half], kv[1][:half], o, lse, causal=False, scale=scale)
            st["dq"] += dq.float()
            pack[1][0][:half] += dk.float()
            pack[1][1][:half] += dv.float()
        else:
            dq, dk, dv = ATT.attn_bwd(do[half:], q[half:], kv[0], kv[1], o[half:], lse[:, :, half:].contiguous(),
                                      causal=False, scale=scale)
            st["dq"][half:] += dq.float()
            pack[1][0] += dk.float()
            pack[1][1] += dv.float()
        st["pack_next"], st["reqs"] = _post(run, pack)
    return step
