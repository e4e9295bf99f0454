"""Pair profiler: for every candidate (forward group, backward group) measures the time of
running the two groups one after the other on one stream and of running them side by side
(forward ops on stream 1, backward ops on stream 2, collectives on the communication
stream), and appends one line per pair to the profile file in the reference's format
(search/profiler.py:177-180)::

    [[f0, f1, ...],[b0, b1, ...]] speedup: <x> seq_time:<ms> para_time:<ms>

Pairs that would put a collective on both sides are skipped, as in the reference
(search/profiler.py:151-169).  Times are device times (CUDA events), max over the ranks of
the tensor-parallel group; on CPU ranks the host clock is used so the pipeline can be
exercised without a GPU.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..common.benchmark import device_time_ms
from ..common.common import print_rank0
from .harness import LayerHarness
from .op_table import get_candidate_operator_groups, has_collective, operator_list_prune


def _bundle(h: LayerHarness, fwd_ids, bwd_ids, overlapped: bool):
    fbegin, fc, fm = h.replay(fwd_ids)
    bbegin, bc, bm = h.replay(bwd_ids)
    st = h.streams
    cuda = st.cuda

    def run():
        fbegin()
        bbegin()
        if not cuda:
            for f in fm + fc + bm + bc:
                f()
            return
        cur = torch.cuda.current_stream()
        if not overlapped:
            for f in fm + fc + bm + bc:
                f()
            return
        for s in (st.s1, st.s2, st.s3):
            s.wait_stream(cur)
        for lst_m, lst_c, s in ((fm, fc, st.s1), (bm, bc, st.s2)):
            if lst_m:
                with torch.cuda.stream(st.s3):
                    for f in lst_m:
                        f()
                if lst_c:
                    s.wait_stream(st.s3)          # compute of the same strand consumes the collective
        # the strand that does not wait for a collective goes first (dhellam/core/dstb.py:1174-1264)
        order = ((bc, st.s2), (fc, st.s1)) if fm else ((fc, st.s1), (bc, st.s2))
        for lst, s in order:
            with torch.cuda.stream(s):
                for f in lst:
                    f()
        for s in (st.s1, st.s2, st.s3):
            cur.wait_stream(s)
    return run


def measure_pair(h: LayerHarness, fwd_ids: Sequence[int], bwd_ids: Sequence[int], repeat: int = 5, group=None):
    seq = device_time_ms(_bundle(h, fwd_ids, bwd_ids, False), repeat=repeat, warmup=1, group=group)
    if fwd_ids and bwd_ids:
        par = device_time_ms(_bundle(h, fwd_ids, bwd_ids, True), repeat=repeat, warmup=1, group=group)
    else:
        par = seq
    speedup = seq / par if par > 0 else 1.0
    return speedup, seq, par


def run_profiler(h: LayerHarness, out_path: str = "op_profile_num.txt", repeat: int = 5, limit: Optional[int] = None,
                 use_program_skeleton: bool = True):
    """Measures all legal candidate pairs and writes the profile file (rank 0).  Returns the
    number of pairs measured."""
    (_, _, fskel), (_, _, bskel) = operator_list_prune(h.ps.cp, h.program if use_program_skeleton else None)
    fwd_groups, bwd_groups = get_candidate_operator_groups(fskel, bskel)
    rank0 = not dist.is_initialized() or dist.get_rank() == 0
    if rank0 and os.path.exists(out_path):
        os.remove(out_path)
    n = 0
    for f in fwd_groups:
        for b in bwd_groups:
            if not f and not b:
                continue
            if f and b and has_collective(f, h.program) and has_collective(b, h.program):
                continue
            if limit is not None and n >= limit and f and b:
                continue
            speedup, seq, par = measure_pair(h, f, b, repeat, group=h.ps.tp_group)
            n += 1
            if rank0:
                with open(out_path, "a") as fp:
                    fp.write(f"[{list(f)},{list(b)}] speedup: {speedup} seq_time:{seq} para_time:{par}\n")
    print_rank0(f">>>> profiled {n} operator-group pairs -> {out_path}")
    return n
