"""Op table of the strategy search: ids, the legal grouping skeleton of each strand, and the
candidate groups the profiler measures.

Ids and the cp = 1 / cp = 2 skeletons are the reference's (search/op_table.py:1-92); other
configurations (more ring steps, GeLU MLP, expert MLP) get a skeleton derived from the
layer program: a group never crosses a collective, and a column-parallel weight gradient
stays with the reduce-scatter it overlaps (the reference's fused entries 8 and 9).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from ..sched.ir import BWD, COMM, FWD, LayerProgram
from ..sched.optable import OP_TABLE_IDX, OP_TABLE_NAME

# entries of the table that stand for a compute op plus the collective launched beside it
FUSED_ENTRIES = {
    8: ("gemm_wgrad_attn_c", "reduce_scatter_attn_c_bwd"),
    9: ("gemm_wgrad_mlp_c", "reduce_scatter_mlp_c_bwd"),
}
_FUSED_BY_COMPUTE = {v[0]: k for k, v in FUSED_ENTRIES.items()}


def expand(op_id: int) -> Tuple[str, ...]:
    """Program op names behind a table id."""
    if op_id in FUSED_ENTRIES:
        return FUSED_ENTRIES[op_id]
    return (OP_TABLE_NAME[op_id],)


def skeleton_from_program(program: LayerProgram):
    """``(fwd groups, bwd groups)`` of table ids for any layer program."""
    out = []
    for strand in (FWD, BWD):
        ops = list((program.fwd if strand == FWD else program.bwd).values())
        groups, cur, skip = [], [], set()
        for i, o in enumerate(ops):
            if o.name in skip:
                continue
            if o.name in _FUSED_BY_COMPUTE:
                comm = FUSED_ENTRIES[_FUSED_BY_COMPUTE[o.name]][1]
                if program.has(comm):
                    if cur:
                        groups.append(cur)
                        cur = []
                    groups.append([_FUSED_BY_COMPUTE[o.name]])
                    skip.add(comm)
                    continue
            if o.kind == COMM:
                if cur:
                    groups.append(cur)
                    cur = []
                groups.append([OP_TABLE_IDX[o.name]])
            else:
                cur.append(OP_TABLE_IDX[o.name])
        if cur:
            groups.append(cur)
        out.append(groups)
    return out[0], out[1]


def operator_list_prune(context_parallel_size: int = 1, program: LayerProgram = None):
    """``((min groups, op count, fwd skeleton), (min groups, op count, bwd skeleton))``."""
    if program is not None:
        fwd, bwd = skeleton_from_program(program)
    elif context_parallel_size == 1:
        fwd = [[24], [0], [16, 11, 17], [4], [12, 25], [2], [20, 29, 21], [5], [13]]
        bwd = [[15], [3], [19, 23, 28, 7], [9], [27, 14], [1], [18, 22, 10, 6], [8], [26]]
    elif context_parallel_size == 2:
        fwd = [[24], [0, 16], [30], [31, 17], [4, 12, 25], [2, 20, 29, 21], [5, 13]]
        bwd = [[15], [3, 19, 23, 28, 7], [9], [27, 14], [1, 18, 22], [32], [33], [34, 6], [8], [26]]
    else:
        raise ValueError("pass the layer program for context-parallel sizes other than 1 and 2")
    return (len(fwd), sum(len(g) for g in fwd), fwd), (len(bwd), sum(len(g) for g in bwd), bwd)


def get_candidate_operator_groups(fwd_skeleton, bwd_skeleton):
    """All contiguous sub-runs of every skeleton group plus the empty group
    (search/op_table.py:405-420)."""
    def runs(skel):
        out = [[]]
        for g in skel:
            for i in range(len(g)):
                for j in range(i + 1, len(g) + 1):
                    out.append(g[i:j])
        return out
    return runs(fwd_skeleton), runs(bwd_skeleton)


def has_collective(ids, program: LayerProgram = None) -> bool:
    for i in ids:
        for n in expand(i):
            if "allgather" in n or "reduce_scatter" in n or n.startswith(("dispatch", "combine")):
                return True
            if program is not None and program.has(n) and program.op(n).kind == COMM:
                return True
    return False
