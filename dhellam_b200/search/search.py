"""Pairing solver: chooses how to cut each strand's skeleton into groups and how to align
the two group sequences so that the summed measured time is minimal.

Same search space and cost model as the reference (search/search.py:77-158): a schedule is
a monotone path through (forward groups) x (backward groups); a step runs a forward group
alone, a backward group alone, or a pair side by side (forbidden when both contain a
collective, :13-21); the cost of a step is its measured ``para_time``.  The reference
enumerates every way of splitting the skeleton into m and n groups and runs an alignment
DP for each; here one DP over *op positions* covers all splits at once,

    T[i][j] = min over legal groups f = fwd[i':i], b = bwd[j':j] of
              T[i'][j] + t(f),  T[i][j'] + t(b),  T[i'][j'] + t(f || b)

where a legal group is a contiguous run inside one skeleton group, so the result is the
optimum of the reference's enumeration at polynomial cost (which also makes skeletons with
many ring steps or expert ops tractable).
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Sequence, Tuple

from ..sched.optable import OP_TABLE_NAME
from ..sched.strategy import Block, Strategy
from .op_table import FUSED_ENTRIES, has_collective, operator_list_prune

_LINE = re.compile(r"\[\s*\[\s*((?:\d+(?:,\s*\d+)*)?)\s*\],\s*\[\s*((?:\d+(?:,\s*\d+)*)?)\s*\]\]\s*speedup:\s*([0-9.eE+-]+)\s*"
                   r"seq_time:\s*([0-9.eE+-]+)\s*para_time:\s*([0-9.eE+-]+)")


def _key(f: Sequence[int], b: Sequence[int]) -> str:
    return f"{list(f)}|{list(b)}"


def parse_op_file(path: str) -> Dict[str, float]:
    """Profile file -> ``{"[f ids]|[b ids]": para_time}``."""
    table = {}
    with open(path) as fp:
        for line in fp:
            m = _LINE.match(line.strip())
            if not m:
                continue
            f = [int(x) for x in m.group(1).split(",") if x.strip()]
            b = [int(x) for x in m.group(2).split(",") if x.strip()]
            table[_key(f, b)] = float(m.group(5))
    return table


def illegal_pair(f: Sequence[int], b: Sequence[int]) -> bool:
    return bool(f) and bool(b) and has_collective(f) and has_collective(b)


def _runs(skeleton: List[List[int]]):
    """For every end position i (1-based over the flattened strand) the legal start
    positions i' of a group ending at i."""
    flat, starts = [], {}
    for g in skeleton:
        base = len(flat)
        for k in range(len(g)):
            starts[base + k + 1] = list(range(base, base + k + 1))
        flat.extend(g)
    return flat, starts


def solve(table: Dict[str, float], fwd_skeleton: List[List[int]], bwd_skeleton: List[List[int]]):
    """Returns ``(total time, [(fwd ids, bwd ids), ...])``."""
    F, fstarts = _runs(fwd_skeleton)
    B, bstarts = _runs(bwd_skeleton)
    INF = float("inf")
    nf, nb = len(F), len(B)
    T = [[INF] * (nb + 1) for _ in range(nf + 1)]
    back: List[List[Optional[tuple]]] = [[None] * (nb + 1) for _ in range(nf + 1)]
    T[0][0] = 0.0

    def cost(f, b):
        return table.get(_key(f, b), INF)

    for i in range(nf + 1):
        for j in range(nb + 1):
            if i == 0 and j == 0:
                continue
            best, arg = INF, None
            if i > 0:
                for ip in fstarts[i]:
                    c = T[ip][j] + cost(F[ip:i], [])
                    if c < best:
                        best, arg = c, (ip, j)
            if j > 0:
                for jp in bstarts[j]:
                    c = T[i][jp] + cost([], B[jp:j])
                    if c < best:
                        best, arg = c, (i, jp)
            if i > 0 and j > 0:
                for ip in fstarts[i]:
                    for jp in bstarts[j]:
                        f, b = F[ip:i], B[jp:j]
                        if illegal_pair(f, b):
                            continue
                        c = T[ip][jp] + cost(f, b)
                        if c < best:
                            best, arg = c, (ip, jp)
            T[i][j], back[i][j] = best, arg
    if T[nf][nb] == INF:
        raise ValueError("the profile table does not cover the skeleton (missing single-strand entries?)")
    steps = []
    i, j = nf, nb
    while (i, j) != (0, 0):
        ip, jp = back[i][j]
        steps.append((F[ip:i], B[jp:j]))
        i, j = ip, jp
    steps.reverse()
    return T[nf][nb], steps


def brute_force(table, fwd_skeleton, bwd_skeleton):
    """Exhaustive reference for tests: enumerates every split and every alignment."""
    def splits(skel):
        out = [[]]
        for g in skel:
            ways = []
            n = len(g)
            for mask in range(1 << (n - 1)):
                parts, cur = [], [g[0]]
                for k in range(1, n):
                    if mask >> (k - 1) & 1:
                        parts.append(cur)
                        cur = []
                    cur.append(g[k])
                parts.append(cur)
                ways.append(parts)
            out = [o + w for o in out for w in ways]
        return out
    INF = float("inf")
    best = INF
    for fs in splits(fwd_skeleton):
        for bs in splits(bwd_skeleton):
            m, n = len(fs), len(bs)
            T = [[INF] * (n + 1) for _ in range(m + 1)]
            T[0][0] = 0.0
            for i in range(m + 1):
                for j in range(n + 1):
                    if i == 0 and j == 0:
                        continue
                    c = INF
                    if i > 0:
                        c = min(c, T[i - 1][j] + table.get(_key(fs[i - 1], []), INF))
                    if j > 0:
                        c = min(c, T[i][j - 1] + table.get(_key([], bs[j - 1]), INF))
                    if i > 0 and j > 0 and not illegal_pair(fs[i - 1], bs[j - 1]):
                        c = min(c, T[i - 1][j - 1] + table.get(_key(fs[i - 1], bs[j - 1]), INF))
                    T[i][j] = c
            best = min(best, T[m][n])
    return best


def steps_to_strategy(steps, program=None) -> Strategy:
    """Blocks in the strategy-file form: compute ops on S1 / S2, collectives on S3.  With the
    layer program at hand an op's kind decides its lane; without it, names do."""
    def is_comm(n):
        if program is not None and program.has(n):
            return program.op(n).kind == "comm"
        return "allgather" in n or "reduce_scatter" in n or n.startswith(("dispatch", "combine"))

    def lanes(ids):
        comp, comm = [], []
        for i in ids:
            for n in (FUSED_ENTRIES[i] if i in FUSED_ENTRIES else (OP_TABLE_NAME[i],)):
                (comm if is_comm(n) else comp).append(n)
        return comp, comm
    blocks = []
    for f, b in steps:
        fc, fm = lanes(f)
        bc, bm = lanes(b)
        blocks.append(Block(s1=fc, s2=bc, s3=fm + bm))
    return Strategy(dcblocks=blocks)


def run_search(profile_path: str, cp: int = 1, program=None, out_dir: str = "config") -> Tuple[float, str]:
    """Profile file -> ``<out_dir>/dhellam-cp{cp}/best_result.json`` (search/search.py:240-244)."""
    (_, _, fskel), (_, _, bskel) = operator_list_prune(cp, program)
    table = parse_op_file(profile_path)
    total, steps = solve(table, fskel, bskel)
    strat = steps_to_strategy(steps, program)
    d = os.path.join(out_dir, f"dhellam-cp{cp}")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, "best_result.json")
    with open(path, "w") as fp:
        json.dump(strat.to_dict(), fp, indent=4)
    return total, path
