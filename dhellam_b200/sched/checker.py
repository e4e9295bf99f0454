"""Happens-before checker for dual-strand schedules.

The engine orders work on three streams with events instead of device-wide
synchronisation, so a wrong wait is a silent race.  ``check_schedule`` replays a strategy
on the host exactly as the executor would launch it and verifies, for the launch order and
the event waits the executor really issues, that

* every op is ordered after each op it depends on (same stream earlier, or an event wait
  that reaches the producer), and
* every op that reads a value is ordered after the op that produced it when the producer
  ran on another stream (the dependency lists of the layer program are the source of
  truth for who reads what).

``check_trace`` does the same on an explicit list of launches, which is how the tests feed
it hand-made racy schedules.  The reference has nothing comparable: it synchronises the
device after every block (dhellam/core/dstb.py:1266).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Tuple

from .ir import LayerProgram
from .strategy import CARRIED, CARRY_SUFFIX, Block, Strategy, split_budget


class RaceError(AssertionError):
    pass


@dataclass
class Launch:
    op: str
    stream: str                       # "S1" | "S2" | "S3"
    waits: Tuple[str, ...] = ()       # ops whose completion event this launch waits on
    reads: Tuple[str, ...] = ()       # ops whose outputs this launch reads


def _ancestors(launches: Sequence[Launch]) -> List[Set[int]]:
    """For every launch the set of launch indices that happen before it: everything earlier
    on its stream, everything an awaited event covers, transitively."""
    last_on: Dict[str, int] = {}
    idx_of: Dict[str, int] = {}
    before: List[Set[int]] = []
    for i, l in enumerate(launches):
        s: Set[int] = set()
        if l.stream in last_on:
            j = last_on[l.stream]
            s |= before[j] | {j}
        for w in l.waits:
            if w not in idx_of:
                raise RaceError(f"{l.op} waits on {w}, which has not been launched")
            j = idx_of[w]
            s |= before[j] | {j}
        before.append(s)
        last_on[l.stream] = i
        idx_of[l.op] = i
    return before


def check_trace(launches: Sequence[Launch]):
    """Raises ``RaceError`` if some launch reads an op's output without being ordered after it."""
    before = _ancestors(launches)
    idx_of = {l.op: i for i, l in enumerate(launches)}
    for i, l in enumerate(launches):
        for r in l.reads:
            if r not in idx_of:
                raise RaceError(f"{l.op} reads {r}, which is never launched")
            if idx_of[r] >= i or idx_of[r] not in before[i]:
                raise RaceError(f"{l.op} on {l.stream} reads the output of {r} without a happens-before edge")
    return True


def launches_of(program: LayerProgram, blocks: Sequence[Block], compute_streams: int = 2) -> List[Launch]:
    """The launch list the executor produces for ``blocks`` (see ``Executor.run``)."""
    markers = program.marker_targets()
    listed = {split_budget(e)[0] for b in blocks for e in b.all_entries()}
    deferred = {markers[m] for m in listed if m in markers}
    pending: Dict[str, str] = {}
    carried: List[tuple] = []
    out: List[Launch] = []
    stream_of: Dict[str, str] = {}

    def lane_stream(lane):
        return "S1" if (lane == "S2" and compute_streams < 2) else lane

    def emit(name, lane):
        op = program.op(name)
        st = lane_stream(lane)
        waits = tuple(d for d in op.deps if stream_of.get(d) not in (None, st))
        out.append(Launch(name, st, waits, tuple(op.deps)))
        stream_of[name] = st

    for blk in blocks:
        for e in blk.s3:
            emit(split_budget(e)[0], "S3")
        fwd_comm = any(program.has(split_budget(e)[0]) and program.op(split_budget(e)[0]).strand == "fwd" for e in blk.s3)
        order = (("S2", blk.s2), ("S1", blk.s1)) if fwd_comm else (("S1", blk.s1), ("S2", blk.s2))
        for lane, lst in order:
            for e in lst:
                name = split_budget(e)[0]
                if name == CARRIED:
                    continue                      # ops of the previous layer run: checked where that run hands them over
                if name.endswith(CARRY_SUFFIX) and name[:-len(CARRY_SUFFIX)] in markers.values():
                    carried.append((name[:-len(CARRY_SUFFIX)], lane))
                    continue
                if name in markers:
                    if markers[name] in pending:
                        pending.pop(markers[name])
                        emit(markers[name], lane)
                    continue
                if name in deferred:
                    pending[name] = lane
                    continue
                emit(name, lane)
    for name in list(pending):
        emit(name, "S2")
    for name, lane in carried:                    # the next layer run (or the flush) launches them after everything here
        emit(name, lane)
    return out


def check_schedule(program: LayerProgram, strategy: Strategy, compute_streams: int = 2):
    """Validates the strategy and proves its launch order race-free for the paired and the
    two single-strand schedules."""
    strat = strategy.completed(program)
    strat.validate(program)
    for blocks in (strat.dcblocks, strat.fwd_only, strat.bwd_only):
        check_trace(launches_of(program, blocks, compute_streams))
    return True
