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


# ------------------------------------------------------------------------------------------
# Reuse of the double-buffered symmetric-memory slots (write-after-read across ranks)
# ------------------------------------------------------------------------------------------
# The tensor-parallel collectives stage data in per-site buffers with two slots, used in turn.
# Use k+2 of a site overwrites the slot of use k.  The writer can be ANOTHER rank (an all-gather
# push stores into every peer's staging slot) or the reader can be (a reduce-scatter reads every
# peer's partial product), so stream order on one rank proves nothing.  What does order two
# ranks is a collective: rank R finishes collective X only after every rank Q has contributed
# to X, and Q contributes after everything that precedes the contribution in Q's own streams.
# Every rank issues the same launches in the same order, so "the last reader of use k on Q
# happens before Q's contribution to X, and X's completion on R happens before R's writer of
# use k+2" can be decided on ONE launch list: the reader must reach the writer through a path
# that crosses some collective X strictly between them.  ``check_buffer_reuse`` replays several
# consecutive layer runs (so that carried weight-gradient GEMMs are checked in the run that
# executes them) and verifies this for every site.
#
# ``effects`` maps an op name to a list of ``(action, site)`` with action in
#   "push"       all-gather push into every rank's staging slot of ``site``  (contribution)
#   "wait_read"  waits for the arrival counters of ``site``, then reads the slot (completion + reader)
#   "read"       reads the staged slot of ``site`` (no wait of its own)
#   "write"      local GEMM writes this rank's partial product of ``site``
#   "reduce"     announces + waits for all announcements of ``site`` + reads all ranks' partials
#                (contribution, completion and reader at once)
#   "push_s3"    like "push" but issued from inside a compute op onto the communication stream
#                (ordered after what preceded the op on its own stream, not after the op)

def launches_of_runs(program: LayerProgram, strat: Strategy, kinds: Sequence[str], compute_streams: int = 1,
                     effects: Optional[Dict[str, list]] = None):
    """Launch list of consecutive layer runs (``kinds``: "fwd" | "pair" | "bwd"), op names made
    unique as ``name#run``; returns ``(launches, notes)`` where ``notes[i]`` is the list of
    ``(action, site)`` of launch ``i``."""
    effects = effects or {}
    markers = program.marker_targets()
    out: List[Launch] = []
    notes: List[list] = []
    stream_of: Dict[str, str] = {}
    last_on: Dict[str, str] = {}
    carried: List[tuple] = []          # (op name, run it belongs to, lane, waits)

    def lane_stream(lane):
        return "S1" if (lane == "S2" and compute_streams < 2) else lane

    def emit(name, run, lane, waits=None):
        op = program.op(name)
        st = lane_stream(lane)
        uid = f"{name}#{run}"
        if waits is None:
            waits = tuple(f"{d}#{run}" for d in op.deps if stream_of.get(f"{d}#{run}") not in (None, st))
        eff = list(effects.get(name, ()))
        s3_pushes = [(a, s) for a, s in eff if a == "push_s3"]
        if s3_pushes:
            prev = last_on.get(st)
            out.append(Launch(f"{name}.push#{run}", "S3", (prev,) if prev is not None and stream_of.get(prev) != "S3" else (), ()))
            notes.append([("push", s) for _, s in s3_pushes])
            stream_of[out[-1].op] = "S3"
            last_on["S3"] = out[-1].op
        out.append(Launch(uid, st, tuple(waits), tuple(f"{d}#{run}" for d in op.deps)))
        notes.append([(a, s) for a, s in eff if a != "push_s3"])
        stream_of[uid] = st
        last_on[st] = uid

    def flush(lane=None):
        nonlocal carried
        todo, carried = carried, []
        for name, run, own_lane, waits in todo:
            emit(name, run, lane or own_lane, waits)

    for r, kind in enumerate(kinds):
        blocks = {"pair": strat.dcblocks, "fwd": strat.fwd_only, "bwd": strat.bwd_only}[kind]
        listed = {split_budget(e)[0] for b in blocks for e in b.all_entries()}
        deferred = {markers[m] for m in listed if m in markers}
        pending: Dict[str, str] = {}
        if carried and CARRIED not in listed:
            flush()
        for blk in blocks:
            for e in blk.s3:
                emit(split_budget(e)[0], r, "S3")
            fwd_comm = any(program.has(split_budget(e)[0]) and program.op(split_budget(e)[0]).strand == "fwd" for e in blk.s3)
            order = (("S2", blk.s2), ("S1", blk.s1)) if fwd_comm else (("S1", blk.s1), ("S2", blk.s2))
            for lane, lst in order:
                for e in lst:
                    name = split_budget(e)[0]
                    if name == CARRIED:
                        flush(lane)
                        continue
                    if name.endswith(CARRY_SUFFIX) and name[:-len(CARRY_SUFFIX)] in markers.values():
                        base = name[:-len(CARRY_SUFFIX)]
                        st = lane_stream(lane)
                        # the executor snapshots the producers' streams at hand-over time
                        waits = tuple(f"{d}#{r}" for d in program.op(base).deps if stream_of.get(f"{d}#{r}") not in (None, st))
                        carried.append((base, r, lane, waits))
                        continue
                    if name in markers:
                        if markers[name] in pending:
                            pending.pop(markers[name])
                            emit(markers[name], r, lane)
                        continue
                    if name in deferred:
                        pending[name] = lane
                        continue
                    emit(name, r, lane)
        for name in list(pending):
            emit(name, r, "S2")
    flush()
    return out, notes


def check_buffer_reuse(program: LayerProgram, strategy: Strategy, effects: Dict[str, list], compute_streams: int = 1,
                       kinds: Sequence[str] = ("fwd", "fwd", "fwd", "pair", "pair", "pair", "pair", "bwd", "bwd", "bwd"), slots: int = 2):
    """Raises ``RaceError`` if some use k+``slots`` of a staging / partial-product site can
    overwrite its slot while a rank may still read use k (see the comment block above)."""
    strat = strategy.completed(program)
    launches, notes = launches_of_runs(program, strat, kinds, compute_streams, effects)
    before = _ancestors(launches)
    n = len(launches)
    # collectives as (contribution index, completion index)
    open_push: Dict[str, List[int]] = {}
    syncs: List[Tuple[int, int]] = []
    uses: Dict[str, List[dict]] = {}             # site -> [{"writers": [...], "readers": [...]}] in order of use
    for i, acts in enumerate(notes):
        for action, site in acts:
            u = uses.setdefault(site, [])
            if action == "push":
                open_push.setdefault(site, []).append(i)
                u.append({"writers": [i], "readers": []})
            elif action == "wait_read":
                q = open_push.get(site) or []
                if not q:
                    raise RaceError(f"{launches[i].op} waits for an all-gather of {site} that was never started")
                c = q.pop(0)
                syncs.append((c, i))
                # the use this wait belongs to is the oldest one without a waiting reader
                tgt = next((x for x in u if not x.get("waited")), None)
                if tgt is None:
                    raise RaceError(f"{launches[i].op}: no pending use of {site}")
                tgt["waited"] = True
                tgt["readers"].append(i)
                tgt["last_wait"] = i
            elif action == "read":
                tgt = next((x for x in reversed(u) if x.get("waited")), None)
                if tgt is None:
                    raise RaceError(f"{launches[i].op} reads {site} before any wait for it")
                # a carried reader belongs to the use whose wait happened before it in its own run: the latest waited use
                # whose wait is an ancestor of (or is) this launch
                cand = [x for x in u if x.get("waited") and (x["last_wait"] in before[i] or x["last_wait"] == i)]
                (cand[-1] if cand else tgt)["readers"].append(i)
            elif action == "write":
                u.append({"writers": [i], "readers": [], "rs": True})
            elif action == "reduce":
                tgt = next((x for x in u if x.get("rs") and not x.get("reduced")), None)
                if tgt is None:
                    raise RaceError(f"{launches[i].op} reduces {site} but no partial product was written")
                tgt["reduced"] = True
                tgt["readers"].append(i)
                # The reduction on rank R finishes only after every rank's GEMM has delivered every row
                # block of R (per-block counters; or, in the whole-buffer form, after every rank announced,
                # which it does after its GEMM).  So the contribution is the GEMM that wrote the partial
                # product and the completion is the reduction.
                syncs.append((tgt["writers"][0], i))
            else:
                raise ValueError(f"unknown buffer action {action!r}")

    def ordered_across_ranks(r: int, w: int) -> bool:
        for c, d in syncs:
            if (r in before[c] or r == c) and r != d and (d in before[w] or d == w):
                return True
        return False

    for site, u in uses.items():
        for k in range(len(u) - slots):
            for r in u[k]["readers"]:
                for w in u[k + slots]["writers"]:
                    if not ordered_across_ranks(r, w):
                        raise RaceError(f"site {site}: {launches[w].op} (use {k + slots}) may overwrite the slot that "
                                        f"{launches[r].op} (use {k}) still reads on another rank: no collective orders them")
    return True
