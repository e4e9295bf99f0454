"""Dual-strand executor: runs the forward strand of one micro-batch and the backward
strand of another through one transformer layer each, following a strategy.

What it keeps from the reference's interpreter (dhellam/core/dstb.py:1133-1281): blocks
run in order; a block first launches its collectives (``S3``), then the compute ops of the
strand that does *not* wait for those collectives, then the other strand; deferred weight
gradients run at their ``*_n`` marker or at the end.  What is different: there is no
device-wide synchronisation per block (the reference calls ``torch.cuda.synchronize()``
after every block, dstb.py:1266).  Ordering is carried by CUDA events between three
streams (forward compute, backward compute, communication), so the host runs ahead of the
device; on CPU tensors the same code runs synchronously without streams.
"""
from __future__ import annotations

import contextlib
import os
from typing import Dict, List, Optional

import torch

from .ir import BWD, COMM, FWD, LayerProgram, LayerRun
from .strategy import CARRIED, CARRY_SUFFIX, Block, Strategy, split_budget


class StreamSet:
    """Three CUDA streams (forward compute, backward compute, communication)."""

    def __init__(self, device=None, single_stream: bool = False, compute_streams: int = 2):
        """``compute_streams = 1`` issues both strands' compute ops to one stream in schedule
        order (collectives still overlap from the communication stream), which is how the
        reference actually trains (it aliases its second stream to the first,
        dhellam/core/dsllm.py:59-61); ``2`` lets compute kernels of the two strands co-run."""
        self.cuda = device is not None and torch.device(device).type == "cuda"
        if self.cuda:
            with torch.cuda.device(device):
                if single_stream:
                    s = torch.cuda.current_stream()
                    self.s1 = self.s2 = self.s3 = s
                else:
                    self.s1 = torch.cuda.Stream()
                    self.s2 = torch.cuda.Stream() if compute_streams >= 2 else self.s1
                    self.s3 = torch.cuda.Stream()
        else:
            self.s1 = self.s2 = self.s3 = None

    def lane(self, lane: str):
        return {"S1": self.s1, "S2": self.s2, "S3": self.s3}[lane]

    def ctx(self, stream):
        return torch.cuda.stream(stream) if (self.cuda and stream is not None) else contextlib.nullcontext()

    def join_all_into(self, target):
        """Makes ``target`` wait for everything enqueued so far on the three streams."""
        if not self.cuda:
            return
        for s in {self.s1, self.s2, self.s3}:
            if s is not target:
                target.wait_stream(s)

    def fork_from(self, source):
        if not self.cuda:
            return
        for s in {self.s1, self.s2, self.s3}:
            if s is not source:
                s.wait_stream(source)


class ExposedTimer:
    """Measures how long compute streams stand still waiting for communication.

    When enabled, every place where a compute stream waits for the communication stream (an event
    wait on a collective's completion, the arrival-counter wait in front of a GEMM that reads a
    gathered operand, a library collective issued on the compute stream itself) is bracketed by
    two timing events on the waiting stream: the first completes when the stream's earlier work
    is done, the second when the wait is over, so their distance is time in which that stream had
    nothing else to run.  ``total_ms`` sums the spans (it synchronises)."""

    def __init__(self):
        self.enabled = False
        self.spans: List[tuple] = []

    @contextlib.contextmanager
    def span(self, stream):
        if not self.enabled or stream is None:
            yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        yield
        e1.record(stream)
        self.spans.append((e0, e1))

    def total_ms(self) -> float:
        torch.cuda.synchronize()
        spans, self.spans = self.spans, []
        return float(sum(a.elapsed_time(b) for a, b in spans))


class Executor:
    def __init__(self, program: LayerProgram, strategy: Strategy, streams: StreamSet, profile: bool = False,
                 trace=None, sync_per_block: bool = False):
        self.program = program
        # True reproduces the reference interpreter's device-wide synchronisation after every
        # schedule block (dhellam/core/dstb.py:1266); only the benchmark's composition arm sets it
        self.sync_per_block = sync_per_block and streams.cuda
        self.exposed = ExposedTimer()
        # producers whose consumers synchronise with them inside the kernels: for those an event is also
        # recorded BEFORE the producer runs, and the consumer waits for that one only
        self.pipeline = False
        self._pipelined_producers = {d for o in list(program.fwd.values()) + list(program.bwd.values()) for d in o.pipelined_deps}
        self._pre_events: Dict[str, object] = {}
        self.strategy = strategy.completed(program)
        self.strategy.validate(program)
        self.streams = streams
        self.profile = profile
        self.trace = trace                       # optional list collecting (name, lane) launch records
        # NVTX range per op ("F:" forward strand, "B:" backward strand, layer and micro-batch in the
        # name) for timelines taken with an external tool; the reference has no ranges at all.
        self.nvtx = streams.cuda and os.environ.get("DHELLAM_NVTX", "0") == "1"
        self.timings: Dict[str, List] = {}
        self._events: Dict[str, object] = {}
        self._lane_of: Dict[str, Dict[str, str]] = {}
        self._markers = program.marker_targets()
        self._carry_names = {f"{n}{CARRY_SUFFIX}": n for n in self._markers.values()}
        self._carry: List[tuple] = []            # weight-gradient ops handed to the next layer run
        for key, blocks in (("pair", self.strategy.dcblocks), ("fwd", self.strategy.fwd_only), ("bwd", self.strategy.bwd_only)):
            lanes = {}
            for blk in blocks:
                for lane, lst in (("S3", blk.s3), ("S1", blk.s1), ("S2", blk.s2)):
                    for e in lst:
                        n = split_budget(e)[0]
                        lanes[self._carry_names.get(n, n)] = lane
            self._lane_of[key] = lanes

    # ------------------------------------------------------------------ public
    def run(self, fwd_run: Optional[LayerRun], bwd_run: Optional[LayerRun]):
        if fwd_run is not None and bwd_run is not None:
            key, blocks = "pair", self.strategy.dcblocks
        elif fwd_run is not None:
            key, blocks = "fwd", self.strategy.fwd_only
        elif bwd_run is not None:
            key, blocks = "bwd", self.strategy.bwd_only
        else:
            return
        lanes = self._lane_of[key]
        deferred_names = {self._markers[m] for m in lanes if m in self._markers}
        pending: Dict[str, tuple] = {}
        runs = {FWD: fwd_run, BWD: bwd_run}

        has_slot = any(split_budget(e)[0] == CARRIED for blk in blocks for e in blk.s1 + blk.s2)
        if self._carry and not has_slot:
            self.flush_carry()

        def launch(entry: str, lane: str):
            name, budget = split_budget(entry)
            if name == CARRIED:                             # slot for what the previous layer run handed over
                self.flush_carry(lane)
                return
            if name in self._carry_names:                   # hand this op to the next layer run
                op = self.program.op(self._carry_names[name])
                self._carry.append((op, runs[op.strand], lane, dict(lanes), budget, self._snapshot(op, lane)))
                return
            if name in self._markers:                       # placement marker of a deferred wgrad
                target = self._markers[name]
                if target in pending:
                    op, run, b = pending.pop(target)
                    self._exec(op, run, lane, lanes, b or budget)
                return
            op = self.program.op(name)
            run = runs[op.strand]
            if name in deferred_names:
                pending[name] = (op, run, budget)
                return
            self._exec(op, run, lane, lanes, budget)

        for blk in blocks:
            for e in blk.s3:
                launch(e, "S3")
            fwd_comm = any(self.program.has(split_budget(e)[0]) and self.program.op(split_budget(e)[0]).strand == FWD
                           for e in blk.s3)
            order = (("S2", blk.s2), ("S1", blk.s1)) if fwd_comm else (("S1", blk.s1), ("S2", blk.s2))
            for lane, lst in order:
                for e in lst:
                    launch(e, lane)
            if self.sync_per_block:
                torch.cuda.synchronize()
        for target, (op, run, b) in list(pending.items()):   # flush what no marker claimed
            self._exec(op, run, "S2", lanes, b)

    def flush_carry(self, lane: Optional[str] = None):
        """Runs the ops that earlier layer runs handed over (on ``lane``, else on the lane they
        were scheduled on).  The engine calls it where their results are needed: before a
        layer's gradients are reduced and at the end of the step."""
        carried, self._carry = self._carry, []
        for op, run, own_lane, lanes, budget, waits in carried:
            self._exec(op, run, lane or own_lane, lanes, budget, waits)

    # ------------------------------------------------------------------ internals
    def _snapshot(self, op, lane: str):
        """Fresh events for the producers of ``op`` that ran on other streams: the per-op
        events are re-recorded by the next layer run, which a carried op must not wait for."""
        st = self.streams
        if not st.cuda:
            return []
        stream = st.lane(lane)
        waits = []
        for s in {rec[1] for d in op.deps if (rec := self._events.get(d)) is not None and rec[1] is not stream}:
            ev = torch.cuda.Event()
            ev.record(s)
            waits.append(ev)
        return waits

    def _exec(self, op, run: LayerRun, lane: str, lanes: Dict[str, str], budget: int, waits=None):
        st = self.streams
        stream = st.lane(lane)
        if self.trace is not None:
            self.trace.append((op.name, lane, run.layer_index, getattr(run.mb, "index", -1)))
        if st.cuda and waits is not None:
            for ev in waits:
                stream.wait_event(ev)
        elif st.cuda:
            for d in op.deps:
                if self.pipeline and d in op.pipelined_deps and d in self._pre_events:
                    stream.wait_event(self._pre_events[d])     # ordered after the producer's launch point only
                    continue
                rec = self._events.get(d)
                if rec is not None and rec[1] is not stream:   # produced on another stream
                    if rec[1] is st.s3 and self.exposed.enabled:
                        with self.exposed.span(stream):        # a compute stream waiting for a collective
                            stream.wait_event(rec[0])
                    else:
                        stream.wait_event(rec[0])
        if budget:
            run.sm_budget[op.name] = budget
        run.env.cur_stream = stream
        if st.cuda and self.pipeline and op.name in self._pipelined_producers:
            pre = self._pre_events.get(op.name) or torch.cuda.Event()
            pre.record(stream)
            self._pre_events[op.name] = pre
        if self.nvtx:
            torch.cuda.nvtx.range_push(f"{'F' if op.strand == FWD else 'B'}:{op.name} L{run.layer_index} mb{getattr(run.mb, 'index', -1)}")
        with st.ctx(stream):
            if self.profile and st.cuda:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                op.fn(run)
                e1.record(stream)
                self.timings.setdefault(op.name, []).append((e0, e1))
            else:
                op.fn(run)
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        if st.cuda:
            rec = self._events.get(op.name)
            ev = rec[0] if rec is not None else torch.cuda.Event()
            ev.record(stream)
            self._events[op.name] = (ev, stream)

    def timing_ms(self) -> Dict[str, float]:
        """Mean device time per op (profile mode); synchronises."""
        if self.streams.cuda:
            torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in self.timings.items() if v}
