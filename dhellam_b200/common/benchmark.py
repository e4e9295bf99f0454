"""Timing harness: device-timed (CUDA events) counterparts of the reference's
``dhellam/common/benchmark.py`` (host wall clock, 20 % trimmed mean on rank 0, :31-79).

``benchmark_ms_ops`` times "stream-1 op list || stream-2 op list || collectives" the way the
pair profiler needs it.  Times are taken with events on the launching streams after a
warm-up and reduced with MAX over the ranks of ``group``.
"""
from __future__ import annotations

import time
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


def _trimmed_mean(xs, frac=0.2):
    xs = sorted(xs)
    k = int(len(xs) * frac)
    if k > 0 and len(xs) > 10:
        xs = xs[k:-k]
    return sum(xs) / max(len(xs), 1)


def device_time_ms(fn: Callable[[], None], repeat: int = 5, warmup: int = 2, group=None, streams: Sequence = ()) -> float:
    """Mean device time of ``fn()`` in ms.  ``streams``: side streams that ``fn`` uses; the
    measurement brackets them with events on the current stream.  On CPU tensors (no CUDA)
    the host clock is used instead."""
    cuda = torch.cuda.is_available()
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(repeat):
        if cuda:
            cur = torch.cuda.current_stream()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(cur)
            for s in streams:
                s.wait_stream(cur)
            fn()
            for s in streams:
                cur.wait_stream(s)
            e1.record(cur)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        else:
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    ms = _trimmed_mean(times)
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda" if cuda and dist.get_backend(group) == "nccl" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        ms = float(t)
    return ms


def benchmark(repeat: int, fn, *args, **kwargs) -> float:
    """Mean time of ``fn(*args, **kwargs)`` in ms (reference: benchmark.py:4-14)."""
    return device_time_ms(lambda: fn(*args, **kwargs), repeat=repeat, warmup=1)


def benchmark_ms(repeat: int, s1, s2, fn1, fn2) -> float:
    """``fn1`` on stream ``s1`` beside ``fn2`` on ``s2`` (reference: benchmark.py:17-29)."""
    def both():
        with torch.cuda.stream(s1):
            fn1()
        with torch.cuda.stream(s2):
            fn2()
    return device_time_ms(both, repeat=repeat, warmup=1, streams=[s for s in (s1, s2) if s is not None])


def benchmark_ms_ops(repeat: int, s1, s2, ops1: Sequence[Callable], ops2: Sequence[Callable], comm: Optional[Callable] = None,
                     comm_stream=None, group=None) -> float:
    """Launches ``comm`` first (on ``comm_stream``), then ``ops1`` on ``s1`` and ``ops2`` on
    ``s2``; returns the device time of the whole bundle, max over ``group``."""
    cuda = torch.cuda.is_available()

    def bundle():
        if comm is not None:
            if cuda and comm_stream is not None:
                with torch.cuda.stream(comm_stream):
                    comm()
            else:
                comm()
        for lst, s in ((ops1, s1), (ops2, s2)):
            for op in lst:
                if cuda and s is not None:
                    with torch.cuda.stream(s):
                        op()
                else:
                    op()
    streams = [s for s in (s1, s2, comm_stream) if s is not None] if cuda else []
    return device_time_ms(bundle, repeat=repeat, warmup=2, group=group, streams=streams)


def benchmark_ms_ops_cp(repeat: int, s1, s2, ops1: Sequence[Callable], ops2: Sequence[Callable], comms: Sequence[Callable] = (),
                        comm_stream=None, group=None, wait_fwd: bool = False, wait_bwd: bool = False) -> float:
    """As ``benchmark_ms_ops`` with several collectives (the ring steps of context-parallel
    attention): all of ``comms`` are launched first on ``comm_stream``; with ``wait_fwd`` /
    ``wait_bwd`` the stream-1 / stream-2 list starts only after them (the consumer of a ring
    step cannot start before its KV block arrived).  Reference: benchmark.py:82-149."""
    cuda = torch.cuda.is_available()

    def bundle():
        for c in comms:
            if cuda and comm_stream is not None:
                with torch.cuda.stream(comm_stream):
                    c()
            else:
                c()
        done = None
        if cuda and comm_stream is not None and comms and (wait_fwd or wait_bwd):
            done = torch.cuda.Event()
            done.record(comm_stream)
        for lst, s, wait in ((ops1, s1, wait_fwd), (ops2, s2, wait_bwd)):
            if cuda and s is not None and wait and done is not None:
                s.wait_event(done)
            for op in lst:
                if cuda and s is not None:
                    with torch.cuda.stream(s):
                        op()
                else:
                    op()
    streams = [s for s in (s1, s2, comm_stream) if s is not None] if cuda else []
    return device_time_ms(bundle, repeat=repeat, warmup=2, group=group, streams=streams)


def benchmark_dhellam(repeat: int, sequential: Callable[[], None], paired: Callable[[], None], group=None, streams: Sequence = ()):
    """Times a sequential execution (forward-only then backward-only schedule) against the
    paired schedule of the same work and returns ``(sequential_ms, paired_ms, speedup)``, the
    three figures the reference's strategy validator prints (benchmark.py:151-195,
    search/execute.py:107-113)."""
    seq = device_time_ms(sequential, repeat=repeat, warmup=2, group=group, streams=streams)
    par = device_time_ms(paired, repeat=repeat, warmup=2, group=group, streams=streams)
    return seq, par, (seq / par if par > 0 else float("nan"))
