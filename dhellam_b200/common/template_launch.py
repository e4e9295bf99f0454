"""Launch templates: run a callable on a given CUDA stream, optionally timed on the device.

Same role as the reference's ``launch_cuda_stream`` / ``launch_cuda_stream_with_event``
helpers (dhellam/common/template_launch.py:1-69), which every Python-level op of the
reference goes through; the executor of this framework does the same work per op
(``sched/executor.py``), these free functions serve user code and the operator wrappers with
the reference's signatures.  On CPU tensors (no stream) the callable simply runs.
"""
from __future__ import annotations

import time
from typing import Callable, Optional, Tuple

import torch


def launch_on_stream(fn: Callable, *args, stream: Optional["torch.cuda.Stream"] = None, profiling: bool = False, **kwargs) -> Tuple[object, float]:
    """Runs ``fn(*args, **kwargs)`` on ``stream`` (current stream if ``None``).  Returns
    ``(result, elapsed_ms)``; the time is measured with CUDA events on that stream when
    ``profiling`` is set (it synchronises the stream), else it is 0."""
    if not torch.cuda.is_available() or (stream is None and not profiling):
        t0 = time.perf_counter()
        out = fn(*args, **kwargs)
        return out, ((time.perf_counter() - t0) * 1e3 if profiling and not torch.cuda.is_available() else 0.0)
    s = stream if stream is not None else torch.cuda.current_stream()
    with torch.cuda.stream(s):
        if profiling:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            out = fn(*args, **kwargs)
            e1.record(s)
            e1.synchronize()
            return out, e0.elapsed_time(e1)
        return fn(*args, **kwargs), 0.0


def launch_with_event(fn: Callable, *args, stream: Optional["torch.cuda.Stream"] = None, wait: Optional["torch.cuda.Event"] = None,
                      **kwargs) -> Tuple[object, Optional["torch.cuda.Event"]]:
    """Runs ``fn`` on ``stream`` after ``wait`` (an event of another stream) and returns
    ``(result, done_event)`` so that a consumer on a third stream can wait for it; this is the
    building block of the event-chained schedule (no device-wide synchronisation)."""
    if not torch.cuda.is_available():
        return fn(*args, **kwargs), None
    s = stream if stream is not None else torch.cuda.current_stream()
    if wait is not None:
        s.wait_event(wait)
    with torch.cuda.stream(s):
        out = fn(*args, **kwargs)
    done = torch.cuda.Event()
    done.record(s)
    return out, done
