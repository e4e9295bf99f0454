"""Launch templates: run a callable on a given CUDA stream, optionally timed on the device.

The reference has four helpers (dhellam/common/template_launch.py): ``template_fwd`` /
``template_bwd`` (:4-36, dictionary-style ops with a user-supplied backward) and
``template_fwd_new`` / ``template_bwd_new`` (:38-70), which build a hand-made autograd context
``[[inputs that require grad], outputs]`` in the forward and differentiate it with
``torch.autograd.backward`` in the backward; its head block is driven through the latter pair.
All four are provided here with the same signatures and return values.  ``launch_on_stream`` /
``launch_with_event`` are this framework's own building blocks (the executor does the same
work per op in ``sched/executor.py``).  On a machine without CUDA the callables simply run.
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


def _timed_on(stream, profiling: bool, body: Callable):
    """Runs ``body()`` on ``stream``; returns ``(result, elapsed ms)`` (CUDA events on that stream
    when ``profiling``; 0 otherwise)."""
    if not torch.cuda.is_available():
        t0 = time.perf_counter()
        out = body()
        return out, ((time.perf_counter() - t0) * 1e3 if profiling else 0)
    s = stream if stream is not None else torch.cuda.current_stream()
    with torch.cuda.stream(s):
        if not profiling:
            return body(), 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = body()
        e1.record()
        e1.synchronize()
        return out, e0.elapsed_time(e1)


def template_fwd(fwd_func: Callable, inputs, stream=None, profiling: bool = False):
    """``outputs = fwd_func(inputs)``; returns ``([inputs, outputs], ms)`` (reference :4-19)."""
    outputs, ms = _timed_on(stream, profiling, lambda: fwd_func(inputs))
    return [inputs, outputs], ms


def template_bwd(bwd_func: Callable, ctx, grad_outputs, stream=None, profiling: bool = False):
    """``grads = bwd_func(ctx, grad_outputs)``; returns ``(grads, ms)`` (reference :21-36)."""
    return _timed_on(stream, profiling, lambda: bwd_func(ctx, grad_outputs))


def template_fwd_new(fwd_func: Callable, *inputs, stream=None, profiling: bool = False):
    """``outputs = fwd_func(*inputs)``; returns ``([[tensor inputs that require grad], outputs], ms)``:
    the list is the context that ``template_bwd_new`` differentiates (reference :38-53)."""
    outputs, ms = _timed_on(stream, profiling, lambda: fwd_func(*inputs))
    return [[t for t in inputs if isinstance(t, torch.Tensor) and t.requires_grad], outputs], ms


def template_bwd_new(ctx, grad_outputs, stream=None, profiling: bool = False):
    """Back-propagates ``grad_outputs`` through ``ctx[1]`` down to the tensors in ``ctx[0]`` (all
    leaves of the graph when that list is empty) and returns ``([t.grad for t in ctx[0]], ms)``
    (reference :55-70)."""
    _, ms = _timed_on(stream, profiling,
                      lambda: torch.autograd.backward(ctx[1], grad_tensors=grad_outputs, inputs=ctx[0] if ctx[0] else None))
    return [t.grad for t in ctx[0]], ms
