"""Data-parallel gradient reduction overlapped with the backward pass.

The engine writes weight gradients straight into the flat fp32 ``main_grad`` buffer, so no
autograd hook ever fires; the reference therefore reduces all gradients only after the last
micro-batch (``finalize_model_grads``; dhellam/core/dstb.py:541-563, megatron.patch:696-700).
Here the engine tells the reducer when a layer's gradients are final (the backward strand of
the LAST micro-batch has left that layer) and the reducer launches the all-reduce of that
layer's contiguous slice of the flat buffer on the communication stream, under the rest of
the backward pass.  Because of the fold, layers become final in two interleaved descending
orders (second-half layers during down sweeps, first-half layers during up sweeps); each
(block pair, half) is one bucket.

With the distributed optimizer (every rank owns a contiguous 1/dp slice of the flat buffer) a
bucket is not all-reduced but reduce-scattered: every piece of the bucket is reduced straight to
the rank whose optimizer shard it falls into (``shard_bounds``), half the bytes of an all-reduce,
and still under the backward pass.
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist


class OverlappedGradReducer:
    def __init__(self, model, ps, streams=None):
        self.model, self.ps, self.streams = model, ps, streams
        self.group = ps.dp_cp_group
        self.size = ps.dp * ps.cp
        self.buckets: Dict[int, Tuple[int, int]] = {}
        # storage order inside a block pair: all "first" parameters, then all "second" ones
        for j, m in enumerate(model.dctb):
            for which, idx in (("first", m.first_index), ("second", m.second_index)):
                offs = []
                for base in m.shapes:
                    off, shape = model.param_index[f"dctb.{j}.{base}_{which}"]
                    offs.append((off, off + math.prod(shape)))
                self.buckets[idx] = (min(o for o, _ in offs), max(e for _, e in offs))
        self.handles: List = []
        self.done: set = set()
        # [lo, hi) of every group rank's optimizer shard; None = replicated optimizer (all-reduce)
        self.shard_bounds = None

    def set_shards(self, bounds):
        """``bounds[r] = (lo, hi)`` of group rank ``r``'s slice of the flat buffer (distributed optimizer)."""
        self.shard_bounds = list(bounds)

    def _reduce(self, lo: int, hi: int, async_op: bool):
        """Reduces ``flat_grad[lo:hi]`` over the group: to everybody, or piecewise to the owners."""
        g = self.model.flat_grad
        out = []
        if self.shard_bounds is None:
            out.append(dist.all_reduce(g[lo:hi], group=self.group, async_op=async_op))
            return out
        ranks = dist.get_process_group_ranks(self.group)
        for r, (slo, shi) in enumerate(self.shard_bounds):
            a, b = max(lo, slo), min(hi, shi)
            if a < b:
                out.append(dist.reduce(g[a:b], dst=ranks[r], group=self.group, async_op=async_op))
        return out

    def active(self) -> bool:
        return self.size > 1 and not (self.model.cfg.is_moe and self.ps.ep > 1)

    def start_step(self):
        self.handles, self.done = [], set()

    def layer_final(self, layer_index: int, producer_stream=None):
        """Called by the engine once ``layer_index`` will receive no more gradient."""
        if not self.active() or layer_index in self.done:
            return
        lo, hi = self.buckets[layer_index]
        st = self.streams
        if st is not None and st.cuda:
            st.s3.wait_stream(producer_stream if producer_stream is not None else st.s2)
            with torch.cuda.stream(st.s3):
                self.handles.extend(self._reduce(lo, hi, True))
        else:
            self._reduce(lo, hi, False)
        self.done.add(layer_index)

    def finish(self):
        """Reduces what is left (head block, padding) and waits for the overlapped buckets.
        Returns True if the flat buffer (this rank's shard of it, with the distributed optimizer) now holds
        the SUM over the group."""
        if not self.active():
            return False
        for h in self.handles:
            h.wait()
        g = self.model.flat_grad
        covered = sorted(self.buckets[i] for i in self.done)
        pos = 0
        for lo, hi in covered + [(g.numel(), g.numel())]:
            if lo > pos:
                self._reduce(pos, lo, False)
            pos = max(pos, hi)
        return True
