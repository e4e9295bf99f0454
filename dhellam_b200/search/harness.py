"""Layer harness for the strategy search: one block pair with synthetic inputs on which any
contiguous group of forward-strand or backward-strand ops can be replayed and timed.

The reference builds per-op synthetic inputs by hand (search/op_table.py:127-361).  Here a
reference pass through the real layer program records, before every op, which transient
values and saved activations exist; replaying a group restores that record (tensors are
shared, dictionaries are copied) and runs the ops themselves, so the profiler measures
exactly the kernels and collectives that training runs, at the training shapes.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config import ModelConfig, TrainConfig
from ..core.engine import Env
from ..core.modules import DSLLM
from ..data import make_microbatch, synthetic_tokens
from ..models.transformer import build_layer_program
from ..sched.executor import StreamSet
from ..sched.ir import BWD, FWD, LayerRun
from .op_table import expand


class LayerHarness:
    def __init__(self, cfg: ModelConfig, ps, train: TrainConfig, device, fused=None):
        self.cfg, self.ps, self.train, self.device = cfg, ps, train, torch.device(device)
        one_pair = ModelConfig(**{**cfg.__dict__, "num_layers": 2 * ps.pp})
        self.model = DSLLM(one_pair, ps, train, device=self.device)
        self.env = Env(one_pair, ps, train, self.device, self.model.dtype, fused=fused)
        if fused is not None:
            fused.lenient = True           # ops are replayed out of context: never wait for a collective that is not part of the group
        self.program = build_layer_program(one_pair, cp=ps.cp)
        self.streams = StreamSet(self.device if self.device.type == "cuda" else None)
        self.env.streams = self.streams
        self.mb = make_microbatch(one_pair, ps, synthetic_tokens(one_pair, train.micro_batch_size, 17), 0, 17, self.device)
        self.first, self.second = self.model.blocks[0]
        self.snap: Dict[str, tuple] = {}
        self._reference_pass()

    def _reference_pass(self):
        rows = self.mb.tokens.numel() // self.ps.tp
        g = torch.Generator(device="cpu").manual_seed(5)
        x = (torch.randn(rows, self.cfg.hidden_size, generator=g) * 0.5).to(self.model.dtype).to(self.device)
        dout = (torch.randn(rows, self.cfg.hidden_size, generator=g) * 0.01).to(self.model.dtype).to(self.device)
        acts: dict = {}
        frun = LayerRun(self.first, acts, self.mb, self.env, {"x": x}, 0)
        for name, op in self.program.fwd.items():
            self.snap[name] = (dict(frun.v), dict(frun.acts))
            op.fn(frun)
        brun = LayerRun(self.first, dict(acts), self.mb, self.env, {"dout": dout}, 0)
        for name, op in self.program.bwd.items():
            self.snap[name] = (dict(brun.v), dict(brun.acts))
            op.fn(brun)
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def names(self, ids: Sequence[int]) -> List[str]:
        out = []
        for i in ids:
            out.extend(n for n in expand(i) if self.program.has(n))
        return out

    def replay(self, ids: Sequence[int]):
        """Returns ``(begin, compute closures, comm closures)`` that re-run the ops behind
        ``ids`` (a contiguous group of one strand) from the recorded state; call ``begin()``
        once before each replay of the group."""
        names = self.names(ids)
        if not names:
            return (lambda: None), [], []
        v, acts = self.snap[names[0]]
        state = {"run": None}

        def begin():
            # the fused-comm re-gather bookkeeping is per call; start it from a clean slate
            fused = self.env.fused
            if fused is not None:
                fused._pending.clear()
                fused._split_pending.clear()
            state["run"] = LayerRun(self.first, dict(acts), self.mb, self.env, dict(v), 0)

        comp, comm = [], []
        for n in names:
            op = self.program.op(n)

            def call(op=op):
                run = state["run"]
                self.env.cur_stream = torch.cuda.current_stream() if self.device.type == "cuda" else None
                # a value that an op of the group expects but that was produced by an op the
                # group's launch order placed later (a collective launched first) comes from
                # the record
                try:
                    op.fn(run)
                except KeyError:
                    sv, sa = self.snap[op.name]
                    for kk, vv in sv.items():
                        run.v.setdefault(kk, vv)
                    for kk, vv in sa.items():
                        run.acts.setdefault(kk, vv)
                    op.fn(run)
            (comm if op.kind == "comm" else comp).append(call)
        return begin, comp, comm
