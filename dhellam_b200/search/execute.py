"""Strategy executor / validator: times candidate strategy files on a real block pair
(single-strand forward + backward versus the paired schedule) and keeps the fastest as
``config/best.json``.  Role of the reference's ``search/execute.py:34-116``; candidates are
sharded over the data-parallel ranks the same way and the winner is agreed on with a MAX
all-reduce.
"""
from __future__ import annotations

import glob
import json
import os
import shutil
from typing import List, Optional

import torch
import torch.distributed as dist

from ..common.benchmark import device_time_ms
from ..common.common import print_rank0
from ..sched.executor import Executor
from ..sched.ir import LayerRun
from ..sched.strategy import Strategy
from .harness import LayerHarness


def time_strategy(h: LayerHarness, strategy: Strategy, repeat: int = 10):
    """Returns ``(sequential ms, paired ms)`` for one block pair."""
    ex = Executor(h.program, strategy, h.streams)
    if h.env.fused is not None:
        ex.pipeline = h.env.fused.rs_blocks and h.env.fused.policy == "split"
        h.env.exposed = ex.exposed
    name0_f, name0_b = next(iter(h.program.fwd)), next(iter(h.program.bwd))
    vf, af = h.snap[name0_f]
    vb, ab = h.snap[name0_b]

    def runs():
        if h.env.fused is not None:
            h.env.fused._pending.clear()
            h.env.fused._split_pending.clear()
        return (LayerRun(h.first, dict(af), h.mb, h.env, dict(vf), 0), LayerRun(h.first, dict(ab), h.mb, h.env, dict(vb), 0))

    def sequential():
        f, b = runs()
        ex.run(f, None)
        ex.run(None, b)

    def paired():
        f, b = runs()
        ex.run(f, b)
    streams = [s for s in (h.streams.s1, h.streams.s2, h.streams.s3) if s is not None]
    seq = device_time_ms(sequential, repeat=repeat, warmup=2, group=h.ps.tp_group, streams=streams)
    par = device_time_ms(paired, repeat=repeat, warmup=2, group=h.ps.tp_group, streams=streams)
    return seq, par


def run_execute(h: LayerHarness, config_dir: str, out_path: str = "config/best.json", repeat: int = 10):
    """Evaluates every ``*.json`` under ``config_dir`` plus the built-in schedule; copies the
    best one to ``out_path``.  Returns ``(best file or "builtin", speedup percent)``."""
    files = sorted(glob.glob(os.path.join(config_dir, "*.json")))
    dp_rank, dp = h.ps.dp_rank, max(h.ps.dp, 1)
    mine = files[dp_rank::dp]
    results = []
    candidates = [("builtin", Strategy())] + [(f, None) for f in mine]
    for name, strat in candidates:
        try:
            strat = strat if strat is not None else Strategy.load(name)
            if h.env.fused is not None and not h.cfg.is_moe and h.ps.cp == 1:
                # a candidate whose launch order lets a rank overwrite a symmetric slot that another
                # rank still reads is illegal however fast it is
                from ..models.transformer import FUSED_BUFFER_EFFECTS
                from ..sched.checker import check_buffer_reuse
                check_buffer_reuse(h.program, strat, FUSED_BUFFER_EFFECTS, compute_streams=1 if h.streams.s2 is h.streams.s1 else 2)
            seq, par = time_strategy(h, strat, repeat)
        except Exception as e:                      # an illegal candidate is skipped, not fatal
            print_rank0(f"skip {name}: {e}")
            continue
        sp = (seq / par - 1.0) * 100.0
        results.append((sp, name, seq, par))
        print_rank0(f"sequence time :{seq:.3f} schedule time: {par:.3f} speedup: {sp:.2f}% file: {name}")
    best = max(results) if results else (0.0, "builtin", 0.0, 0.0)
    if dist.is_initialized() and h.ps.dp > 1 and h.ps.dp_group is not None:
        t = torch.tensor([best[0]], dtype=torch.float64, device=h.device if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=h.ps.dp_group)
        winner = float(t) == best[0]
    else:
        winner = True
    if winner and h.ps.tp_rank == 0 and h.ps.cp_rank == 0 and best[1] != "builtin":
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        shutil.copy(best[1], out_path)
    return best[1], best[0]
