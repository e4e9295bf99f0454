"""Operator IR of the dual-strand engine.

A transformer layer is described by two ordered op lists, the *forward strand* and the
*backward strand*.  Every op has the name used in strategy files, a numeric id from the
search's op table, the names of the ops of its own strand it depends on, and a callable
that performs it on a ``LayerRun``.  This replaces the reference's integer-dispatched
``DCoperation.perform_operation`` / ``DCOP`` linked list / ``FuncChoice`` enum
(dhellam/core/dstb.py:24-58, 427-695) with typed data; the op names and the dependency
structure are those of ``init_DCBlocks`` (dhellam/core/dstb.py:698-843).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Tuple

FWD, BWD = "fwd", "bwd"
COMPUTE, COMM, MARKER = "compute", "comm", "marker"
# resource classes used by the pairing search: tensor cores, memory system, NVLink
MMA, MEM, NVL = "MMA", "MEM", "NVL"


@dataclass
class Op:
    name: str
    strand: str
    kind: str
    fn: Optional[Callable] = None
    deps: Tuple[str, ...] = ()
    resource: str = MEM
    op_id: int = -1
    # deferred-wgrad support: ops named here may be postponed to a "<name>_n" marker
    deferrable: bool = False
    # dependencies that are synchronised INSIDE the kernels (per-row-block counters): when the
    # engine enables it, this op may start as soon as such a producer has been launched
    pipelined_deps: Tuple[str, ...] = ()


class LayerProgram:
    """Two strands of ops for one transformer layer."""

    def __init__(self, name: str = "layer"):
        self.name = name
        self.fwd: "OrderedDict[str, Op]" = OrderedDict()
        self.bwd: "OrderedDict[str, Op]" = OrderedDict()

    def add(self, op: Op) -> Op:
        table = self.fwd if op.strand == FWD else self.bwd
        if op.name in self.fwd or op.name in self.bwd:
            raise ValueError(f"duplicate op name {op.name}")
        for d in op.deps:
            if d not in table:
                raise ValueError(f"op {op.name} depends on unknown or later op {d}")
        table[op.name] = op
        return op

    def op(self, name: str) -> Op:
        if name in self.fwd:
            return self.fwd[name]
        if name in self.bwd:
            return self.bwd[name]
        raise KeyError(name)

    def has(self, name: str) -> bool:
        return name in self.fwd or name in self.bwd

    def names(self, strand: str) -> List[str]:
        return list((self.fwd if strand == FWD else self.bwd).keys())

    def marker_targets(self) -> Dict[str, str]:
        """``{marker name: op name}`` for every deferrable op."""
        return {f"{n}_n": n for n, o in self.bwd.items() if o.deferrable}


@dataclass
class LayerRun:
    """One strand's execution of one layer on one micro-batch."""
    params: object                 # LayerParams
    acts: dict                     # saved activations of (micro-batch, layer); forward fills, backward drains
    mb: object                     # MicroBatch (shapes, positions, seeds)
    env: object                    # Env (config, parallel state, implementation switches)
    v: dict = field(default_factory=dict)   # transient values flowing between the ops of this run
    layer_index: int = 0
    sm_budget: Dict[str, int] = field(default_factory=dict)

    def budget(self, op_name: str) -> int:
        return self.sm_budget.get(op_name, 0)
