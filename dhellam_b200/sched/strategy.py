"""Strategy files: the paired schedule of forward-strand and backward-strand ops.

File format (unchanged from the reference, dhellam/core/dstb.py:891-1041 reads it and
search/search.py:180-244 writes it)::

    { "DCBlocks": [[S1, S2, S3], ...],   # both strands live
      "fwd_only": [[S1, S2, S3], ...],   # optional: no backward input (first round / warm-up)
      "bwd_only": [[S1, S2, S3], ...] }  # optional: no forward input (last round / cool-down)

``S1`` = forward-strand compute ops (stream 1), ``S2`` = backward-strand compute ops
(stream 2), ``S3`` = collectives / ring steps launched first.  Each ``S*`` is a list of op
names, one name, or the string ``"None"``.  One extension: a name may carry an SM budget
as ``"name@96"`` (number of persistent CTAs for that op), which is how co-running two
compute kernels is expressed here instead of TPC masks.

Two more extensions move a weight-gradient GEMM (which nothing downstream waits for) across
the layer boundary, where both strands otherwise wait for a collective at the same time:
``"<wgrad op>_next"`` in place of the op hands it to the next layer run, and ``"carried"``
marks where that next run executes what it was handed.  The reference's ``*_n`` markers
(dhellam/core/dstb.py:1043-1059) defer a weight gradient only within its own layer.

Fused names that the search writes, e.g. ``gemm_wgrad_mlp_c_reduce_scatter_mlp_c_bwd``,
are split into the compute op (``S2``) and the collective (``S3``) as in
search/search.py:189-228.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

from .ir import BWD, COMM, COMPUTE, FWD, LayerProgram

CARRY_SUFFIX = "_next"      # "<op>_next": run <op> in the next layer run
CARRIED = "carried"         # slot where a layer run executes the ops handed over by the previous one

FUSED_SPLIT = {
    "gemm_wgrad_mlp_c_reduce_scatter_mlp_c_bwd": ("gemm_wgrad_mlp_c", "reduce_scatter_mlp_c_bwd"),
    "gemm_wgrad_attn_c_reduce_scatter_attn_c_bwd": ("gemm_wgrad_attn_c", "reduce_scatter_attn_c_bwd"),
}


def _as_list(x) -> List[str]:
    if x is None or x == "None":
        return []
    if isinstance(x, str):
        return [x]
    return [n for n in x if n is not None and n != "None"]


def split_budget(entry: str) -> Tuple[str, int]:
    if "@" in entry:
        n, b = entry.split("@", 1)
        return n, int(b)
    return entry, 0


@dataclass
class Block:
    s1: List[str] = field(default_factory=list)
    s2: List[str] = field(default_factory=list)
    s3: List[str] = field(default_factory=list)

    def to_json(self):
        return [self.s1 or "None", self.s2 or "None", self.s3 or "None"]

    def all_entries(self):
        return self.s3 + self.s1 + self.s2


def _parse_blocks(raw) -> List[Block]:
    blocks = []
    for item in raw or []:
        if len(item) != 3:
            raise ValueError(f"a schedule block needs three entries [S1, S2, S3], got {item!r}")
        s1, s2, s3 = (_as_list(x) for x in item)
        # split the search's fused wgrad+reduce-scatter names
        s2_out = []
        for n in s2:
            base, b = split_budget(n)
            if base in FUSED_SPLIT:
                c, comm = FUSED_SPLIT[base]
                s2_out.append(c if b == 0 else f"{c}@{b}")
                s3 = s3 + [comm]
            else:
                s2_out.append(n)
        blocks.append(Block(s1, s2_out, s3))
    return blocks


@dataclass
class Strategy:
    dcblocks: List[Block] = field(default_factory=list)
    fwd_only: List[Block] = field(default_factory=list)
    bwd_only: List[Block] = field(default_factory=list)

    # ---- (de)serialisation
    @classmethod
    def from_dict(cls, d: dict) -> "Strategy":
        return cls(_parse_blocks(d.get("DCBlocks")), _parse_blocks(d.get("fwd_only")), _parse_blocks(d.get("bwd_only")))

    @classmethod
    def load(cls, path: str) -> "Strategy":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        d = {"DCBlocks": [b.to_json() for b in self.dcblocks]}
        if self.fwd_only:
            d["fwd_only"] = [b.to_json() for b in self.fwd_only]
        if self.bwd_only:
            d["bwd_only"] = [b.to_json() for b in self.bwd_only]
        return d

    def save(self, path: str):
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=1)

    # ---- completion with built-in defaults
    def completed(self, program: LayerProgram) -> "Strategy":
        """Fills missing parts with built-in schedules (the reference falls back the same
        way, dhellam/core/dstb.py:1042-1129; unlike the reference, a missing file is fine)."""
        return Strategy(self.dcblocks or default_paired(program), self.fwd_only or default_single(program, FWD),
                        self.bwd_only or _dense_tp_bwd_only(program) or default_single(program, BWD))

    def validate(self, program: LayerProgram):
        """Checks every part that is present (absent parts are filled by ``completed``)."""
        if self.dcblocks:
            validate_blocks(self.dcblocks, program, need_fwd=True, need_bwd=True)
        if self.fwd_only:
            validate_blocks(self.fwd_only, program, need_fwd=True, need_bwd=False)
        if self.bwd_only:
            validate_blocks(self.bwd_only, program, need_fwd=False, need_bwd=True)


# --------------------------------------------------------------------------- defaults
def _segments(program: LayerProgram, strand: str):
    """Splits a strand into ``(compute ops, trailing comm ops)`` segments.  A deferrable
    compute op that directly follows a collective's producer stays with the collective,
    so that e.g. the column wgrad overlaps its reduce-scatter."""
    segs, cur = [], []
    ops = list((program.fwd if strand == FWD else program.bwd).values())
    i = 0
    while i < len(ops):
        o = ops[i]
        if o.kind == COMM:
            comm = [o.name]
            segs.append((cur, comm))
            cur = []
        else:
            cur.append(o.name)
        i += 1
    if cur:
        segs.append((cur, []))
    return segs


def default_single(program: LayerProgram, strand: str) -> List[Block]:
    blocks = []
    for comp, comm in _segments(program, strand):
        if comp:
            blocks.append(Block(s1=comp) if strand == FWD else Block(s2=comp))
        if comm:
            blocks.append(Block(s3=comm))
    return blocks


def _dense_tp_paired(program: LayerProgram) -> Optional[List[Block]]:
    """Built-in pairing for the dense transformer layer (no ring steps, no experts).

    Every collective but the very first is launched beside work that does not wait for it
    and that lasts longer than the transfer at the headline shapes: the big GEMM groups of
    the other strand, or a weight-gradient GEMM, which nothing downstream waits for.  The
    row-parallel MLP weight gradient is deferred (``gemm_wgrad_mlp_l_n``) to sit beside the
    last reduce-scatter, and the QKV weight gradient is handed to the next layer run, where it
    covers the first all-gather of the forward strand (both strands start a layer with a
    collective, so nothing of the new layer can).  The reference's built-in
    schedule (dhellam/core/dstb.py:1043-1059) follows the same idea with fewer fillers."""
    act_f = "swiglu_mlp" if program.has("swiglu_mlp") else "gelu_mlp"
    act_b = "swiglu_bwd" if program.has("swiglu_bwd") else "gelu_bwd"
    needed = ["ln_attn", "allgather_attn", "gemm_attn_c", "fl_attn", "gemm_attn_l", "reduce_scatter_attn", "bda_attn", "ln_mlp",
              "allgather_mlp", "gemm_mlp_c", act_f, "gemm_mlp_l", "reduce_scatter_mlp", "bda_mlp", "attn_bwd", act_b]
    if not all(program.has(n) for n in needed) or len(program.fwd) != 14 or len(program.bwd) != 18:
        return None
    if os.environ.get("DHELLAM_CARRY_WGRAD", "1") != "0":
        last_fillers = ["gemm_wgrad_mlp_l_n", "gemm_wgrad_attn_c" + CARRY_SUFFIX]
    else:                                     # everything stays inside its own layer run
        last_fillers = ["gemm_wgrad_attn_c", "gemm_wgrad_mlp_l_n"]
    return [
        Block(s1=["ln_attn"]),
        Block(s2=["bda_mlp_bwd", CARRIED], s3=["allgather_attn"]),
        Block(s1=["gemm_attn_c", "fl_attn", "gemm_attn_l"], s3=["allgather_mlp_bwd"]),
        Block(s2=["gemm_dgrad_mlp_l", "gemm_wgrad_mlp_l", act_b, "gemm_dgrad_mlp_c"], s3=["reduce_scatter_attn"]),
        Block(s1=["bda_attn", "ln_mlp"], s3=["reduce_scatter_mlp_c_bwd"]),
        Block(s2=["gemm_wgrad_mlp_c"], s3=["allgather_mlp"]),
        Block(s2=["ln_mlp_bwd", "bda_attn_bwd"]),
        Block(s1=["gemm_mlp_c", act_f, "gemm_mlp_l"], s3=["allgather_attn_bwd"]),
        Block(s2=["gemm_dgrad_attn_l", "gemm_wgrad_attn_l", "attn_bwd", "gemm_dgrad_attn_c"], s3=["reduce_scatter_mlp"]),
        Block(s1=["bda_mlp"], s2=last_fillers, s3=["reduce_scatter_attn_c_bwd"]),
        Block(s2=["ln_attn_bwd"]),
    ]


def _dense_tp_bwd_only(program: LayerProgram) -> Optional[List[Block]]:
    """Built-in backward-only schedule of the dense layer (cool-down rounds, where no forward
    strand is left to cover the collectives): the weight-gradient GEMMs, which wait for no
    collective, are placed beside the four collectives of the backward strand, and the QKV
    weight gradient is handed to the next layer run to cover its first all-gather."""
    act_b = "swiglu_bwd" if program.has("swiglu_bwd") else "gelu_bwd"
    needed = ["bda_mlp_bwd", "allgather_mlp_bwd", "gemm_dgrad_mlp_l", "gemm_wgrad_mlp_l", act_b, "gemm_dgrad_mlp_c", "gemm_wgrad_mlp_c",
              "reduce_scatter_mlp_c_bwd", "ln_mlp_bwd", "bda_attn_bwd", "allgather_attn_bwd", "gemm_dgrad_attn_l", "gemm_wgrad_attn_l",
              "attn_bwd", "gemm_dgrad_attn_c", "gemm_wgrad_attn_c", "reduce_scatter_attn_c_bwd", "ln_attn_bwd"]
    if not all(program.has(n) for n in needed) or len(program.bwd) != 18:
        return None
    carry = os.environ.get("DHELLAM_CARRY_WGRAD", "1") != "0"
    return [
        Block(s2=["bda_mlp_bwd"]),
        Block(s2=[CARRIED], s3=["allgather_mlp_bwd"]),
        Block(s2=["gemm_dgrad_mlp_l", "gemm_wgrad_mlp_l", act_b, "gemm_dgrad_mlp_c"]),       # wgrad_mlp_l waits for its marker
        Block(s2=["gemm_wgrad_mlp_c"], s3=["reduce_scatter_mlp_c_bwd"]),
        Block(s2=["ln_mlp_bwd", "bda_attn_bwd"]),
        Block(s2=["gemm_wgrad_mlp_l_n"], s3=["allgather_attn_bwd"]),
        Block(s2=["gemm_dgrad_attn_l", "gemm_wgrad_attn_l", "attn_bwd", "gemm_dgrad_attn_c"]),    # wgrad_attn_l waits for its marker
        Block(s2=["gemm_wgrad_attn_l_n", "gemm_wgrad_attn_c" + CARRY_SUFFIX if carry else "gemm_wgrad_attn_c"],
              s3=["reduce_scatter_attn_c_bwd"]),
        Block(s2=["ln_attn_bwd"]),
    ]


def reference_paired(program: LayerProgram) -> Optional[List[Block]]:
    """The reference's own built-in paired schedule (dhellam/core/dstb.py:1043-1059), 17 blocks,
    for the dense layer.  Used by the benchmark's composition arm; the engine's default is
    ``default_paired``."""
    act_f = "swiglu_mlp" if program.has("swiglu_mlp") else "gelu_mlp"
    act_b = "swiglu_bwd" if program.has("swiglu_bwd") else "gelu_bwd"
    if not program.has("fl_attn") or not program.has("gemm_mlp_c"):
        return None
    return [
        Block(s1=["ln_attn"]),
        Block(s2=["bda_mlp_bwd"], s3=["allgather_attn"]),
        Block(s1=["gemm_attn_c", "fl_attn"], s3=["allgather_mlp_bwd"]),
        Block(s1=["gemm_attn_l"]),
        Block(s2=["gemm_dgrad_mlp_l", "gemm_wgrad_mlp_l"], s3=["reduce_scatter_attn"]),
        Block(s2=[act_b]),
        Block(s2=["gemm_dgrad_mlp_c"]),
        Block(s2=["gemm_wgrad_mlp_c"], s3=["reduce_scatter_mlp_c_bwd"]),
        Block(s1=["bda_attn", "ln_mlp"]),
        Block(s2=["ln_mlp_bwd", "bda_attn_bwd"], s3=["allgather_mlp"]),
        Block(s1=["gemm_mlp_c"], s3=["allgather_attn_bwd"]),
        Block(s1=[act_f, "gemm_mlp_l"]),
        Block(s2=["gemm_dgrad_attn_l", "gemm_wgrad_attn_l", "attn_bwd"], s3=["reduce_scatter_mlp"]),
        Block(s1=["bda_mlp"]),
        Block(s2=["gemm_dgrad_attn_c"]),
        Block(s2=["gemm_wgrad_attn_c"], s3=["reduce_scatter_attn_c_bwd"]),
        Block(s2=["ln_attn_bwd"]),
    ]


def default_paired(program: LayerProgram) -> List[Block]:
    """Built-in paired schedule.  Dense layers get the hand-placed pairing above; any other
    program gets the generic alternation: each strand's collective is launched together with
    the other strand's next compute segment."""
    dense = _dense_tp_paired(program)
    if dense is not None:
        return dense
    f = _segments(program, FWD)
    b = _segments(program, BWD)
    blocks: List[Block] = []
    pending: List[str] = []          # collectives to launch with the next block
    i = j = 0
    while i < len(f) or j < len(b):
        if i < len(f):
            comp, comm = f[i]
            blocks.append(Block(s1=comp, s3=pending))
            pending = comm
            i += 1
        if j < len(b):
            comp, comm = b[j]
            blocks.append(Block(s2=comp, s3=pending))
            pending = comm
            j += 1
    if pending:
        blocks.append(Block(s3=pending))
    return blocks


# --------------------------------------------------------------------------- validation
class StrategyError(ValueError):
    pass


def validate_blocks(blocks: List[Block], program: LayerProgram, need_fwd: bool, need_bwd: bool):
    """Every op of the needed strands appears exactly once, on the right stream list, and
    never before an op it depends on."""
    markers = program.marker_targets()
    seen: Dict[str, int] = {}
    order = 0
    deferred = set()
    for bi, blk in enumerate(blocks):
        for lst, lane in ((blk.s3, "S3"), (blk.s1, "S1"), (blk.s2, "S2")):
            for entry in lst:
                name, _ = split_budget(entry)
                if name == CARRIED:
                    if lane == "S3":
                        raise StrategyError(f"the slot for carried ops cannot be a collective (block {bi})")
                    continue
                if name.endswith(CARRY_SUFFIX) and name[:-len(CARRY_SUFFIX)] in markers.values():
                    name = name[:-len(CARRY_SUFFIX)]          # scheduled here, executed by the next layer run
                if name in markers:
                    if lane == "S3":
                        raise StrategyError(f"marker {name} cannot be a collective (block {bi})")
                    deferred.add(markers[name])
                    seen[name] = order
                    order += 1
                    continue
                if not program.has(name):
                    raise StrategyError(f"unknown op {name!r} in block {bi}")
                op = program.op(name)
                if name in seen:
                    raise StrategyError(f"op {name} scheduled twice (block {bi})")
                if lane == "S1" and op.strand != FWD:
                    raise StrategyError(f"backward op {name} on the forward stream list (block {bi})")
                if lane == "S2" and op.strand != BWD:
                    raise StrategyError(f"forward op {name} on the backward stream list (block {bi})")
                for d in op.deps:
                    if d not in seen:
                        raise StrategyError(f"op {name} scheduled before its dependency {d} (block {bi})")
                seen[name] = order
                order += 1
    for strand, need in ((FWD, need_fwd), (BWD, need_bwd)):
        for n in program.names(strand):
            if need and n not in seen:
                raise StrategyError(f"op {n} missing from the schedule")
            if not need and n in seen:
                raise StrategyError(f"op {n} of the absent strand appears in a single-strand schedule")
    for m, target in markers.items():
        if m in seen and target in seen and seen[m] < seen[target]:
            raise StrategyError(f"marker {m} placed before {target}")
