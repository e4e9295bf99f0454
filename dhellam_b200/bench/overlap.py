"""Pairwise overlap micro-benchmark: how much two operators gain from running side by side
on two streams, for every pair out of {gemm, bda, ln, swiglu, fa, rs, a2a} (forward form)
x the same list (backward form).  Writes ``speedup.csv`` and ``efficiency.csv`` where

    speedup    = (a + b) / c            a, b: times alone, c: time side by side
    efficiency = (a + b - c) / min(a, b)

as the reference's ``micro_benchmark/overlap.py:152-223`` does, plus one extension: the
``--budgets`` sweep co-runs the pair with the first operator confined to k CTAs and the
second to the remaining SMs, which is this framework's knob for partitioning the GPU between
the strands (the reference would use TPC masks).

    torchrun --nproc-per-node 2 -m dhellam_b200.bench.overlap --rows 8192 --hidden 8192
"""
from __future__ import annotations

import argparse
import csv
import os

import torch
import torch.distributed as dist

from ..common.benchmark import benchmark_ms_ops, device_time_ms
from ..common.common import print_rank0
from ..ops import activation as A
from ..ops import attention as ATT
from ..ops import bda as BDA
from ..ops import comm as C
from ..ops import gemm as G
from ..ops import norm as N

NAMES = ["gemm", "bda", "ln", "swiglu", "fa", "rs", "a2a"]


def build_ops(rows, h, ffn, heads, kv_heads, seq, device, dtype, group, backward: bool, budget: int = 0):
    """Returns ``{name: (closure, is_comm)}`` on fresh tensors."""
    def t(*shape):
        return (torch.randn(*shape, device=device) * 0.1).to(dtype)
    x, w, dy = t(rows, h), t(ffn, h), t(rows, ffn)
    lnw = t(h) + 1
    y2 = t(rows, 2 * ffn // 4)
    B = max(rows // seq, 1)
    d = 128 if device.type == "cuda" else 16
    q, k, v = t(seq, B, heads, d), t(seq, B, kv_heads, d), t(seq, B, kv_heads, d)
    ws = C.group_size(group)
    ops = {}
    if backward:
        ops["gemm"] = (lambda: G.gemm_nn(dy, w, sm_budget=budget), False)
        ops["bda"] = (lambda: BDA.bda_bwd(x, 0.1, 3), False)
        y, rstd = N.rmsnorm_fwd(x, lnw)
        ops["ln"] = (lambda: N.rmsnorm_bwd(x, x, lnw, rstd, sm_budget=budget), False)
        do = t(rows, y2.shape[1] // 2)
        ops["swiglu"] = (lambda: A.swiglu_bwd(do, y2, sm_budget=budget), False)
        o, lse = ATT.attn_fwd(q, k, v, True)
        dq = torch.empty_like(q)
        ops["fa"] = (lambda: ATT.attn_bwd(o, q, k, v, o, lse, True), False)
    else:
        ops["gemm"] = (lambda: G.gemm_nt(x, w, sm_budget=budget), False)
        ops["bda"] = (lambda: BDA.bda_fwd(x, x, None, 0.1, 3, sm_budget=budget), False)
        ops["ln"] = (lambda: N.rmsnorm_fwd(x, lnw, sm_budget=budget), False)
        ops["swiglu"] = (lambda: A.swiglu_fwd(y2, sm_budget=budget), False)
        ops["fa"] = (lambda: ATT.attn_fwd(q, k, v, True), False)
    if ws > 1:
        shard = x[: rows // ws].contiguous()
        ops["rs"] = ((lambda: C.gather_along_first_dim(shard, group)) if backward else
                     (lambda: C.reduce_scatter_along_first_dim(x, group)), True)
        out = torch.empty_like(x)
        ops["a2a"] = (lambda: dist.all_to_all_single(out, x, group=group), True)
    return ops


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=7168)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=1)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--repeat", type=int, default=5)
    ap.add_argument("--budgets", type=str, default="", help="comma-separated CTA budgets for the first operator")
    ap.add_argument("--out-dir", default=".")
    args = ap.parse_args(argv)
    from ..parallel import state as PS
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if world > 1:
        PS.init_distributed()
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    group = dist.group.WORLD if world > 1 else None
    s1 = torch.cuda.Stream() if cuda else None
    s2 = torch.cuda.Stream() if cuda else None
    s3 = torch.cuda.Stream() if cuda else None
    fwd = build_ops(args.rows, args.hidden, args.ffn, args.heads, args.kv_heads, args.seq, device, dtype, group, False)
    bwd = build_ops(args.rows, args.hidden, args.ffn, args.heads, args.kv_heads, args.seq, device, dtype, group, True)

    def alone(entry):
        fn, is_comm = entry
        return benchmark_ms_ops(args.repeat, s1, s2, [] if is_comm else [fn], [], fn if is_comm else None, s3, group)

    speed, eff = {}, {}
    for fn_name, fe in fwd.items():
        a = alone(fe)
        for bn_name, be in bwd.items():
            if fe[1] and be[1]:
                continue                      # two collectives are never paired
            b = alone(be)
            comm = fe[0] if fe[1] else (be[0] if be[1] else None)
            c = benchmark_ms_ops(args.repeat, s1, s2, [] if fe[1] else [fe[0]], [] if be[1] else [be[0]], comm, s3, group)
            speed[(fn_name, bn_name)] = (a + b) / c if c > 0 else 0.0
            eff[(fn_name, bn_name)] = (a + b - c) / min(a, b) if min(a, b) > 0 else 0.0
            print_rank0(f"{fn_name:7s} || {bn_name:7s}: alone {a:.3f} + {b:.3f} ms, together {c:.3f} ms, "
                        f"speedup {speed[(fn_name, bn_name)]:.3f}, efficiency {eff[(fn_name, bn_name)]:.3f}")
    if not dist.is_initialized() or dist.get_rank() == 0:
        os.makedirs(args.out_dir, exist_ok=True)
        for fname, table in (("speedup.csv", speed), ("efficiency.csv", eff)):
            with open(os.path.join(args.out_dir, fname), "w", newline="") as fp:
                wr = csv.writer(fp)
                wr.writerow(["fwd\\bwd"] + [n for n in NAMES if n in bwd])
                for f in NAMES:
                    if f in fwd:
                        wr.writerow([f] + [f"{table.get((f, b), float('nan')):.4f}" for b in NAMES if b in bwd])
    if args.budgets and cuda:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        for k in [int(x) for x in args.budgets.split(",")]:
            f1 = build_ops(args.rows, args.hidden, args.ffn, args.heads, args.kv_heads, args.seq, device, dtype, group, False, k)
            b1 = build_ops(args.rows, args.hidden, args.ffn, args.heads, args.kv_heads, args.seq, device, dtype, group, True, sms - k)
            c = benchmark_ms_ops(args.repeat, s1, s2, [f1["gemm"][0]], [b1["gemm"][0]], None, s3, group)
            print_rank0(f"gemm@{k} || gemm@{sms - k}: {c:.3f} ms")
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
