"""Per-op device times of one training step (the executor's profile mode).

    python -m dhellam_b200.bench.op_profile --layers 8 --micro-batch 2 --micro-batches 4
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 -m dhellam_b200.bench.op_profile --layers 8 --micro-batch 4

Every op of the layer program is bracketed by CUDA events on the stream it runs on (after the
stream has waited for the op's inputs, so a wait for another stream is not counted, but a
wait that happens inside a kernel, such as the arrival counters of a gathered operand, is).
Rank 0 prints the mean time per op, the totals of the compute lane and the communication
lane, and the wall time of the step; the difference between the compute-lane total and the
wall time is what the head, the optimizer and stalls of the compute stream cost.  The
reference's counterpart is its per-op ``profiling`` flag and ``benchmark_ms`` harness
(dhellam/common/benchmark.py, dhellam/core/dstb.py:80-107).
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3.1-70b-8l")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--micro-batches", type=int, default=4)
    ap.add_argument("--no-fused-comm", action="store_true")
    ap.add_argument("--single-stream", action="store_true")
    a = ap.parse_args(argv)
    from ..config import ParallelConfig, TrainConfig, preset
    from ..data import make_microbatch, synthetic_tokens
    from ..parallel import state as PS
    from ..trainer import Trainer
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        PS.init_distributed("nccl", 10)
    cfg = preset(a.model, num_layers=a.layers)
    mbs, nmb = a.micro_batch, a.micro_batches
    train = TrainConfig(micro_batch_size=mbs, global_batch_size=mbs * nmb, dtype="bf16", fused_comm=not a.no_fused_comm)
    tr = Trainer(cfg, ParallelConfig(tp=world), train, device=torch.device("cuda", torch.cuda.current_device()), profile=True,
                 single_stream=a.single_stream)

    def batches(step):
        return [make_microbatch(cfg, tr.ps, synthetic_tokens(cfg, mbs, 7 + i + step * 10), i, 7 + i, tr.device) for i in range(nmb)]

    for s in range(2):
        tr.train_step(batches(s))
    torch.cuda.synchronize()
    ex = tr.engine.executor
    ex.timings.clear()
    b = batches(5)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    tr.train_step(b)
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3
    tm = ex.timing_ms()
    if rank == 0:
        prog = tr.engine.program
        total = comm = 0.0
        for k, v in sorted(tm.items(), key=lambda kv: -kv[1]):
            n = len(ex.timings[k])
            kind = prog.op(k).kind if prog.has(k) else "?"
            total += v * n
            comm += v * n if kind == "comm" else 0.0
            print(f"{k:32s} {v:8.3f} ms x {n:3d}  {kind}")
        print(f"compute-lane ops {total - comm:.1f} ms, communication-lane ops {comm:.1f} ms, step wall {wall:.1f} ms "
              f"({cfg.num_layers} layers, micro-batch {mbs} x {nmb}, {world} GPU(s), fused_comm={bool(tr.env.fused_tp)})")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
