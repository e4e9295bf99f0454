"""Device-timed benchmark of the tensor-parallel communication paths, one JSON line per path (the collectives
of dhellam/operators/comm.py:13-58 alone and beside the GEMMs they feed or follow, dhellam/core/dstb.py:407-425).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m dhellam_b200.bench.comm_bench [--rows 16384] [--width 8192] [--iters 10]

For every path the time is taken with CUDA events on the launching stream (all ranks start behind a
barrier; the reported time is the max over ranks of the per-rank median), and the roofline is the
slower of the bytes that must cross this GPU's NVLink ports at the measured peer-copy bandwidth and
the GEMM's FLOPs at the measured cuBLAS throughput.  Paths:

* ``peer_copy``     a plain ``copy_`` of 1 GiB into a peer's symmetric buffer: the link figure used below
* ``ag_push``       sequence all-gather alone (multimem / per-peer stores + arrival counters) + the wait
* ``rs_reduce``     sequence reduce-scatter alone, row-block-wise, behind a GEMM that signals its row blocks
* ``nccl_ag`` / ``nccl_rs``   the library collectives on the same buffers
* ``ag_gemm``       ONE kernel: push by the communication warps + GEMM with per-row-block waits
* ``gemm_rs``       ONE kernel: GEMM with row-block signals + reduction by the communication warps
* ``split_ag_gemm`` / ``split_gemm_rs``   the same pairs as two kernels on two streams (the default form)
* ``nccl_ag_gemm`` / ``nccl_gemm_rs``     library collective, then / after the plain GEMM
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def _time(fn, iters, warmup, device, group):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(1_000_000)          # the host enqueues fn() behind a short spin kernel: device time only
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ts)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--width", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--emulate-tp8", action="store_true", help="GEMM shapes of one rank of an 8-way split (short K, narrow N) whatever "
                    "the number of ranks: shows the cost of the row-block signals where the main loop is short")
    a = ap.parse_args(argv)
    from ..config import ModelConfig, ParallelConfig, TrainConfig
    from ..ops import comm as C
    from ..ops.fused_comm import FusedTP
    from ..ops.gemm import gemm_nt
    from ..parallel import state as PS
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    PS.init_distributed("nccl", 10)
    ps = PS.initialize_model_parallel(ParallelConfig(tp=world))
    rows, h = a.rows, a.width
    cfg = ModelConfig(hidden_size=h, seq_length=rows, num_attention_heads=h // 128, num_query_groups=h // 128)
    fused = FusedTP(ps, cfg, TrainConfig(micro_batch_size=1), dev, max_rows=rows, width=h)
    side = torch.cuda.Stream()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")))
    except Exception:
        pass
    gemm_peak = peaks.get("bf16_tflops", 1590.0) * 1e12
    out = []

    def emit(name, ms, link_bytes=0.0, flops=0.0, link_gbs=None, note=""):
        rec = {"path": name, "ms": round(ms, 4), "world": world, "rows": rows, "width": h}
        if link_bytes:
            rec["nvlink_bytes_per_gpu"] = int(link_bytes)
            rec["achieved_gbs"] = round(link_bytes / ms / 1e6, 1)
        if flops:
            rec["tflops"] = round(flops / ms / 1e9, 1)
        if link_gbs and (link_bytes or flops):
            bound = max(link_bytes / (link_gbs * 1e9), flops / gemm_peak) * 1e3
            rec["roofline_ms"] = round(bound, 4)
            rec["frac_of_roofline"] = round(bound / ms, 3)
        if note:
            rec["note"] = note
        out.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    # ---- link bandwidth: one GPU copies 1 GiB into its neighbour's symmetric buffer, all ranks at once (a ring of copies)
    nb = min(1 << 30, fused.buf.numel() // 2)
    peer = fused.hdl.get_buffer((rank + 1) % world, (nb,), torch.uint8, 0)
    src = torch.empty(nb, dtype=torch.uint8, device=dev)
    ms = _time(lambda: peer.copy_(src), a.iters, a.warmup, dev, ps.tp_group)
    link = nb / ms / 1e6
    emit("peer_copy", ms, link_bytes=nb, note="copy_ of %d MiB into the next rank's buffer, every rank at once" % (nb >> 20))

    shard = torch.randn(rows // world, h, device=dev).to(torch.bfloat16)
    full = torch.randn(rows, h, device=dev).to(torch.bfloat16)
    ag_bytes = (world - 1) / world * rows * h * 2            # bytes one GPU receives (= sends through the switch multicast)
    n_c, n_l = 1280 * 8 // world if world <= 8 else 1280, h  # column-parallel output width per rank (QKV), row-parallel output width
    if a.emulate_tp8:
        n_c = 1280
    w_c = (torch.randn(n_c, h, device=dev) * 0.02).to(torch.bfloat16)
    k_l = 1024 if a.emulate_tp8 else 1024 * 8 // world
    a_l = torch.randn(rows, k_l, device=dev).to(torch.bfloat16)
    w_l = (torch.randn(h, k_l, device=dev) * 0.02).to(torch.bfloat16)
    fl_c, fl_l = 2.0 * rows * n_c * h, 2.0 * rows * h * k_l

    # ---- stand-alone collectives
    emit("ag_push", _time(lambda: fused.all_gather(shard, "attn_c"), a.iters, a.warmup, dev, ps.tp_group), ag_bytes, 0, link)
    emit("nccl_ag", _time(lambda: C.gather_along_first_dim(shard, ps.tp_group), a.iters, a.warmup, dev, ps.tp_group), ag_bytes, 0, link)

    def rs_alone():
        part, sync = fused.partial_produce("attn_l", rows, h)
        gemm_nt(a_l, w_l, out=part, sync=sync)
        return fused.rs_reduce("attn_l")
    t_pair = _time(rs_alone, a.iters, a.warmup, dev, ps.tp_group)
    t_gemm_l = _time(lambda: gemm_nt(a_l, w_l), a.iters, a.warmup, dev, ps.tp_group)
    emit("gemm_row_parallel_alone", t_gemm_l, 0, fl_l, link, note="[%d, %d] x [%d, %d]^T, no collective" % (rows, k_l, h, k_l))
    emit("gemm_col_parallel_alone", _time(lambda: gemm_nt(full, w_c), a.iters, a.warmup, dev, ps.tp_group), 0, fl_c, link,
         note="[%d, %d] x [%d, %d]^T, no collective" % (rows, h, n_c, h))

    def into_symmetric():
        gemm_nt(a_l, w_l, out=fused.partial_buffer("head_bwd", rows, h))
    emit("gemm_row_parallel_into_symmetric", _time(into_symmetric, a.iters, a.warmup, dev, ps.tp_group), 0, fl_l, link,
         note="the same GEMM writing into the symmetric partial buffer, no signals, usual tile order")

    def owner_order_only():
        from ..ops.gemm import GemmSync
        gemm_nt(a_l, w_l, out=fused.partial_buffer("head_bwd", rows, h), sync=GemmSync(perm_mode=2, world=world, rank=rank))
    emit("gemm_row_parallel_owner_order", _time(owner_order_only, a.iters, a.warmup, dev, ps.tp_group), 0, fl_l, link,
         note="the same with the row-block-by-owner tile order and the 5-deep ring, still no signals")

    def signalling_gemm():
        part, sync = fused.partial_produce("attn_c_bwd", rows, h)
        gemm_nt(a_l, w_l, out=part, sync=sync)
    emit("gemm_row_parallel_signalling", _time(signalling_gemm, a.iters, a.warmup, dev, ps.tp_group), 0, fl_l, link,
         note="the same GEMM writing its partial product row block by row block over all owners and signalling each block")
    emit("rs_reduce", max(t_pair - t_gemm_l, 1e-3), ag_bytes, 0, link, note="GEMM + row-block reduction on one stream minus the GEMM alone")
    emit("nccl_rs", _time(lambda: C.reduce_scatter_along_first_dim(full, ps.tp_group), a.iters, a.warmup, dev, ps.tp_group), ag_bytes, 0, link)

    # ---- compute + collective
    emit("ag_gemm", _time(lambda: fused.ag_gemm(shard, w_c, "mlp_c"), a.iters, a.warmup, dev, ps.tp_group), ag_bytes, fl_c, link,
         note="one kernel")
    emit("gemm_rs", _time(lambda: fused.gemm_rs(a_l, w_l, "mlp_l"), a.iters, a.warmup, dev, ps.tp_group), ag_bytes, fl_l, link,
         note="one kernel")

    def split_ag():
        fused.gather_start(shard, "attn_l_bwd", stream=side)
        view, sync = fused.gather_consume("attn_l_bwd")
        return gemm_nt(view, w_c, sync=sync)
    emit("split_ag_gemm", _time(split_ag, a.iters, a.warmup, dev, ps.tp_group), ag_bytes, fl_c, link, note="push kernel beside a GEMM that waits per row block")

    def split_rs():
        part, sync = fused.partial_produce("mlp_c_bwd", rows, h)
        ev = torch.cuda.Event()
        ev.record()
        gemm_nt(a_l, w_l, out=part, sync=sync)
        side.wait_event(ev)
        with torch.cuda.stream(side):
            o = fused.rs_reduce("mlp_c_bwd")
        torch.cuda.current_stream().wait_stream(side)
        return o
    emit("split_gemm_rs", _time(split_rs, a.iters, a.warmup, dev, ps.tp_group), ag_bytes, fl_l, link, note="signalling GEMM beside the row-block reduction kernel")

    def nccl_ag_gemm():
        g, _ = C.gather_along_first_dim(shard, ps.tp_group)
        return gemm_nt(g, w_c)
    emit("nccl_ag_gemm", _time(nccl_ag_gemm, a.iters, a.warmup, dev, ps.tp_group), ag_bytes, fl_c, link)

    def nccl_gemm_rs():
        return C.reduce_scatter_along_first_dim(gemm_nt(a_l, w_l), ps.tp_group)
    emit("nccl_gemm_rs", _time(nccl_gemm_rs, a.iters, a.warmup, dev, ps.tp_group), ag_bytes, fl_l, link)

    torch.cuda.synchronize()
    from .. import kernels as K
    st = K.read_status()
    if rank == 0 and st.code != 0:
        print(json.dumps({"device_status": [st.code, st.where, st.extra]}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
