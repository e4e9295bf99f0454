"""How much does a copy kernel that shares the GPU slow the persistent GEMM, by how the copy is spread over SMs
(a one-pair version of the reference's pairwise overlap matrix, micro_benchmark/overlap.py:1-227).

    python -m dhellam_b200.bench.corun_bench [M N K]
    python -m dhellam_b200.bench.corun_bench attn            # the attention forward (seq 4096, batch 4, 8 heads) instead of a GEMM

One GPU.  The copy is the all-gather push kernel (``dh_ag_push``) with both "ranks'" buffers in this GPU's
memory, run on a second stream for the whole duration of the GEMM; the GEMM is timed with CUDA events on
its own stream behind a spin kernel (device time only).  One JSON line per (copy CTAs, threads) pair: the
GEMM's time and slowdown against running alone, and the copy's own time per 268 MB.  The persistent GEMM
assigns tiles to CTAs statically, so a copy that occupies few SMs makes those SMs' CTAs the stragglers of
the whole GEMM; the table this prints is the reason the communication kernels run one CTA per SM.
"""
from __future__ import annotations

import json
import statistics
import sys
from ctypes import c_int, c_void_p

import torch

from .. import kernels as K
from ..ops.gemm import gemm_nt


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    dev = "cuda"
    M, N, Kd = 16384, 7168, 8192
    attn = bool(argv) and argv[0] == "attn"
    if len(argv) >= 3:
        M, N, Kd = (int(x) for x in argv[:3])
    if attn:
        from ..ops.attention import attn_fwd
        qkv = torch.randn(4096, 4, 10, 128, device=dev).to(torch.bfloat16)
        q, k, v = qkv[:, :, :8], qkv[:, :, 8:9], qkv[:, :, 9:]
        work = lambda: attn_fwd(q, k, v, True)
        label = {"kernel": "attn_fwd", "shape": [4096, 4, 8, 1]}
    else:
        a = (torch.randn(M, Kd, device=dev)).to(torch.bfloat16)
        w = (torch.randn(N, Kd, device=dev) * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        work = lambda: gemm_nt(a, w, out=out)
        label = {"kernel": "gemm_nt", "shape": [M, N, Kd]}
    rows, width = 16384, 8192
    shard = torch.randn(rows // 2, width, device=dev).to(torch.bfloat16)      # "rank 0 of 2": both ranks' buffers are local
    stage0 = torch.empty(rows, width, device=dev, dtype=torch.bfloat16)
    stage1 = torch.empty(rows, width, device=dev, dtype=torch.bfloat16)
    cnt0 = torch.zeros(1024, device=dev, dtype=torch.int32)
    cnt1 = torch.zeros(1024, device=dev, dtype=torch.int32)
    arr1 = (c_void_p * 2)(stage0.data_ptr(), stage1.data_ptr())
    arr2 = (c_void_p * 2)(cnt0.data_ptr(), cnt1.data_ptr())
    push = K.proto("dh_ag_push", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    slices_fn = K.proto("dh_comm_slices", [c_int, c_int, c_int])
    side = torch.cuda.Stream()

    def run(ctas, threads, iters=10):
        slices = slices_fn(rows // 2 // 128, width, ctas) if ctas else 0
        ts, tc = [], []
        for _ in range(iters + 3):
            torch.cuda.synchronize()
            torch.cuda._sleep(1_000_000)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if ctas:
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    c0.record()
                    for _ in range(3):     # keep the copy busy for the whole GEMM
                        K.check(push(shard.data_ptr(), arr1, arr2, None, rows, width, 0, 2, ctas, threads, slices, side.cuda_stream), "push")
                    c1.record()
            e0.record()
            work()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
            if ctas:
                tc.append(c0.elapsed_time(c1) / 3)
        return statistics.median(ts[3:]), (statistics.median(tc[3:]) if tc else 0.0)

    base, _ = run(0, 0)
    print(json.dumps(dict(label, alone_ms=round(base, 4))))
    for ctas, threads in ((16, 256), (32, 256), (64, 256), (148, 64), (148, 128), (148, 256)):
        t, c = run(ctas, threads)
        print(json.dumps({"copy_ctas": ctas, "copy_threads": threads, "kernel_ms": round(t, 4), "slowdown": round(t / base, 3),
                          "copy_ms_per_268MB": round(c, 4)}), flush=True)
    st = K.read_status()
    print(json.dumps({"status": st.code}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
