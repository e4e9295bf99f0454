"""Single-kernel benchmark with roofline fractions.

    python -m dhellam_b200.bench.kernel_bench --kernel gemm_nt --m 8192 --n 8192 --k 8192
    python -m dhellam_b200.bench.kernel_bench --kernel attn_fwd --seq 4096 --batch 2 --heads 8 --kv-heads 1
    python -m dhellam_b200.bench.kernel_bench --suite headline        # the per-GPU shapes of the TP8 headline run

Times with CUDA events on the launching stream after warm-up, flushes L2 between timed
launches (a 256 MiB buffer is overwritten), and reports achieved TFLOP/s or GB/s against the
measured peaks in ``MEASURED_PEAKS.json`` (copy bandwidth, cuBLAS bf16) when that file is
present, else against the stated fallback.  One JSON line per kernel.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def time_ms(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        # a short spin kernel in front of the first event: the host enqueues fn()'s launches while it runs, so the
        # events bracket device time only and not the host's launch path (which would otherwise sit inside the
        # bracket for every kernel shorter than its own launch sequence)
        torch.cuda._sleep(1_000_000)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def build(kernel, a):
    """Returns ``(closure, flops, bytes)``."""
    from ..ops import activation as A
    from ..ops import attention as ATT
    from ..ops import gemm as G
    from ..ops import loss as L
    from ..ops import norm as N
    M, Nn, Kd = a.m, a.n, a.k
    if kernel == "gemm_nt":
        x, w = bf(M, Kd), bf(Nn, Kd)
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda")
        return (lambda: G.gemm_nt(x, w, out=out, sm_budget=a.sm_budget)), 2.0 * M * Nn * Kd, 2.0 * (M * Kd + Nn * Kd + M * Nn)
    if kernel == "gemm_nn":
        dy, w = bf(M, Nn), bf(Nn, Kd)
        out = torch.empty(M, Kd, dtype=torch.bfloat16, device="cuda")
        return (lambda: G.gemm_nn(dy, w, out=out, sm_budget=a.sm_budget)), 2.0 * M * Nn * Kd, 2.0 * (M * Kd + Nn * Kd + M * Nn)
    if kernel == "gemm_tn":
        dy, x = bf(M, Nn), bf(M, Kd)
        g = torch.zeros(Nn, Kd, device="cuda")
        return (lambda: G.gemm_tn_acc(dy, x, g, sm_budget=a.sm_budget)), 2.0 * M * Nn * Kd, 2.0 * (M * Kd + M * Nn) + 8.0 * Nn * Kd
    if kernel == "torch_nt":
        x, w = bf(M, Kd), bf(Nn, Kd)
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda")
        return (lambda: torch.matmul(x, w.t(), out=out)), 2.0 * M * Nn * Kd, 2.0 * (M * Kd + Nn * Kd + M * Nn)
    if kernel == "torch_nn":
        dy, w = bf(M, Nn), bf(Nn, Kd)
        out = torch.empty(M, Kd, dtype=torch.bfloat16, device="cuda")
        return (lambda: torch.matmul(dy, w, out=out)), 2.0 * M * Nn * Kd, 2.0 * (M * Kd + Nn * Kd + M * Nn)
    if kernel == "torch_tn":        # the library's weight gradient: bf16 product, then added into the fp32 buffer
        dy, x = bf(M, Nn), bf(M, Kd)
        g = torch.zeros(Nn, Kd, device="cuda")
        return (lambda: g.add_(torch.matmul(dy.t(), x))), 2.0 * M * Nn * Kd, 2.0 * (M * Kd + M * Nn) + 8.0 * Nn * Kd
    if kernel in ("flash_fwd", "flash_bwd"):      # the flash-attn 2 package (or SDPA) on the same operands, for comparison
        from ..ops import library as LIB
        S, B, H, Hk, d = a.seq, a.batch, a.heads, a.kv_heads, 128
        qkv = bf(S, B, H + 2 * Hk, d)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hk], qkv[:, :, H + Hk:]
        fl = 4.0 * S * S * d * H * B * (0.5 if a.causal else 1.0)
        sc = 1.0 / d ** 0.5
        if kernel == "flash_fwd":
            return (lambda: LIB.attn_fwd(q, k, v, a.causal, sc)), fl, 2.0 * (qkv.numel() + S * B * H * d)
        o, lse = LIB.attn_fwd(q, k, v, a.causal, sc)
        do = bf(S, B, H, d)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :H], dqkv[:, :, H:H + Hk], dqkv[:, :, H + Hk:]
        return (lambda: LIB.attn_bwd(do, q, k, v, o, lse, dq, dk, dv, a.causal, sc)), 2.5 * fl, 2.0 * (3 * qkv.numel() + 2 * do.numel())
    if kernel in ("attn_fwd", "attn_bwd"):
        S, B, H, Hk, d = a.seq, a.batch, a.heads, a.kv_heads, 128
        qkv = bf(S, B, H + 2 * Hk, d)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hk], qkv[:, :, H + Hk:]
        fl = 4.0 * S * S * d * H * B * (0.5 if a.causal else 1.0)
        if kernel == "attn_fwd":
            return (lambda: ATT.attn_fwd(q, k, v, a.causal)), fl, 2.0 * (qkv.numel() + S * B * H * d)
        o, lse = ATT.attn_fwd(q, k, v, a.causal)
        do = bf(S, B, H, d)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :H], dqkv[:, :, H:H + Hk], dqkv[:, :, H + Hk:]
        # useful work: 5 products per tile pair (the kernels execute 7, two are recomputation)
        return (lambda: ATT.attn_bwd(do, q, k, v, o, lse, a.causal, dq=dq, dk=dk, dv=dv)), 2.5 * fl, 2.0 * (3 * qkv.numel() + 2 * do.numel())
    if kernel == "rmsnorm_fwd":
        x, w = bf(M, Nn), bf(Nn) + 1
        return (lambda: N.rmsnorm_fwd(x, w)), 0.0, 4.0 * M * Nn
    if kernel == "rmsnorm_bwd":
        x, w, dy = bf(M, Nn), bf(Nn) + 1, bf(M, Nn)
        _, rstd = N.rmsnorm_fwd(x, w)
        mg = torch.zeros(Nn, device="cuda")
        return (lambda: N.rmsnorm_bwd(dy, x, w, rstd, weight_main_grad=mg, residual_grad=dy)), 0.0, 8.0 * M * Nn
    if kernel == "swiglu_fwd":
        y = bf(M, 2 * Nn)
        return (lambda: A.swiglu_fwd(y)), 0.0, 6.0 * M * Nn
    if kernel == "swiglu_bwd":
        y, d = bf(M, 2 * Nn), bf(M, Nn)
        return (lambda: A.swiglu_bwd(d, y)), 0.0, 10.0 * M * Nn
    if kernel == "ce_stats":
        lg = bf(M, Nn, scale=3.0)
        lab = torch.randint(0, Nn, (M,), dtype=torch.int32, device="cuda")
        return (lambda: L.ce_local_stats(lg, lab, 0)), 0.0, 2.0 * M * Nn
    raise SystemExit(f"unknown kernel {kernel}")


# the per-GPU GEMM shapes of the 8-way tensor-parallel headline run, each followed by the library (cuBLAS through
# torch.matmul) on the same operands in the same call
_G = [("nt", dict(m=16384, n=1280, k=8192)), ("nt", dict(m=16384, n=8192, k=1024)), ("nt", dict(m=16384, n=7168, k=8192)),
      ("nt", dict(m=16384, n=8192, k=3584)), ("nn", dict(m=16384, n=7168, k=8192)), ("nn", dict(m=16384, n=1024, k=8192)),
      ("tn", dict(m=16384, n=7168, k=8192)), ("tn", dict(m=16384, n=8192, k=3584)), ("tn", dict(m=16384, n=1280, k=8192)),
      ("nt", dict(m=16384, n=16032, k=8192))]
HEADLINE = [(f"{lib}_{kind}", shape) for kind, shape in _G for lib in ("gemm", "torch")] + [
    ("attn_fwd", dict(seq=4096, batch=4, heads=8, kv_heads=1)), ("flash_fwd", dict(seq=4096, batch=4, heads=8, kv_heads=1)),
    ("attn_bwd", dict(seq=4096, batch=4, heads=8, kv_heads=1)), ("flash_bwd", dict(seq=4096, batch=4, heads=8, kv_heads=1)),
    ("rmsnorm_fwd", dict(m=2048, n=8192)), ("rmsnorm_bwd", dict(m=2048, n=8192)),
    ("swiglu_fwd", dict(m=16384, n=3584)), ("swiglu_bwd", dict(m=16384, n=3584)), ("ce_stats", dict(m=16384, n=16032)),
]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="gemm_nt")
    ap.add_argument("--suite", default=None, choices=[None, "headline"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=1)
    ap.add_argument("--causal", type=int, default=1)
    ap.add_argument("--sm-budget", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--gemm-mode", type=int, default=0, help="0 per problem, 1 single-CTA tiles, 2 CTA-pair tiles")
    a = ap.parse_args(argv)
    a.causal = bool(a.causal)
    hbm, tflops, src = peaks()
    if a.gemm_mode:
        from ..ops.gemm import set_gemm_mode
        set_gemm_mode(a.gemm_mode)
    flush = None if a.no_flush else torch.empty(256 * 1024 * 1024 // 4, device="cuda")
    jobs = HEADLINE if a.suite else [(a.kernel, {})]
    for kernel, over in jobs:
        b = argparse.Namespace(**{**vars(a), **over})
        try:
            fn, fl, by = build(kernel, b)
            ms = time_ms(fn, a.iters, a.warmup, flush)
        except Exception as e:                 # e.g. the flash-attn wheel has no kernel for this GPU
            print(json.dumps({"kernel": kernel, "shape": over, "error": f"{type(e).__name__}: {str(e)[:160]}"}), flush=True)
            continue
        rec = {"kernel": kernel, "shape": over or {k: getattr(a, k) for k in ("m", "n", "k", "seq", "batch", "heads", "kv_heads")},
               "ms": round(ms, 4), "l2": "flushed between launches" if flush is not None else "not flushed"}
        if fl:
            rec["tflops"] = round(fl / ms / 1e9, 1)
            rec[f"frac_of_{src}_cublas_bf16"] = round(fl / ms / 1e9 / tflops, 3)
        rec["gbs"] = round(by / ms / 1e6, 1)
        if not fl:
            rec[f"frac_of_{src}_copy_bw"] = round(by / ms / 1e6 / hbm, 3)
        print(json.dumps(rec), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
