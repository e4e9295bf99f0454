"""Tensor-parallel collectives fused into the GEMM kernels over NVLink peer memory.

``FusedTP`` owns the symmetric memory of one tensor-parallel group (double-buffered
all-gather staging, double-buffered reduce-scatter partial slots, arrival counters) and
launches the two fused kernels of ``csrc/comm_fused.cu``:

* ``ag_gemm(shard, w)``  = ``all_gather(shard) @ op(w)`` and the gathered operand itself
  (kept for the weight gradient), replacing ``allgather_* + gemm_*`` of the reference
  (dhellam/core/dstb.py:412-425 + :80-107);
* ``gemm_rs(a, w)``      = ``reduce_scatter(a @ op(w))``, replacing ``gemm_* + reduce_scatter``
  (dstb.py:407-410).

Fused kernels wait on data that peers produce inside the *same* kernel, so two of them must
never run in a different order on different ranks.  Every launch is therefore chained to the
previous fused launch with an event, whichever stream it is on; other kernels still overlap
with them freely.

The peer pointers come from ``torch.distributed._symmetric_memory`` (one allocation, one
rendezvous); NCCL stays the transport of everything that is not a named fused path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_uint, c_void_p

import torch
import torch.distributed as dist

from .. import kernels as K


def _align(n, a=1024):
    return (n + a - 1) // a * a


class FusedTP:
    def __init__(self, ps, cfg, train, device, max_rows: int | None = None, width: int | None = None, copy_ctas: int = 16):
        import torch.distributed._symmetric_memory as symm_mem
        self.ps, self.device = ps, torch.device(device)
        self.world, self.rank = ps.tp, ps.tp_rank
        self.copy_ctas = copy_ctas
        rows = max_rows or train.micro_batch_size * cfg.seq_length // max(ps.cp, 1)
        width = width or cfg.hidden_size
        assert rows % (self.world * 128) == 0, "rows per micro-batch must divide by tp x 128 for the fused kernels"
        self.rows, self.width = rows, width
        self.blocks = rows // 128
        stage_bytes = rows * width * 2
        cnt_bytes = _align(max(self.blocks, self.world) * 4)
        # layout: [stage0 | stage1 | part0 | part1 | ag_cnt0 | ag_cnt1 | rs_cnt0 | rs_cnt1]
        self.off_stage = [0, stage_bytes]
        self.off_part = [2 * stage_bytes, 3 * stage_bytes]
        base = 4 * stage_bytes
        self.off_agc = [base, base + cnt_bytes]
        self.off_rsc = [base + 2 * cnt_bytes, base + 3 * cnt_bytes]
        total = base + 4 * cnt_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        group = ps.tp_group
        self.hdl = symm_mem.rendezvous(self.buf, group=group.group_name)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        assert len(self.ptrs) == self.world
        self.buf[base:].zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)                 # nobody pushes before every rank's counters are zero
        self.total_ag = [0, 0]          # counter value every row block of the slot has reached so far
        self.total_rs = [0, 0]          # arrival count per source the slot has reached so far
        self.n_ag = self.n_rs = 0
        self._last = None
        self._arr = ctypes.c_void_p * self.world

    # ------------------------------------------------------------------ helpers
    def _ptr_array(self, off):
        return self._arr(*[p + off for p in self.ptrs])

    def _chain(self):
        s = torch.cuda.current_stream(self.device)
        if self._last is not None:
            s.wait_event(self._last)
        return s

    def _done(self, s):
        ev = torch.cuda.Event()
        ev.record(s)
        self._last = ev

    # ------------------------------------------------------------------ fused ops
    def ag_gemm(self, shard, w, tag: str = "", transpose_w: bool = False, sm_budget: int = 0, save: bool = True):
        """``shard [M/t, K]``; ``w [N, K]`` (or ``[K, N']`` with ``transpose_w``: the product is
        ``gathered @ w``).  Returns ``(out [M, N], gathered [M, K] or None)``."""
        rows_local, Kd = shard.shape
        M = rows_local * self.world
        assert M == self.rows, "the fused all-gather works on full micro-batches (fixed row count per group)"
        assert Kd <= self.width and shard.dtype == torch.bfloat16 and shard.is_contiguous()
        if transpose_w:
            assert w.shape[0] == Kd
            N = w.shape[1]
        else:
            assert w.shape[1] == Kd
            N = w.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        saved = torch.empty((M, Kd), dtype=torch.bfloat16, device=self.device) if save else None
        slot = self.n_ag & 1
        self.n_ag += 1
        before = self.total_ag[slot]
        slices = K.proto("dh_ag_gemm_slices", [c_int, c_int, c_int, c_int, c_int])(M, Kd, self.world, self.copy_ctas, int(sm_budget))
        self.total_ag[slot] = before + slices
        s = self._chain()
        fn = K.proto("dh_ag_gemm_bf16", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int,
                                          c_int, c_int, c_int, c_int, c_int, c_uint, c_int, c_void_p])
        K.check(fn(shard.data_ptr(), self._ptr_array(self.off_stage[slot]), self._ptr_array(self.off_agc[slot]), K.ptr(saved),
                   w.data_ptr(), w.stride(0), int(transpose_w), out.data_ptr(), out.stride(0), M, N, Kd, self.rank, self.world,
                   self.copy_ctas, before, int(sm_budget), s.cuda_stream), "dh_ag_gemm_bf16")
        self._done(s)
        return out, saved

    def gemm_rs(self, a, w, tag: str = "", transpose_w: bool = False, sm_budget: int = 0):
        """``a [M, K]``; returns this rank's ``[M/t, N]`` shard of ``sum_ranks(a @ op(w))``."""
        M, Kd = a.shape
        assert M == self.rows and a.dtype == torch.bfloat16 and a.stride(1) == 1
        if transpose_w:
            assert w.shape[0] == Kd
            N = w.shape[1]
        else:
            assert w.shape[1] == Kd
            N = w.shape[0]
        assert N <= self.width
        out = torch.empty((M // self.world, N), dtype=torch.bfloat16, device=self.device)
        slot = self.n_rs & 1
        self.n_rs += 1
        before = self.total_rs[slot]
        self.total_rs[slot] = before + (M // self.world // 128) * ((N + 255) // 256) * 4
        s = self._chain()
        fn = K.proto("dh_gemm_rs_bf16", [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_int, c_int, c_uint, c_int, c_void_p])
        K.check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), int(transpose_w), self._ptr_array(self.off_part[slot]),
                   self._ptr_array(self.off_rsc[slot]), out.data_ptr(), M, N, Kd, self.rank, self.world, before,
                   int(sm_budget), s.cuda_stream), "dh_gemm_rs_bf16")
        self._done(s)
        return out
