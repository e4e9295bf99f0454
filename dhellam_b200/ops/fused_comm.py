"""Tensor-parallel (and context-parallel) collectives over NVLink peer memory.

``FusedTP`` owns the symmetric memory of one tensor-parallel group and launches the kernels of
``csrc/comm_fused.cu`` and the collective forms of the GEMM in ``csrc/gemm_sm100.cu``:

* ``gather_start(shard, tag)`` pushes this rank's rows into every rank's staging buffer from a few CTAs
  on the communication stream and raises per-128-row-block arrival counters; ``gather_consume(tag)``
  hands the consuming GEMM the staged operand plus a ``GemmSync`` that makes the kernel wait per row
  block (own rows first); ``gather_wait(tag)`` is the whole-buffer wait in front of any other consumer.
  Also used to re-gather the sequence-parallel input of a column-parallel layer for its weight gradient
  instead of keeping the gathered activation alive from the forward pass.  Replaces ``allgather_*``
  of the reference (dhellam/core/dstb.py:412-425, dhellam/operators/comm.py:13-33).
* ``partial_produce(tag, M, N)`` gives the producing GEMM a symmetric partial buffer plus a ``GemmSync``
  that makes it write row block by row block over all owners and signal each finished block to its owner;
  ``rs_reduce(tag)`` launches the reduction that follows those signals (in-switch ``multimem.ld_reduce`` or
  peer loads) and may be launched as soon as the GEMM has been launched.  ``partial_buffer`` /
  ``rs_reduce`` without signals is the whole-buffer form.  Replaces ``reduce_scatter_*``
  (dstb.py:407-410, comm.py:35-58).
* ``ag_gemm(shard, w, tag)`` / ``gemm_rs(a, w, tag)``: the same two pairs as ONE kernel each, with the push /
  reduction carried by communication warps inside every GEMM CTA (policy ``fused``).

``split(M, N, K)`` says per call site which form the layer ops use (``DHELLAM_FUSED_POLICY``).

Every staging / partial buffer is double-buffered per tag, with monotonically increasing counters (no resets,
no host barriers).  Kernels that wait for peers inside the kernel (``ag_gemm``, ``gemm_rs``) are chained to one
another with events so that all ranks run them one at a time in the same order; pure pushes wait for nobody.

The NVSwitch multicast address of the buffer is used for the in-switch reduction whenever the platform
provides it, and for the push on 4 or more GPUs (``DHELLAM_MULTIMEM``, ``DHELLAM_MULTIMEM_PUSH``).  Peer
pointers come from ``torch.distributed._symmetric_memory`` (one allocation, one rendezvous).

``FusedCP`` is the context-parallel counterpart: key/value chunks pushed into global order in every rank's
buffer, per-chunk arrival waits, partial dK|dV reduced by the chunk owners (role of the reference's ring,
dhellam/operators/ring_attn.py:43-201, without its per-step exchanges).  ``SimulatedCP`` runs the same data
flow on library collectives for the CPU tests.
"""
from __future__ import annotations

import collections
import contextlib
import ctypes
import os
from ctypes import c_int, c_int64, c_uint, c_void_p

import torch
import torch.distributed as dist

from .. import kernels as K

AG_TAGS = ("attn_c", "mlp_c", "attn_l_bwd", "mlp_l_bwd", "regather_attn", "regather_mlp", "head", "embed_bwd")
RS_TAGS = ("attn_l", "mlp_l", "mlp_c_bwd", "attn_c_bwd", "head_bwd", "embed")


def _align(n, a=1024):
    return (n + a - 1) // a * a


class FusedTP:
    def __init__(self, ps, cfg, train, device, max_rows: int | None = None, width: int | None = None, copy_ctas: int = 0,
                 push_ctas: int = 0):
        import torch.distributed._symmetric_memory as symm_mem
        self.ps, self.device = ps, torch.device(device)
        self.world, self.rank = ps.tp, ps.tp_rank
        # the shard a rank pushes is 1/tp of the operand: fewer ranks -> more bytes per rank -> more copy CTAs
        self.sms = K.lib().dh_sm_count()
        # Stand-alone communication kernels: a few 256-thread CTAs (16 on 8 GPUs).  Measured alone, more is better: a
        # persistent GEMM deals its tiles to CTAs statically, so a copy kernel on 16 SMs makes those 16 CTAs the
        # stragglers of the whole GEMM (one GPU, copy beside the FC1-shaped GEMM: +24 % with 16 copy CTAs, +7 % with
        # one per SM, and the copy itself 3x faster).  Measured in the training step on 8 GPUs (same call) it is the
        # other way round: 16 CTAs 146.4k tokens/s, one CTA per SM 142.2k.  Why is not known (the attention forward
        # beside the same copy loses only 5 % on one GPU, so it is not that kernel being kept off the SMs); the step
        # decides the default.  DHELLAM_PUSH_CTAS / DHELLAM_RS_CTAS set the counts; DHELLAM_COMM_SPREAD=1 selects one
        # 64-thread CTA per SM (not yet measured in the step on 8 GPUs).
        spread = os.environ.get("DHELLAM_COMM_SPREAD", "0") == "1"
        self.comm_threads = 64 if spread else 256
        self.push_ctas = push_ctas or int(os.environ.get("DHELLAM_PUSH_CTAS", "0")) or (self.sms if spread else max(16, 96 // self.world))
        rows = max_rows or train.micro_batch_size * cfg.seq_length // max(ps.cp, 1)
        width = width or cfg.hidden_size
        assert rows % (self.world * 128) == 0, "rows per micro-batch must divide by tp x 128 for the fused kernels"
        self.rows, self.width = rows, width
        self.blocks = rows // 128
        stage_bytes = rows * width * 2
        cnt_bytes = _align(max(self.blocks, self.world) * 4)
        # layout: AG staging (tag x 2) | AG counters (tag x 2) | RS counters / flags (tag x 2) | RS partial products (tag x 2)
        self.off_stage, self.off_agc = {}, {}
        off = 0
        for t in AG_TAGS:
            self.off_stage[t] = [off, off + stage_bytes]
            off += 2 * stage_bytes
        cnt_base = off
        for t in AG_TAGS:
            self.off_agc[t] = [off, off + cnt_bytes]
            off += 2 * cnt_bytes
        self.off_rsflag = {}
        for t in RS_TAGS:
            self.off_rsflag[t] = [off, off + cnt_bytes]
            off += 2 * cnt_bytes
        self.off_split = {}
        for t in RS_TAGS:                       # partial products of the split reduce-scatter, [rows, width] each
            self.off_split[t] = [off, off + stage_bytes]
            off += 2 * stage_bytes
        cnt_end = self.off_split[RS_TAGS[0]][0]
        self.buf = symm_mem.empty(off, dtype=torch.uint8, device=self.device)
        group = ps.tp_group
        self.hdl = symm_mem.rendezvous(self.buf, group=group.group_name)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        assert len(self.ptrs) == self.world
        mc = 0
        if os.environ.get("DHELLAM_MULTIMEM", "1") != "0":
            try:
                mc = int(self.hdl.multicast_ptr or 0)
            except Exception:
                mc = 0
        self.mc_ptr = mc
        e = os.environ.get("DHELLAM_MULTIMEM_PUSH", "")
        self.mc_push = (e != "0") if e else self.world >= 4
        self.buf[cnt_base:cnt_end].zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)                 # nobody pushes before every rank's counters are zero
        self.total_ag = {t: [0, 0] for t in AG_TAGS}     # counter value reached so far, per (tag, parity)
        self.calls_ag = {t: 0 for t in AG_TAGS}
        self._last = None
        self._arr = ctypes.c_void_p * self.world
        self._pending = {}
        self.calls_split = {t: 0 for t in RS_TAGS}
        self._split_pending = {}
        self._split_sync = {}
        self._start_flag = None
        # "split" (default): every collective is its own small kernel on the communication stream, beside a
        # GEMM that waits per row block / signals finished row blocks, so that the schedule hides the transfer
        # behind the other strand's kernels too; "fused": every collective inside its GEMM kernel (communication
        # warps), overlapped tile by tile with that GEMM only; "auto": split while both strands are live, fused
        # in the warm-up and cool-down rounds.  Measured on 8 GPUs (tokens/s, headline model, one process):
        # split 139.5k, fused 130.8k, library collectives 137.0k; on 2 GPUs split and fused are within 1 %.
        self.policy = os.environ.get("DHELLAM_FUSED_POLICY", "split")
        self.paired = True                # set by the engine before every layer run
        self.rs_ctas = int(os.environ.get("DHELLAM_RS_CTAS", "0")) or (self.sms if spread else max(16, 128 // self.world))
        self.exposed = None               # the engine's ExposedTimer (set by the trainer); None = no measurement
        # Tile-granular overlap between a GEMM and the collective beside it (split policy):
        #   DHELLAM_AG_INKERNEL=1  the GEMM that consumes a gathered operand waits per 128-row block inside the kernel
        #                          (own rows first) instead of behind a whole-buffer wait kernel;
        #   DHELLAM_RS_BLOCKS=1    the GEMM that produces a partial product signals every finished row block to its
        #                          owner, whose reduction kernel starts on a block as soon as all ranks delivered it.
        # (not with two compute streams: a GEMM that spins on arrival counters holds every SM's shared memory, so the
        #  other strand's GEMM, whose output some peer's push may be waiting for, could never start)
        self.ag_inkernel = os.environ.get("DHELLAM_AG_INKERNEL", "1") != "0" and getattr(train, "compute_streams", 1) < 2
        self.rs_blocks = os.environ.get("DHELLAM_RS_BLOCKS", "1") != "0" and getattr(train, "compute_streams", 1) < 2
        self.total_sig = {t: [0, 0] for t in RS_TAGS}      # block-counter value reached so far, per (tag, slot)
        self._sig_arrays = {}
        # The strategy search replays single ops out of their layer context (a consumer without its push, a
        # reduction without its GEMM).  In lenient mode such a call works on the slot's last contents with the
        # counter value already reached, so it measures the kernel without waiting; training never sets it.
        self.lenient = False

    def split(self, M: int, N: int, Kd: int) -> bool:
        """Whether the collective beside the GEMM ``[M, Kd] x [Kd, N]`` runs as its own kernel."""
        if self.policy == "split":
            return True
        if self.policy == "fused":
            return False
        return self.paired

    # ------------------------------------------------------------------ helpers
    def _ptr_array(self, off):
        return self._arr(*[p + off for p in self.ptrs])

    def _mc(self, off):
        return (self.mc_ptr + off) if self.mc_ptr else 0

    def _mc_push(self, off):
        """Multicast alias for the all-gather push, or 0 for per-peer stores.  A multicast store also returns the
        sender's own rows through the switch, so a GPU receives world/(world-1) times the bytes of per-peer stores:
        twice as many on 2 GPUs (measured there: 0.64 ms multicast, 0.53 ms per-peer for 134 MB), 1.14x on 8,
        where one store instead of seven is worth it."""
        return (self.mc_ptr + off) if (self.mc_ptr and self.mc_push) else 0

    def _stage_view(self, tag, slot, M, Kd):
        off = self.off_stage[tag][slot]
        return self.buf[off:off + M * Kd * 2].view(torch.bfloat16).view(M, Kd)

    def _chain(self):
        s = torch.cuda.current_stream(self.device)
        if self._last is not None:
            s.wait_event(self._last)
        return s

    def _done(self, s):
        ev = torch.cuda.Event()
        ev.record(s)
        self._last = ev

    def _slices(self, blocks: int, width: int, groups: int) -> int:
        """Column slices per 128-row block such that (blocks x slices) work items keep ``groups`` thread groups busy."""
        return K.proto("dh_comm_slices", [c_int, c_int, c_int])(int(blocks), int(width), int(groups))

    def _next_ag(self, tag, M, Kd, groups: int):
        """Reserves the next staging slot of ``tag``.  Returns ``(slot, counter value before, slices)``; every
        row-block counter of the slot rises by ``slices`` in this call."""
        slot = self.calls_ag[tag] & 1
        self.calls_ag[tag] += 1
        before = self.total_ag[tag][slot]
        slices = self._slices(M // self.world // 128, Kd, groups)
        self.total_ag[tag][slot] = before + slices
        return slot, before, slices

    # ------------------------------------------------------------------ fused ops
    def ag_gemm(self, shard, w, tag: str, transpose_w: bool = False, sm_budget: int = 0):
        """``shard [M/t, K]``; ``w [N, K]`` (or ``[K, N']`` with ``transpose_w``: the product is
        ``gathered @ w``).  ONE kernel: the communication warps of the CTA-pair GEMM push the shard
        to every rank while its tensor-core warps multiply the staged operand, own rows first.
        Returns ``(out [M, N], gathered [M, K] view of the staging buffer)``."""
        rows_local, Kd = shard.shape
        M = rows_local * self.world
        assert M == self.rows, "the fused all-gather works on full micro-batches (fixed row count per group)"
        assert Kd == self.width and shard.dtype == torch.bfloat16 and shard.is_contiguous()
        N = w.shape[1] if transpose_w else w.shape[0]
        assert (w.shape[0] if transpose_w else w.shape[1]) == Kd
        out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        slot, before, slices = self._next_ag(tag, M, Kd, self.sms)
        s = self._chain()
        fn = K.proto("dh_ag_gemm_bf16", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int,
                                          c_int, c_int, c_int, c_int, c_int, c_uint, c_int, c_void_p])
        K.check(fn(shard.data_ptr(), self._ptr_array(self.off_stage[tag][slot]), self._ptr_array(self.off_agc[tag][slot]),
                   self._mc_push(self.off_stage[tag][slot]), w.data_ptr(), w.stride(0), int(transpose_w), out.data_ptr(), out.stride(0),
                   M, N, Kd, self.rank, self.world, slices, before, int(sm_budget), s.cuda_stream), "dh_ag_gemm_bf16")
        self._done(s)
        return out, self._stage_view(tag, slot, M, Kd)

    def gemm_rs(self, a, w, tag: str = "attn_l", transpose_w: bool = False, sm_budget: int = 0):
        """``a [M, K]``; returns this rank's ``[M/t, N]`` shard of ``sum_ranks(a @ op(w))``.  ONE kernel:
        the tensor-core warps write and signal the partial product row block by row block, the
        communication warps reduce this rank's rows as the blocks complete on all ranks."""
        M, Kd = a.shape
        assert M == self.rows and a.dtype == torch.bfloat16 and a.stride(1) == 1
        N = w.shape[1] if transpose_w else w.shape[0]
        assert (w.shape[0] if transpose_w else w.shape[1]) == Kd and N <= self.width and tag in self.off_split
        out = torch.empty((M // self.world, N), dtype=torch.bfloat16, device=self.device)
        slot = self.calls_split[tag] & 1
        self.calls_split[tag] += 1
        self.total_sig[tag][slot] += self.world * ((N + 255) // 256)      # every rank: one signal per tile column
        target = self.total_sig[tag][slot]
        off = self.off_split[tag][slot]
        s = self._chain()
        fn = K.proto("dh_gemm_rs_bf16", [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_int, c_int, c_int, c_uint, c_int, c_void_p])
        K.check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), int(transpose_w), self._ptr_array(off), self._mc(off),
                   self._ptr_array(self.off_rsflag[tag][slot]), out.data_ptr(), M, N, Kd, self.rank, self.world, target,
                   int(sm_budget), s.cuda_stream), "dh_gemm_rs_bf16")
        self._done(s)
        return out

    # ------------------------------------------------------------------ stand-alone gather
    def gather_start(self, shard, tag: str, stream=None):
        """Starts pushing ``shard [M/t, K]`` to every rank (on ``stream`` if given, else the
        current one).  ``gather_wait(tag)`` on the consumer's stream returns the gathered view."""
        rows_local, Kd = shard.shape
        M = rows_local * self.world
        assert M == self.rows and Kd == self.width and shard.dtype == torch.bfloat16 and shard.is_contiguous()
        slot, before, slices = self._next_ag(tag, M, Kd, self.push_ctas)
        cur = torch.cuda.current_stream(self.device)
        s = stream if stream is not None else cur
        if s is not cur:
            s.wait_stream(cur)
            shard.record_stream(s)
        fn = K.proto("dh_ag_push", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
        K.check(fn(shard.data_ptr(), self._ptr_array(self.off_stage[tag][slot]), self._ptr_array(self.off_agc[tag][slot]),
                   self._mc_push(self.off_stage[tag][slot]), M, Kd, self.rank, self.world, self.push_ctas, self.comm_threads, slices,
                   s.cuda_stream), "dh_ag_push")
        ev = torch.cuda.Event()
        ev.record(s)
        self._pending.setdefault(tag, collections.deque()).append((slot, self.total_ag[tag][slot], M, Kd, ev))

    def gather_wait(self, tag: str):
        if self.lenient and not self._pending.get(tag):
            slot = (self.calls_ag[tag] - 1) & 1 if self.calls_ag[tag] else 0
            return self._stage_view(tag, slot, self.rows, self.width)
        slot, target, M, Kd, ev = self._pending[tag].popleft()     # oldest first: a weight gradient may trail by one layer
        s = torch.cuda.current_stream(self.device)
        ctx = self.exposed.span(s) if (self.exposed is not None and self.exposed.enabled) else contextlib.nullcontext()
        with ctx:                        # the consumer's stream stands still until every rank's rows have arrived
            s.wait_event(ev)
            fn = K.proto("dh_wait_counters", [c_void_p, c_int, c_uint, c_int64, c_void_p])
            K.check(fn(self.ptrs[self.rank] + self.off_agc[tag][slot], M // 128, target, 0, s.cuda_stream), "dh_wait_counters")
        return self._stage_view(tag, slot, M, Kd)

    def gather_consume(self, tag: str):
        """For a GEMM that reads the gathered operand of ``tag`` as its A matrix: returns
        ``(view, GemmSync or None)``.  With in-kernel waiting the kernel itself waits per 128-row
        block for the arrival counters (own rows first); otherwise a whole-buffer wait kernel is
        launched in front (also while exposed communication is being measured, so that the waiting
        time shows up between events: an upper bound of what the in-kernel form exposes)."""
        measuring = self.exposed is not None and self.exposed.enabled
        if not self.ag_inkernel or measuring:
            return self.gather_wait(tag), None
        from .gemm import GemmSync
        if self.lenient and not self._pending.get(tag):
            slot = (self.calls_ag[tag] - 1) & 1 if self.calls_ag[tag] else 0
            return self._stage_view(tag, slot, self.rows, self.width), None
        slot, target, M, Kd, ev = self._pending[tag].popleft()
        sync = GemmSync(wait_count=self.ptrs[self.rank] + self.off_agc[tag][slot], wait_target=target, perm_mode=1,
                        world=self.world, rank=self.rank)
        return self._stage_view(tag, slot, M, Kd), sync

    def all_gather(self, shard, tag: str):
        self.gather_start(shard, tag)
        return self.gather_wait(tag)

    # ------------------------------------------------------------------ stand-alone reduce-scatter
    def partial_buffer(self, tag: str, M: int, N: int):
        """Symmetric-memory tensor ``[M, N]`` for this rank's partial product of ``tag``; the GEMM
        writes it, ``rs_reduce(tag)`` then returns this rank's rows of the sum over ranks."""
        assert M == self.rows and N <= self.width and tag in self.off_split
        slot = self.calls_split[tag] & 1
        self.calls_split[tag] += 1
        off = self.off_split[tag][slot]
        self._split_pending[tag] = (slot, (self.calls_split[tag] + 1) // 2, M, N, None)
        return self.buf[off:off + M * N * 2].view(torch.bfloat16).view(M, N)

    def partial_produce(self, tag: str, M: int, N: int):
        """Like ``partial_buffer`` but for a GEMM that signals finished row blocks: returns
        ``(buffer, GemmSync or None)``; ``rs_reduce(tag)`` then runs the row-block-wise reduction,
        which may be launched as soon as the GEMM has been launched."""
        buf = self.partial_buffer(tag, M, N)
        if not self.rs_blocks or (M // self.world) % 128 != 0:
            return buf, None
        from .gemm import GemmSync
        slot, use, _, _, _ = self._split_pending[tag]
        tiles_n = (N + 255) // 256
        self.total_sig[tag][slot] += self.world * tiles_n           # every rank: one signal per tile column
        target = self.total_sig[tag][slot]
        key = (tag, slot)
        if key not in self._sig_arrays:
            self._sig_arrays[key] = self._ptr_array(self.off_rsflag[tag][slot])
        sync = GemmSync(sig_ptrs=self._sig_arrays[key], sig_bpr=M // self.world // 128, perm_mode=2, world=self.world, rank=self.rank)
        self._split_pending[tag] = (slot, use, M, N, target)
        self._split_sync[tag] = sync
        return buf, sync

    def rs_reduce(self, tag: str):
        """Runs on the current stream, which must already wait for the GEMM that filled the buffer."""
        if self.lenient and tag not in self._split_pending:
            slot = (self.calls_split[tag] - 1) & 1 if self.calls_split[tag] else 0
            self._split_pending[tag] = (slot, 0, self.rows, self.width, self.total_sig[tag][slot])
        slot, use, M, N, block_target = self._split_pending.pop(tag)
        out = torch.empty((M // self.world, N), dtype=torch.bfloat16, device=self.device)
        s = torch.cuda.current_stream(self.device)
        if block_target is not None:
            sync = self._split_sync.pop(tag, None)
            if sync is not None and sync.start_id:
                # The reduction spins on the GEMM's row-block signals and may be launched while that GEMM has not
                # started: a one-CTA wait in front of it holds this stream until every CTA of the GEMM is resident,
                # so the spinning CTAs can never keep a CTA pair of the GEMM (static tile assignment) off its SMs.
                if self._start_flag is None:
                    self._start_flag = K.proto("dh_gemm_start_flag_ptr", [], c_void_p)()
                wfn = K.proto("dh_wait_counters", [c_void_p, c_int, c_uint, c_int64, c_void_p])
                K.check(wfn(self._start_flag, 1, sync.start_id, 0, s.cuda_stream), "dh_wait_counters")
            fn = K.proto("dh_rs_reduce_blocks", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_uint, c_int, c_int,
                                                  c_void_p])
            off = self.off_split[tag][slot]
            K.check(fn(self._ptr_array(off), self._mc(off), self.ptrs[self.rank] + self.off_rsflag[tag][slot], out.data_ptr(), M, N,
                       self.rank, self.world, block_target, self.rs_ctas, self.comm_threads, s.cuda_stream), "dh_rs_reduce_blocks")
            return out
        fn = K.proto("dh_rs_reduce", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_uint, c_int, c_void_p])
        off = self.off_split[tag][slot]
        K.check(fn(self._ptr_array(off), self._mc(off), self._ptr_array(self.off_rsflag[tag][slot]), out.data_ptr(), M, N, self.rank,
                   self.world, use, self.rs_ctas, s.cuda_stream), "dh_rs_reduce")
        return out


class FusedCP:
    """Context-parallel key/value exchange over NVLink peer memory (one instance per context-parallel group).

    The reference moves KV blocks around a ring with ``batch_isend_irecv`` and merges per-step partial
    outputs through the log-sum-exp (dhellam/operators/ring_attn.py:43-201); its backward sends the KV
    block and a travelling dKV accumulator around the ring (:204-411).  NVSwitch gives every GPU full
    bandwidth to every peer, so a ring buys nothing here: every rank PUSHES its two sequence chunks
    straight to their places in every peer's key/value buffer (global sequence order; ``multimem.st`` or
    per-peer stores, bf16, per-128-row-block arrival counters), and each of a rank's two query chunks
    then runs ONE causal attention call over the keys it may see: no per-step outputs, no merges.  In
    the backward every rank writes its dK/dV contributions for all keys into its own symmetric buffer
    and each owner reduces its two chunks over the ranks (``multimem.ld_reduce``: fp32 adds inside the
    switch, or peer loads).

    Sites are double-buffered with monotonically increasing counters like ``FusedTP``.
    """
    SITES = ("kv_fwd", "kv_bwd")

    def __init__(self, ps, cfg, train, device, batch: int | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.ps, self.device = ps, torch.device(device)
        self.world, self.rank = ps.cp, ps.cp_rank
        B = batch or train.micro_batch_size
        nkv = max(cfg.num_query_groups // ps.tp, 1)
        self.width = 2 * nkv * cfg.head_dim                     # one row: K heads then V heads
        self.chunk_rows = cfg.seq_length // (2 * self.world) * B  # rows (sequence position x batch) per chunk
        assert self.chunk_rows % 128 == 0, "sequence chunk x micro-batch must be a multiple of 128 rows for the peer-memory exchange"
        self.chunk_blocks = self.chunk_rows // 128
        self.total_rows = 2 * self.world * self.chunk_rows
        self.total_blocks = 2 * self.world * self.chunk_blocks
        buf_bytes = self.total_rows * self.width * 2
        cnt_bytes = _align((self.total_blocks + 8) * 4)
        self.off_buf, self.off_cnt = {}, {}
        off = 0
        for s in self.SITES + ("dkv",):
            self.off_buf[s] = [off, off + buf_bytes]
            off += 2 * buf_bytes
        cnt_base = off
        for s in self.SITES + ("dkv",):
            self.off_cnt[s] = [off, off + cnt_bytes]
            off += 2 * cnt_bytes
        self.buf = symm_mem.empty(off, dtype=torch.uint8, device=self.device)
        group = ps.cp_group
        self.hdl = symm_mem.rendezvous(self.buf, group=group.group_name)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        mc = 0
        if os.environ.get("DHELLAM_MULTIMEM", "1") != "0":
            try:
                mc = int(self.hdl.multicast_ptr or 0)
            except Exception:
                mc = 0
        self.mc_ptr = mc
        self.buf[cnt_base:off].zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        self.calls = {s: 0 for s in self.SITES + ("dkv",)}
        self.total = {s: [0, 0] for s in self.SITES + ("dkv",)}
        self._arr = ctypes.c_void_p * self.world
        self.ctas = max(16, 96 // self.world)
        self.exposed = None

    def chunk_ids(self):
        """The two sequence chunks this rank holds (local rows: first half, second half)."""
        return self.rank, 2 * self.world - 1 - self.rank

    def _ptr_array(self, off):
        return self._arr(*[p + off for p in self.ptrs])

    def _mc(self, off):
        return (self.mc_ptr + off) if self.mc_ptr else 0

    def view(self, site: str, slot: int):
        off = self.off_buf[site][slot]
        return self.buf[off:off + self.total_rows * self.width * 2].view(torch.bfloat16).view(self.total_rows, self.width)

    def push_kv(self, kv_rows, site: str, stream=None):
        """``kv_rows [2 * chunk_rows, width]`` (row stride free): this rank's K|V rows, first chunk then second.
        Starts pushing both chunks to their global places on every rank; returns ``(slot, target)``."""
        assert kv_rows.shape == (2 * self.chunk_rows, self.width) and kv_rows.stride(1) == 1 and kv_rows.dtype == torch.bfloat16
        slot = self.calls[site] & 1
        self.calls[site] += 1
        slices = K.proto("dh_comm_slices", [c_int, c_int, c_int])(self.chunk_blocks, self.width, self.ctas)
        self.total[site][slot] += slices
        cur = torch.cuda.current_stream(self.device)
        s = stream if stream is not None else cur
        if s is not cur:
            s.wait_stream(cur)
            kv_rows.record_stream(s)
        fn = K.proto("dh_push_blocks", [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p])
        off, coff = self.off_buf[site][slot], self.off_cnt[site][slot]
        for half, chunk in enumerate(self.chunk_ids()):
            src = kv_rows[half * self.chunk_rows:]
            K.check(fn(src.data_ptr(), kv_rows.stride(0), self._ptr_array(off), self._ptr_array(coff), self._mc(off), self.width,
                       self.chunk_blocks, chunk * self.chunk_blocks, self.rank, self.world, self.ctas, 256, slices, s.cuda_stream),
                    "dh_push_blocks")
        return slot, self.total[site][slot]

    def wait_kv(self, site: str, slot: int, target: int, n_chunks: int):
        """Makes the current stream wait (bounded) until the first ``n_chunks`` chunks have arrived; returns
        the gathered ``[total_rows, width]`` view."""
        s = torch.cuda.current_stream(self.device)
        ctx = self.exposed.span(s) if (self.exposed is not None and self.exposed.enabled) else contextlib.nullcontext()
        with ctx:
            fn = K.proto("dh_wait_counters", [c_void_p, c_int, c_uint, c_int64, c_void_p])
            K.check(fn(self.ptrs[self.rank] + self.off_cnt[site][slot], n_chunks * self.chunk_blocks, target, 0, s.cuda_stream),
                    "dh_wait_counters")
        return self.view(site, slot)

    def dkv_buffer(self):
        """This rank's partial dK|dV buffer ``[total_rows, width]`` for the next backward; returns ``(view, slot)``."""
        slot = self.calls["dkv"] & 1
        self.calls["dkv"] += 1
        return self.view("dkv", slot), slot

    def reduce_dkv(self, slot: int, out_rows):
        """Announces this rank's partial dK|dV, waits for every rank's, and reduces this rank's two chunks
        over the ranks into ``out_rows [2 * chunk_rows, width]`` (any row stride).  Runs on the current stream,
        after the kernels that wrote the partial buffer."""
        assert out_rows.shape == (2 * self.chunk_rows, self.width) and out_rows.stride(1) == 1
        s = torch.cuda.current_stream(self.device)
        off, coff = self.off_buf["dkv"][slot], self.off_cnt["dkv"][slot]
        self.total["dkv"][slot] += self.world
        target = self.total["dkv"][slot]
        ann = K.proto("dh_announce", [c_void_p, c_int, c_uint, c_void_p])
        K.check(ann(self._ptr_array(coff), self.world, 1, s.cuda_stream), "dh_announce")
        fn = K.proto("dh_reduce_blocks", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_uint,
                                          c_int, c_int, c_void_p])
        ctx = self.exposed.span(s) if (self.exposed is not None and self.exposed.enabled) else contextlib.nullcontext()
        with ctx:
            for half, chunk in enumerate(self.chunk_ids()):
                dst = out_rows[half * self.chunk_rows:]
                K.check(fn(self._ptr_array(off), self._mc(off), self.ptrs[self.rank] + coff, 0, dst.data_ptr(), out_rows.stride(0),
                           self.width, chunk * self.chunk_blocks, self.chunk_rows, self.rank, self.world, target, self.ctas, 256,
                           s.cuda_stream), "dh_reduce_blocks")


class SimulatedCP:
    """The interface of ``FusedCP`` on library collectives (gloo / NCCL), for CPU ranks: the gather form of
    context parallelism (chunk placement, one causal call per query chunk, zero-filled unseen keys, owner
    reduction of dK|dV) can then be checked against autograd without GPUs.  Everything happens at call time;
    slots and targets are dummies."""

    def __init__(self, ps, cfg, train, device, batch: int | None = None):
        self.ps, self.device = ps, torch.device(device)
        self.world, self.rank = ps.cp, ps.cp_rank
        B = batch or train.micro_batch_size
        nkv = max(cfg.num_query_groups // ps.tp, 1)
        self.width = 2 * nkv * cfg.head_dim
        self.chunk_rows = cfg.seq_length // (2 * self.world) * B
        self.total_rows = 2 * self.world * self.chunk_rows
        self._bufs = {}
        self.exposed = None

    def chunk_ids(self):
        return self.rank, 2 * self.world - 1 - self.rank

    def push_kv(self, kv_rows, site: str, stream=None):
        mine = kv_rows.contiguous()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.ps.cp_group)
        full = torch.empty((self.total_rows, self.width), dtype=mine.dtype, device=mine.device)
        for r, p in enumerate(parts):
            for half, chunk in enumerate((r, 2 * self.world - 1 - r)):
                full[chunk * self.chunk_rows:(chunk + 1) * self.chunk_rows] = p[half * self.chunk_rows:(half + 1) * self.chunk_rows]
        self._bufs[site] = full
        return 0, 0

    def wait_kv(self, site: str, slot: int, target: int, n_chunks: int):
        return self._bufs.pop(site)

    def dkv_buffer(self):
        dtype = next(iter(self._bufs.values())).dtype if self._bufs else torch.float32
        self._part = torch.zeros((self.total_rows, self.width), dtype=torch.float32, device=self.device)
        return self._part, 0

    def reduce_dkv(self, slot: int, out_rows):
        part = self._part
        dist.all_reduce(part, group=self.ps.cp_group)
        for half, chunk in enumerate(self.chunk_ids()):
            out_rows[half * self.chunk_rows:(half + 1) * self.chunk_rows] = part[chunk * self.chunk_rows:(chunk + 1) * self.chunk_rows].to(out_rows.dtype)
