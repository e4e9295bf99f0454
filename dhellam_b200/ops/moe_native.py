"""Device-resident mixture-of-experts exchange (GPU only): plan, dispatch, grouped expert GEMMs, combine.

The reference has no MoE ops at all (it claims expert parallelism, README.md:8; the only trace in its code is the
all-to-all entry of micro_benchmark/overlap.py:141-145; see ``models/moe.py``).  ``ops/moe.py`` is the host-driven
restatement used on CPU ranks: sort / bincount, two ``.tolist()`` reads per layer, a variable-size
``all_to_all_single`` and a Python loop of per-expert GEMMs.  Here nothing about the routing ever
reaches the host:

* ``plan``       ``moe_plan`` (stable position of every copy inside its expert, counts) ->
                 the count rows of all expert-parallel ranks (one tiny device-side all-gather) ->
                 ``moe_offsets`` (where every (source, expert) group lands on the expert's owner;
                 regions padded to 256 rows so GEMM tiles never straddle experts);
* ``dispatch``   one warp per copy stores the token row straight into the owner's expert-major
                 landing buffer over NVLink peer memory, then an arrival counter rises on every rank;
* expert GEMMs   ONE grouped launch of the CTA-pair tcgen05 GEMM per product, driven by the
                 device-side region table (forward, data gradient, weight gradient);
* ``combine``    one warp per token pulls its k expert outputs from their owners and writes the
                 gate-weighted sum (and keeps the copies for the gate gradient).

Landing and output buffers live in symmetric memory of the expert-parallel group (plain tensors when
``ep == 1``), two slots per site with monotonically increasing counters, like ``FusedTP``.  The row
capacity per rank is the worst case ``ep * tokens * k`` (dropless) unless
``DHELLAM_MOE_CAPACITY_FACTOR`` lowers it; a plan that does not fit sets the status word and an
``overflow`` flag instead of writing out of bounds.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_uint, c_void_p
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import kernels as K

PAD = 256
SITES = ("xe", "y", "dy", "xeb", "dxe")


def _align(n, a=1024):
    return (n + a - 1) // a * a


@dataclass
class DevicePlan:
    topi: torch.Tensor         # [T*k] int32 expert of every copy
    pos: torch.Tensor          # [T*k] int32 position inside its expert (this source)
    dst_base: torch.Tensor     # [E] int32
    offs: torch.Tensor         # [el+1] int32 padded region starts of the local experts; offs[el] = rows in use
    rows_e: torch.Tensor       # [el] int32
    dest_rank: torch.Tensor    # [T*k] int32
    dest_row: torch.Tensor     # [T*k] int32
    overflow: torch.Tensor     # [1] int32
    T: int
    k: int


class DeviceMoE:
    def __init__(self, ps, cfg, train, device, tokens: int):
        self.ps, self.device = ps, torch.device(device)
        self.ep, self.rank = max(ps.ep, 1), (ps.ep_rank if ps.ep > 1 else 0)
        self.E, self.k, self.h = cfg.num_experts, cfg.moe_top_k, cfg.hidden_size
        self.el = self.E // self.ep
        self.T = tokens
        factor = float(os.environ.get("DHELLAM_MOE_CAPACITY_FACTOR", "0") or 0) or float(self.ep)
        cap = int(min(self.ep, factor) * tokens * self.k) + self.el * PAD
        self.capacity = (cap + PAD - 1) // PAD * PAD
        buf_bytes = _align(self.capacity * self.h * 2)
        self.off_buf, self.off_cnt = {}, {}
        off = 0
        for s in SITES:
            self.off_buf[s] = [off, off + buf_bytes]
            off += 2 * buf_bytes
        cnt_base = off
        for s in SITES:
            self.off_cnt[s] = [off, off + 256]
            off += 512
        if self.ep > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(off, dtype=torch.uint8, device=self.device)
            self.hdl = symm_mem.rendezvous(self.buf, group=ps.ep_group.group_name)
            self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        else:
            self.buf = torch.empty(off, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()]
        self.buf[cnt_base:off].zero_()
        self.done_ctas = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        if self.ep > 1:
            dist.barrier(group=ps.ep_group)
        self.calls = {s: 0 for s in SITES}
        self.total = {s: [0, 0] for s in SITES}
        self._arr = ctypes.c_void_p * self.ep
        self.ctas = int(os.environ.get("DHELLAM_MOE_CTAS", "64"))

    # ------------------------------------------------------------------ helpers
    def _ptr_array(self, off):
        return self._arr(*[p + off for p in self.ptrs])

    def view(self, site, slot, width=None):
        off = self.off_buf[site][slot]
        w = width or self.h
        return self.buf[off:off + self.capacity * w * 2].view(torch.bfloat16).view(self.capacity, w)

    def next_slot(self, site):
        slot = self.calls[site] & 1
        self.calls[site] += 1
        return slot

    def _counter_ptr(self, site, slot):
        return self.ptrs[self.rank] + self.off_cnt[site][slot]

    def _wait(self, site, slot):
        s = torch.cuda.current_stream(self.device)
        fn = K.proto("dh_wait_counters", [c_void_p, c_int, c_uint, c_int64, c_void_p])
        K.check(fn(self._counter_ptr(site, slot), 1, self.total[site][slot], 0, s.cuda_stream), "dh_wait_counters")

    # ------------------------------------------------------------------ plan
    def plan(self, topi32) -> DevicePlan:
        n = topi32.numel()
        T = n // self.k
        dev = self.device
        s = torch.cuda.current_stream(dev).cuda_stream
        pos = torch.empty(n, dtype=torch.int32, device=dev)
        counts = torch.empty(self.E, dtype=torch.int32, device=dev)
        K.check(K.proto("dh_moe_plan", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])(
            topi32.data_ptr(), n, self.E, pos.data_ptr(), counts.data_ptr(), s), "dh_moe_plan")
        if self.ep > 1:
            cnt_all = torch.empty((self.ep, self.E), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(cnt_all, counts, group=self.ps.ep_group)       # stays on the device
        else:
            cnt_all = counts.view(1, self.E)
        dst_base = torch.empty(self.E, dtype=torch.int32, device=dev)
        offs = torch.empty(self.el + 1, dtype=torch.int32, device=dev)
        rows_e = torch.empty(self.el, dtype=torch.int32, device=dev)
        overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        K.check(K.proto("dh_moe_offsets", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])(
            cnt_all.data_ptr(), self.ep, self.E, self.rank, self.capacity, dst_base.data_ptr(), offs.data_ptr(), rows_e.data_ptr(),
            overflow.data_ptr(), s), "dh_moe_offsets")
        return DevicePlan(topi32.reshape(-1), pos, dst_base, offs, rows_e, torch.empty(n, dtype=torch.int32, device=dev),
                          torch.empty(n, dtype=torch.int32, device=dev), overflow, T, self.k)

    # ------------------------------------------------------------------ dispatch (push)
    def dispatch(self, plan: DevicePlan, src_rows, site: str, scale=None, other=None, record: bool = False):
        """Pushes ``src_rows[i // k]`` (optionally scaled per copy) of every copy to its owner's landing
        buffer of ``site``.  Returns ``(slot, dots)``; ``dots [T*k]`` = row-wise dot with ``other`` if given."""
        slot = self.next_slot(site)
        s = torch.cuda.current_stream(self.device).cuda_stream
        K.check(K.proto("dh_moe_zero_pad", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])(
            self.view(site, slot).data_ptr(), plan.offs.data_ptr(), plan.rows_e.data_ptr(), self.el, self.h, s), "dh_moe_zero_pad")
        n = plan.topi.numel()
        dots = torch.empty(n, dtype=torch.float32, device=self.device) if other is not None else None
        self.total[site][slot] += self.ep
        fn = K.proto("dh_moe_dispatch", [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
        K.check(fn(src_rows.data_ptr(), src_rows.stride(0), plan.topi.data_ptr(), plan.pos.data_ptr(), plan.dst_base.data_ptr(),
                   K.ptr(scale), K.ptr(other), K.ptr(dots), self._ptr_array(self.off_buf[site][slot]),
                   plan.dest_rank.data_ptr() if record else None, plan.dest_row.data_ptr() if record else None,
                   self._ptr_array(self.off_cnt[site][slot]), self.done_ctas.data_ptr(), n, self.k, self.h, self.el, self.ep,
                   self.ctas, s), "dh_moe_dispatch")
        return slot, dots

    def landed(self, site: str, slot: int):
        """Makes the current stream wait (bounded) until every source's rows of ``site`` have arrived; returns the buffer."""
        self._wait(site, slot)
        return self.view(site, slot)

    # ------------------------------------------------------------------ publish + combine (pull)
    def output_buffer(self, site: str):
        slot = self.next_slot(site)
        return self.view(site, slot), slot

    def publish(self, site: str, slot: int):
        """After the kernel that filled the output buffer on the current stream: tells every rank it is complete."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        self.total[site][slot] += self.ep
        K.check(K.proto("dh_announce", [c_void_p, c_int, c_uint, c_void_p])(self._ptr_array(self.off_cnt[site][slot]), self.ep, 1, s),
                "dh_announce")

    def combine(self, plan: DevicePlan, site: str, slot: int, gates=None, keep_copies: bool = False):
        """``out[t] = sum_j gates[t, j] * owner_buffer[copy (t, j)]`` (plain sum without gates)."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        out = torch.empty((plan.T, self.h), dtype=torch.bfloat16, device=self.device)
        copies = torch.empty((plan.T * self.k, self.h), dtype=torch.bfloat16, device=self.device) if keep_copies else None
        fn = K.proto("dh_moe_combine", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p])
        K.check(fn(self._ptr_array(self.off_buf[site][slot]), plan.dest_rank.data_ptr(), plan.dest_row.data_ptr(), K.ptr(gates),
                   out.data_ptr(), K.ptr(copies), self._counter_ptr(site, slot), self.total[site][slot], plan.T, self.k, self.h,
                   self.ep, self.ctas, s), "dh_moe_combine")
        return out, copies

    # ------------------------------------------------------------------ grouped GEMMs
    def _grouped(self, a, b2d, b_mn, d, M, N, Kd, mode, plan, budget):
        s = torch.cuda.current_stream(self.device).cuda_stream
        fn = K.proto("dh_gemm_grouped_bf16", [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                              c_int, c_void_p, c_int, c_int, c_void_p])
        K.check(fn(a.data_ptr(), a.stride(0), b2d.data_ptr(), b2d.stride(0), int(b_mn), d.data_ptr(), d.stride(0), M, N, Kd, self.el, mode,
                   plan.offs.data_ptr(), self.capacity, int(budget), s), "dh_gemm_grouped_bf16")

    def grouped_nt(self, x_rows, w, plan, out=None, sm_budget: int = 0):
        """``out[rows of e] = x_rows[rows of e] @ w[e]^T``; ``w [el, N, K]``."""
        el, N, Kd = w.shape
        if out is None:
            out = torch.empty((self.capacity, N), dtype=torch.bfloat16, device=self.device)
        self._grouped(x_rows, w.view(el * N, Kd), False, out, self.capacity, N, Kd, 1, plan, sm_budget)
        return out

    def grouped_nn(self, dy_rows, w, plan, out=None, sm_budget: int = 0):
        """``out[rows of e] = dy_rows[rows of e] @ w[e]``; ``w [el, N, K]`` -> out width K."""
        el, N, Kd = w.shape
        if out is None:
            out = torch.empty((self.capacity, Kd), dtype=torch.bfloat16, device=self.device)
        # contraction over N: B stack is [el * N, Kd] read MN-major
        self._grouped(dy_rows, w.view(el * N, Kd), True, out, self.capacity, Kd, N, 1, plan, sm_budget)
        return out

    def grouped_tn_acc(self, dy_rows, x_rows, main_grad, plan, sm_budget: int = 0):
        """``main_grad[e] += dy_rows[rows of e]^T @ x_rows[rows of e]``; ``main_grad [el, N, K]`` fp32."""
        el, N, Kd = main_grad.shape
        self._grouped(dy_rows, x_rows, True, main_grad.view(el * N, Kd), N, Kd, self.capacity, 2, plan, sm_budget)
        return main_grad

    # ------------------------------------------------------------------ ragged activation
    def swiglu_fwd(self, z, plan):
        f = z.shape[1] // 2
        out = torch.empty((self.capacity, f), dtype=z.dtype, device=z.device)
        s = torch.cuda.current_stream(self.device).cuda_stream
        K.check(K.proto("dh_swiglu_fwd_n", [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p])(
            z.data_ptr(), out.data_ptr(), self.capacity, plan.offs[self.el:].data_ptr(), f, 0, s), "dh_swiglu_fwd_n")
        return out

    def swiglu_bwd(self, d_a, z, plan):
        f = z.shape[1] // 2
        dz = torch.empty_like(z)
        s = torch.cuda.current_stream(self.device).cuda_stream
        K.check(K.proto("dh_swiglu_bwd_n", [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p])(
            d_a.data_ptr(), z.data_ptr(), dz.data_ptr(), self.capacity, plan.offs[self.el:].data_ptr(), f, 0, s), "dh_swiglu_bwd_n")
        return dz
