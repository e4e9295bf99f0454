"""Mixed-precision Adam over the model's flat buffers: bf16 parameters, fp32 master
weights, fp32 moments, fp32 ``main_grad`` accumulation, global-norm clipping and an
optional data-parallel sharding of the optimizer state.

Supplies what the reference takes from Megatron (Float16 optimizer with
``--use-distributed-optimizer``, ``optimizer.scale_loss``, ``param.main_grad``;
script/run.sh:108-127, megatron.patch:764-770): the engine writes weight gradients straight
into ``main_grad`` (dhellam/core/dstb.py:541-563), and the step happens once after the last
micro-batch.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import kernels as K
from ..config import TrainConfig


def _adam_ref(param, master, m, v, grad, lr, b1, b2, eps, wd, step, grad_scale):
    g = grad * grad_scale
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    bc1 = 1 - b1 ** step
    bc2 = 1 - b2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    master.mul_(1 - lr * wd).addcdiv_(m / bc1, denom, value=-lr)
    param.copy_(master.to(param.dtype))


def adam_update(param, master, m, v, grad, lr, b1, b2, eps, wd, step, grad_scale=1.0, stream=None):
    """One fused Adam(W) update of a contiguous range; writes the low-precision copy too."""
    if K.use_library(param):
        from ..ops import library as LIB
        return LIB.adam_update(param, master, m, v, grad, lr, b1, b2, eps, wd, step, grad_scale)
    if not param.is_cuda:
        return _adam_ref(param, master, m, v, grad, lr, b1, b2, eps, wd, step, grad_scale)
    fn = K.proto("dh_adam_step", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_float, c_float,
                                  c_float, c_float, c_float, c_float, c_float, c_float, c_void_p])
    K.check(fn(param.data_ptr(), master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), param.numel(),
               int(param.dtype == torch.bfloat16), lr, b1, b2, eps, wd, 1 - b1 ** step, 1 - b2 ** step, grad_scale,
               K.stream_ptr(stream)), "dh_adam_step")


def sum_squares(t, stream=None):
    """fp32 sum of squares of a contiguous fp32 tensor (1-element tensor)."""
    if K.use_library(t):
        from ..ops import library as LIB
        return LIB.sum_squares(t)
    if not t.is_cuda:
        return (t.float() ** 2).sum().reshape(1)
    out = torch.zeros(1, dtype=torch.float32, device=t.device)
    if K.deterministic():
        n = K.proto("dh_sum_squares_scratch", [])()
        scratch = K.det_scratch(t.device, n, zero_tail=True)
        fn = K.proto("dh_sum_squares_det", [c_void_p, c_void_p, c_int64, c_void_p, c_void_p])
        K.check(fn(t.data_ptr(), out.data_ptr(), t.numel(), scratch.data_ptr(), K.stream_ptr(stream)), "dh_sum_squares_det")
        return out
    fn = K.proto("dh_sum_squares", [c_void_p, c_void_p, c_int64, c_void_p])
    K.check(fn(t.data_ptr(), out.data_ptr(), t.numel(), K.stream_ptr(stream)), "dh_sum_squares")
    return out


class DynamicLossScaler:
    """Loss scale that backs off on overflow and grows after a window of good steps (the
    behaviour of Megatron's dynamic grad scaler, which the reference's fp16 run relies on:
    script/run.sh:117 ``--initial-loss-scale 65536``).  ``hysteresis`` overflows in a row are
    tolerated before the scale is halved."""

    def __init__(self, initial: float = 65536.0, min_scale: float = 1.0, growth: float = 2.0, backoff: float = 0.5,
                 window: int = 1000, hysteresis: int = 2):
        self.scale, self.min_scale = float(initial), float(min_scale)
        self.growth, self.backoff, self.window, self.hysteresis = growth, backoff, window, hysteresis
        self._good, self._left = 0, hysteresis

    def update(self, overflow: bool):
        if overflow:
            self._good = 0
            self._left -= 1
            if self._left <= 0:
                self.scale = max(self.scale * self.backoff, self.min_scale)
        else:
            self._good += 1
            if self._good >= self.window:
                self._good, self._left = 0, self.hysteresis
                self.scale *= self.growth

    def state_dict(self):
        return {"scale": self.scale, "good": self._good, "left": self._left}

    def load_state_dict(self, sd):
        self.scale, self._good, self._left = float(sd["scale"]), int(sd["good"]), int(sd["left"])


class MixedPrecisionAdam:
    """Adam with fp32 master weights over ``model.flat_param`` / ``model.flat_grad``.

    With ``distributed=True`` every data-parallel rank keeps master weights and moments
    for ``1/dp`` of the flat buffer only: gradients are reduce-scattered, the owned slice
    is updated, and the updated parameters are all-gathered (ZeRO-1).
    """

    def __init__(self, model, train: TrainConfig, ps, distributed: bool = False, loss_scale: Optional[float] = None):
        self.model, self.train, self.ps = model, train, ps
        self.step_count = 0
        self.skipped_steps = 0
        self.scaler = DynamicLossScaler(train.initial_loss_scale, train.min_loss_scale, window=train.loss_scale_window,
                                        hysteresis=train.hysteresis) if train.dynamic_loss_scale else None
        self._static_scale = float(loss_scale if loss_scale is not None else train.loss_scale)
        self.distributed = distributed and ps.dp * ps.cp > 1 and not model.cfg.is_moe
        flat = model.flat_param
        n = flat.numel()
        self.group = ps.dp_cp_group
        self.gsize = ps.dp * ps.cp
        if self.distributed:
            # the last rank's shard may be shorter when n does not divide by the group size
            self.shard = (n + self.gsize - 1) // self.gsize
            grank = dist.get_rank(self.group)
            self.lo = min(grank * self.shard, n)
            self.hi = min(self.lo + self.shard, n)
        else:
            self.lo, self.hi = 0, n
        k = self.hi - self.lo
        self.master = flat[self.lo:self.hi].float().clone()
        self.exp_avg = torch.zeros(k, dtype=torch.float32, device=flat.device)
        self.exp_avg_sq = torch.zeros(k, dtype=torch.float32, device=flat.device)
        # contiguous ranges with the same weight decay (norm weights and biases get none)
        self.segments: List[tuple] = []
        for name, p in model.named_parameters():
            off, shape = model.param_index[name]
            cnt = math.prod(shape)
            wd = 0.0 if (p.sequence_parallel or name.endswith("bias")) else train.weight_decay
            lo, hi = max(off, self.lo), min(off + cnt, self.hi)
            if lo >= hi:
                continue
            if self.segments and self.segments[-1][2] == wd and self.segments[-1][1] >= lo - 256:
                self.segments[-1] = (self.segments[-1][0], hi, wd)
            else:
                self.segments.append((lo, hi, wd))

    @property
    def loss_scale(self) -> float:
        return self.scaler.scale if self.scaler is not None else self._static_scale

    @loss_scale.setter
    def loss_scale(self, value: float):
        if self.scaler is not None:
            self.scaler.scale = float(value)
        else:
            self._static_scale = float(value)

    # ---- hooks kept from the Megatron optimizer API
    def scale_loss(self, loss):
        return loss * self.loss_scale

    def zero_grad(self):
        self.model.zero_grad_buffer()

    # ---- gradient finalisation
    def reduce_gradients(self):
        """Sequence-parallel norm gradients over TP, then data(+context)-parallel reduction."""
        ps, model = self.ps, self.model
        reducer = getattr(self, "grad_reducer", None)
        dp_done = reducer is not None and reducer.finish()       # also waits for the buckets still in flight
        if ps.tp > 1:
            bufs = [p.main_grad for _, p in model.named_parameters() if p.sequence_parallel or p.base_name == "router_weight"
                    or p.base_name == "position_embeddings"]
            if bufs:
                flat = torch.cat([b.reshape(-1) for b in bufs])
                dist.all_reduce(flat, group=ps.tp_group)
                o = 0
                for b in bufs:
                    b.copy_(flat[o:o + b.numel()].view_as(b))
                    o += b.numel()
        if dp_done:
            # buckets were summed under the backward pass; only the data-parallel average is left
            model.flat_grad.mul_(1.0 / ps.dp)
        elif self.gsize > 1:
            g = model.flat_grad
            if model.cfg.is_moe and ps.ep > 1:
                self._reduce_moe(g)
            elif self.distributed:
                n = g.numel()
                if n % self.gsize == 0:
                    out = torch.empty(self.shard, dtype=g.dtype, device=g.device)
                    dist.reduce_scatter_tensor(out, g, group=self.group)
                    g[self.lo:self.hi].copy_(out)
                else:
                    dist.all_reduce(g, group=self.group)
                g[self.lo:self.hi].mul_(1.0 / ps.dp)
            else:
                dist.all_reduce(g, group=self.group)
                g.mul_(1.0 / ps.dp)

    def _reduce_moe(self, g):
        """Dense parameters reduce over DP x CP; expert parameters only over the ranks that
        hold the same experts."""
        ps, model = self.ps, self.model
        dense, expert = [], []
        for _, p in model.named_parameters():
            (expert if p.is_expert else dense).append(p.main_grad)
        for bufs, group, denom in ((dense, ps.dp_cp_group, ps.dp), (expert, getattr(ps, "edp_group", None), ps.dp)):
            if not bufs:
                continue
            for b in bufs:
                if group is not None:
                    dist.all_reduce(b, group=group)
                b.mul_(1.0 / denom)

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the gradients of this optimizer's shard over all model shards."""
        ps, model = self.ps, self.model
        g = model.flat_grad
        total = sum_squares(g[self.lo:self.hi])
        if ps.tp > 1 and ps.tp_rank != 0:
            # replicated parameters are counted on TP rank 0 only
            for name, p in model.named_parameters():
                if p.sequence_parallel or p.base_name in ("router_weight", "position_embeddings"):
                    off, shape = model.param_index[name]
                    lo, hi = max(off, self.lo), min(off + math.prod(shape), self.hi)
                    if lo < hi:
                        total = total - sum_squares(g[lo:hi])
        if dist.is_initialized() and dist.get_world_size() > 1:
            for grp, size in ((ps.tp_group, ps.tp), (ps.pp_group, ps.pp)):
                if size > 1:
                    dist.all_reduce(total, group=grp)
            if self.distributed:
                dist.all_reduce(total, group=self.group)
        return total.clamp_min(0).sqrt()

    # ---- the step
    def step(self, lr: Optional[float] = None):
        """Reduces gradients, clips, updates.  Returns the gradient norm (tensor)."""
        tr = self.train
        self.reduce_gradients()
        norm = self.grad_norm()
        scale = 1.0 / self.loss_scale
        scale_of_norm = scale              # the scaler may change the scale below; the norm was taken with this one
        if self.scaler is not None:
            # the norm is already summed over every model-parallel group, so all ranks see the same
            # overflow; one host read per step, as in Megatron's fp16 optimizer
            overflow = not bool(torch.isfinite(norm))
            used = self.loss_scale
            self.scaler.update(overflow)
            if overflow:
                self.skipped_steps += 1
                return norm * (1.0 / used)
        # host read: one scalar per step, after the last backward.  A non-finite norm (an overflow or a
        # NaN somewhere in the gradients) must not reach the update: inf gives clip = 0 and inf * 0 = NaN
        # would be written into the master weights and both moments for good.  The step is skipped and
        # counted, whichever scaler is in use (the dynamic scaler above has already returned).
        norm_val = float(norm) * scale
        if not math.isfinite(norm_val):
            self.skipped_steps += 1
            return norm * scale_of_norm
        if tr.clip_grad and tr.clip_grad > 0:
            scale = min(tr.clip_grad / (norm_val + 1e-6), 1.0) * scale
        self.step_count += 1
        lr = tr.lr if lr is None else lr
        flat_p, flat_g = self.model.flat_param, self.model.flat_grad
        for lo, hi, wd in self.segments:
            a, b = lo - self.lo, hi - self.lo
            adam_update(flat_p[lo:hi], self.master[a:b], self.exp_avg[a:b], self.exp_avg_sq[a:b], flat_g[lo:hi], lr,
                        tr.adam_beta1, tr.adam_beta2, tr.adam_eps, wd, self.step_count, scale)
        if self.distributed:
            n = flat_p.numel()
            if n % self.gsize == 0:
                dist.all_gather_into_tensor(flat_p, flat_p[self.lo:self.hi].clone(), group=self.group)
            else:
                parts = [torch.empty(self.shard, dtype=flat_p.dtype, device=flat_p.device) for _ in range(self.gsize)]
                mine = torch.zeros(self.shard, dtype=flat_p.dtype, device=flat_p.device)
                mine[: self.hi - self.lo] = flat_p[self.lo:self.hi]
                dist.all_gather(parts, mine, group=self.group)
                flat_p.copy_(torch.cat(parts)[:n])
        return norm * scale_of_norm

    # ---- checkpoint support
    def state_dict(self):
        return {"step": self.step_count, "lo": self.lo, "hi": self.hi, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "loss_scale": self.loss_scale,
                "scaler": self.scaler.state_dict() if self.scaler is not None else None}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        assert (self.lo, self.hi) == (sd["lo"], sd["hi"]), "optimizer shard layout changed"
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.loss_scale = sd.get("loss_scale", 1.0)
        if self.scaler is not None and sd.get("scaler"):
            self.scaler.load_state_dict(sd["scaler"])
