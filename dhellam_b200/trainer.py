"""Trainer: builds the folded model, the double-strand engine and the optimizer for one
rank and runs optimizer steps.  This is the public entry point a user calls
(``Trainer(...).train_step(batches)``); ``train.py`` wraps it with a command line.

Stands in for the parts of Megatron's ``pretrain`` / ``train_step`` that the reference
drives through its patch (megatron.patch:764-812): gradient zeroing, the forward-backward
schedule, gradient finalisation, the optimizer step, and loss / throughput reporting.
"""
from __future__ import annotations

import os
import time
from typing import List, Optional

import torch
import torch.distributed as dist

from .common.global_variables import GLOBAL_VARIABLES
from .config import ModelConfig, ParallelConfig, TrainConfig
from .core.engine import DoubleStrandEngine, Env, MicroBatch
from .core.modules import DSLLM
from .optim.adam import MixedPrecisionAdam
from .parallel import state as PS
from .sched.strategy import Strategy


class Trainer:
    def __init__(self, cfg: ModelConfig, pcfg: ParallelConfig, train: TrainConfig, device=None, ps=None,
                 strategy: Optional[Strategy] = None, distributed_optimizer: bool = False, model_init: str = "random",
                 single_stream: bool = False, profile: bool = False, trace=None):
        self.cfg, self.pcfg, self.train = cfg, pcfg, train
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.ps = ps if ps is not None else PS.initialize_model_parallel(pcfg)
        self.model = DSLLM(cfg, self.ps, train, device=self.device, init=model_init)
        fused = None
        if train.fused_comm and self.device.type == "cuda" and self.ps.tp > 1:
            from .ops.fused_comm import FusedTP
            try:
                fused = FusedTP(self.ps, cfg, train, self.device)
            except Exception as e:       # no symmetric memory / no peer access on this machine
                # Falling back silently would turn a broken symmetric-memory set-up into a different
                # (NCCL) run that looks like a slow one.  It is an error unless explicitly allowed.
                if os.environ.get("DHELLAM_ALLOW_NCCL_FALLBACK", "0") != "1":
                    raise RuntimeError(
                        f"in-kernel tensor-parallel collectives could not be set up on rank {self.ps.rank} "
                        f"({type(e).__name__}: {e}); run with --no-fused-comm (TrainConfig.fused_comm=False) for library "
                        "collectives, or set DHELLAM_ALLOW_NCCL_FALLBACK=1 to fall back automatically") from e
                print(f"[dhellam_b200] in-kernel collectives unavailable on rank {self.ps.rank} ({type(e).__name__}: {e}); "
                      "DHELLAM_ALLOW_NCCL_FALLBACK=1: using NCCL collectives", flush=True)
            # all ranks of the group take the same path
            ok = torch.tensor([1 if fused is not None else 0], device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.ps.tp_group)
            if int(ok) == 0:
                fused = None
        from . import kernels as _K
        if fused is None and self.device.type == "cuda" and self.ps.world > 1 and train.dhellam and _K.backend() == "native":
            # Library collectives co-run with the GEMMs and occupy one SM of many SM pairs;
            # a CTA-pair GEMM then cannot place its clusters (measured 1.6x slower step),
            # so that path keeps the single-CTA tiles.
            from .ops.gemm import set_gemm_mode
            set_gemm_mode(1)
        if train.deterministic:
            _K.set_deterministic(True)
        self.env = Env(cfg, self.ps, train, self.device, self.model.dtype, fused=fused)
        if train.fused_comm and self.device.type == "cuda" and self.ps.cp > 1 and _K.backend() == "native" \
                and os.environ.get("DHELLAM_CP_RING", "0") != "1":
            # key/value exchange of context parallelism over peer memory instead of the library ring
            from .ops.fused_comm import FusedCP
            self.env.fused_cp = FusedCP(self.ps, cfg, train, self.device)
        if cfg.is_moe and self.device.type == "cuda" and _K.backend() == "native" and os.environ.get("DHELLAM_MOE_HOST", "0") != "1":
            # token dispatch / combine and the grouped expert GEMMs without the host in the loop
            from .ops.moe_native import DeviceMoE
            self.env.moe_dev = DeviceMoE(self.ps, cfg, train, self.device, train.micro_batch_size * cfg.seq_length // max(self.ps.cp, 1))
        if self.device.type == "cpu" and self.ps.cp > 1 and os.environ.get("DHELLAM_CP_GATHER_SIM", "0") == "1":
            from .ops.fused_comm import SimulatedCP           # the gather form on library collectives (tests on CPU ranks)
            self.env.fused_cp = SimulatedCP(self.ps, cfg, train, self.device)
        if strategy is None and train.schedule_config:
            strategy = Strategy.load(train.schedule_config)
        if strategy is None and train.reference_schedule:
            from .models.transformer import build_layer_program
            from .sched.strategy import reference_paired
            blocks = reference_paired(build_layer_program(cfg, cp=self.ps.cp))
            if blocks is None:
                raise ValueError("the reference's built-in schedule exists for the dense layer only")
            strategy = Strategy(dcblocks=blocks)
        self.engine = DoubleStrandEngine(self.model, self.env, strategy, single_stream=single_stream or not train.dhellam,
                                         profile=profile, trace=trace, compute_streams=train.compute_streams,
                                         sync_per_block=train.sync_per_block)
        if self.env.fused_tp and not cfg.is_moe and self.ps.cp == 1:
            # The symmetric staging slots are reused every second call; prove for THIS strategy (built in,
            # searched or user-written) and stream count that no rank can overwrite a slot another rank
            # still reads.  A strategy that fails is refused instead of producing silently wrong gradients.
            from .models.transformer import FUSED_BUFFER_EFFECTS
            from .sched.checker import check_buffer_reuse
            check_buffer_reuse(self.engine.program, self.engine.executor.strategy, FUSED_BUFFER_EFFECTS,
                               compute_streams=1 if (single_stream or not train.dhellam) else train.compute_streams)
        if self.env.fused_cp is not None:
            self.env.fused_cp.exposed = self.engine.executor.exposed
        if fused is not None:
            fused.exposed = self.engine.executor.exposed
            # row-block-wise reduce-scatter: the reduction kernel may start once its GEMM has been launched
            self.engine.executor.pipeline = fused.rs_blocks and fused.policy == "split"
        self.optimizer = MixedPrecisionAdam(self.model, train, self.ps, distributed=distributed_optimizer)
        if self.ps.dp * self.ps.cp > 1:
            from .parallel.dp import OverlappedGradReducer
            reducer = OverlappedGradReducer(self.model, self.ps, self.engine.streams)
            if self.optimizer.distributed:
                # gradient reduce-scatter into the optimizer shards, bucket by bucket under the backward pass
                n, sh, gs = self.model.flat_param.numel(), self.optimizer.shard, self.optimizer.gsize
                reducer.set_shards([(min(r * sh, n), min(r * sh + sh, n)) for r in range(gs)])
            self.engine.grad_reducer = reducer
            self.optimizer.grad_reducer = reducer
        GLOBAL_VARIABLES["loss_scale_func"] = self.optimizer.scale_loss
        self.iteration = 0
        self.last_grad_norm = None
        # True: synchronise after the forward-backward pass and read the device status word, so that
        # a bounded device-side wait that gave up (its kernel returned early and left an output
        # unwritten) raises ``CommTimeout`` BEFORE the optimizer folds that garbage into the master
        # weights.  Costs one device synchronisation per step; train.py turns it on (it synchronises
        # every step anyway), the benchmark leaves it off.
        self.check_status = False

    def train_step(self, mbs: List[MicroBatch], lr: Optional[float] = None):
        """One optimizer step over ``mbs``.  Returns the mean loss as a tensor on the first
        pipeline stage (``None`` elsewhere); nothing here synchronises the host."""
        self.optimizer.zero_grad()
        self.engine.loss_scale = self.optimizer.loss_scale
        losses = self.engine.run_step(mbs)
        if self.check_status and self.device.type == "cuda":
            from .runtime.signals import check_device_status
            check_device_status()
        self.last_grad_norm = self.optimizer.step(lr)
        self.iteration += 1
        if losses:
            loss = torch.stack([l.float() for l in losses]).mean()
            if self.ps.dp > 1:
                dist.all_reduce(loss, group=self.ps.dp_group)
                loss = loss / self.ps.dp
            GLOBAL_VARIABLES["loss"] = loss
            return loss
        return None

    def close(self):
        """Drops every reference this trainer (and the module-level blackboard) holds to the model,
        the optimizer state and the symmetric buffers, so that their device memory can be freed
        before another trainer is built in the same process."""
        if GLOBAL_VARIABLES.get("loss_scale_func") == getattr(self.optimizer, "scale_loss", None):
            GLOBAL_VARIABLES.pop("loss_scale_func", None)
        GLOBAL_VARIABLES.pop("loss", None)
        if self.engine is not None:
            self.engine.grad_reducer = None
            self.engine.executor = None
        if self.env is not None:
            self.env.fused = None
            self.env.fused_cp = None
            self.env.moe_dev = None
        self.engine = self.optimizer = self.model = self.env = None

    def tokens_per_step(self) -> int:
        return self.train.global_batch_size * self.cfg.seq_length
