"""Megatron-compatible entry points.

``initialize_dhellam_megatron(megapath, extra_args_provider)`` keeps the reference's
signature (dhellam/adaptor/megatron.py:41-59).  The reference puts a Megatron-LM checkout
on ``sys.path`` and calls its ``initialize_megatron``; this framework carries its own
runtime, so the function parses the same Megatron command-line flags (the ones
script/run.sh:46-148 passes, plus ``--dhellam`` and ``--schedule-config`` from
``_add_dhellam_args``, :33-38), initialises ``torch.distributed`` and the process-group
mesh, and returns the argument namespace.  If ``megapath`` points at a Megatron checkout its
git hash and branch are reported as the reference does (:6-31); it is not imported.
"""
from __future__ import annotations

import argparse
import os
import subprocess
from typing import Callable, Optional

from ..common.common import print_rank0
from ..config import ModelConfig, ParallelConfig, TrainConfig

_ARGS = None


def check_megatron_available(megapath: Optional[str]):
    """Reports the git state of a Megatron checkout, if one is given and exists."""
    if not megapath or not os.path.exists(megapath):
        print_rank0("**** Megatron checkout not used: dhellam_b200 runs on its own runtime ****")
        return False
    def git(cmd):
        try:
            return subprocess.check_output(cmd, cwd=megapath, shell=True, stderr=subprocess.DEVNULL).decode().strip()
        except Exception:
            return "unknown"
    print_rank0(f"**** Git info for Megatron: git_hash={git('git rev-parse --short HEAD')} "
                f"git_branch={git('git rev-parse --abbrev-ref HEAD')} ****")
    return True


def _add_dhellam_args(parser):
    group = parser.add_argument_group(title="dhellam")
    group.add_argument("--dhellam", action="store_true", help="enable forward and backward overlap")
    group.add_argument("--schedule-config", type=str, default=None, help="schedule configuration files")
    return parser


def _add_megatron_args(parser):
    g = parser.add_argument_group(title="model")
    g.add_argument("--num-layers", type=int, default=8)
    g.add_argument("--hidden-size", type=int, default=8192)
    g.add_argument("--ffn-hidden-size", type=int, default=28672)
    g.add_argument("--num-attention-heads", type=int, default=64)
    g.add_argument("--group-query-attention", action="store_true")
    g.add_argument("--num-query-groups", type=int, default=None)
    g.add_argument("--kv-channels", type=int, default=None)
    g.add_argument("--seq-length", type=int, default=4096)
    g.add_argument("--max-position-embeddings", type=int, default=None)
    g.add_argument("--vocab-size", type=int, default=128256)
    g.add_argument("--normalization", default="RMSNorm", choices=["RMSNorm", "LayerNorm"])
    g.add_argument("--norm-epsilon", type=float, default=1e-5)
    g.add_argument("--swiglu", action="store_true")
    g.add_argument("--position-embedding-type", default="rope", choices=["rope", "learned_absolute"])
    g.add_argument("--rotary-base", type=float, default=500000.0)
    g.add_argument("--hidden-dropout", type=float, default=0.0)
    g.add_argument("--attention-dropout", type=float, default=0.0)
    g.add_argument("--untie-embeddings-and-output-weights", action="store_true")
    g.add_argument("--disable-bias-linear", action="store_true")
    g.add_argument("--init-method-std", type=float, default=0.02)
    g.add_argument("--num-experts", type=int, default=0)
    g.add_argument("--moe-router-topk", type=int, default=2)
    g.add_argument("--moe-aux-loss-coeff", type=float, default=0.01)
    g.add_argument("--use-mcore-models", action="store_true")
    g.add_argument("--use-flash-attn", action="store_true")
    g.add_argument("--attention-mask-cuda-init", action="store_true")
    t = parser.add_argument_group(title="training")
    t.add_argument("--micro-batch-size", type=int, default=4)
    t.add_argument("--global-batch-size", type=int, default=32)
    t.add_argument("--train-iters", type=int, default=2)
    t.add_argument("--lr", type=float, default=6.0e-5)
    t.add_argument("--min-lr", type=float, default=6.0e-6)
    t.add_argument("--lr-decay-style", default="cosine")
    t.add_argument("--lr-decay-iters", type=int, default=430000)
    t.add_argument("--lr-warmup-fraction", type=float, default=0.001)
    t.add_argument("--weight-decay", type=float, default=0.1)
    t.add_argument("--adam-beta1", type=float, default=0.9)
    t.add_argument("--adam-beta2", type=float, default=0.95)
    t.add_argument("--clip-grad", type=float, default=1.0)
    t.add_argument("--fp16", action="store_true")
    t.add_argument("--bf16", action="store_true")
    t.add_argument("--initial-loss-scale", type=float, default=2.0 ** 32)
    t.add_argument("--loss-scale", type=float, default=None, help="constant loss scale (else dynamic under --fp16)")
    t.add_argument("--loss-scale-window", type=int, default=1000)
    t.add_argument("--hysteresis", type=int, default=2)
    t.add_argument("--min-loss-scale", type=float, default=1.0)
    t.add_argument("--label-smoothing-factor", type=float, default=0.0)
    t.add_argument("--deterministic-mode", action="store_true", help="fixed-order reductions: two runs give bitwise equal results")
    t.add_argument("--use-distributed-optimizer", action="store_true")
    t.add_argument("--seed", type=int, default=1234)
    t.add_argument("--no-fused-comm", action="store_true", help="library collectives instead of in-kernel ones")
    t.add_argument("--compute-streams", type=int, default=1)
    p = parser.add_argument_group(title="parallelism")
    p.add_argument("--tensor-model-parallel-size", type=int, default=1)
    p.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    p.add_argument("--context-parallel-size", type=int, default=1)
    p.add_argument("--expert-model-parallel-size", type=int, default=1)
    p.add_argument("--sequence-parallel", action="store_true")
    p.add_argument("--distributed-backend", default=None, choices=[None, "nccl", "gloo"])
    p.add_argument("--distributed-timeout-minutes", type=float, default=2.0)
    p.add_argument("--step-gate-timeout", type=float, default=120.0,
                   help="seconds a rank waits for the others to announce a step before raising RankFailure (0: no gate, no heartbeat)")
    p.add_argument("--heartbeat-interval", type=float, default=0.5)
    p.add_argument("--heartbeat-timeout", type=float, default=15.0)
    l = parser.add_argument_group(title="logging and checkpoints")
    l.add_argument("--log-interval", type=int, default=1)
    l.add_argument("--log-throughput", action="store_true")
    l.add_argument("--timing-log-level", type=int, default=0)
    l.add_argument("--save", type=str, default=None)
    l.add_argument("--load", type=str, default=None)
    l.add_argument("--save-interval", type=int, default=10000)
    l.add_argument("--eval-interval", type=int, default=10000)
    l.add_argument("--eval-iters", type=int, default=0)
    l.add_argument("--metrics-jsonl", type=str, default=None)
    d = parser.add_argument_group(title="data")
    d.add_argument("--data-path", nargs="*", default=None)
    d.add_argument("--mock-data", action="store_true")
    d.add_argument("--tokenizer-type", default=None)
    d.add_argument("--tokenizer-model", default=None)
    d.add_argument("--split", default=None)
    # accepted so that the reference's launch lines (script/run.sh:108-160) parse unchanged; tokenisation happens before
    # this engine (it reads token files or synthetic ids), and there is one transformer implementation
    d.add_argument("--vocab-file", default=None)
    d.add_argument("--merge-file", default=None)
    d.add_argument("--data-cache-path", default=None)
    d.add_argument("--transformer-impl", default="local")
    return parser


def build_parser(extra_args_provider: Optional[Callable] = None):
    parser = argparse.ArgumentParser(description="dhellam_b200 (Megatron-style arguments)", allow_abbrev=False)
    parser = _add_megatron_args(parser)
    parser = _add_dhellam_args(parser)
    if extra_args_provider is not None:
        parser = extra_args_provider(parser)
    return parser


def configs_from_args(args, world_size: int):
    """(ModelConfig, ParallelConfig, TrainConfig) from a Megatron-style namespace."""
    nq = args.num_attention_heads
    groups = args.num_query_groups if (args.group_query_attention and args.num_query_groups) else nq
    cfg = ModelConfig(
        name="megatron-args", num_layers=args.num_layers, hidden_size=args.hidden_size, ffn_hidden_size=args.ffn_hidden_size,
        num_attention_heads=nq, num_query_groups=groups, head_dim=args.kv_channels, vocab_size=args.vocab_size,
        seq_length=args.seq_length, norm="rmsnorm" if args.normalization == "RMSNorm" else "layernorm",
        activation="swiglu" if args.swiglu else "gelu", position="rope" if args.position_embedding_type == "rope" else "learned",
        rope_theta=args.rotary_base, norm_eps=args.norm_epsilon, hidden_dropout=args.hidden_dropout,
        tie_embeddings=not args.untie_embeddings_and_output_weights, init_std=args.init_method_std,
        num_experts=args.num_experts or 0, moe_top_k=args.moe_router_topk, moe_aux_loss_coeff=args.moe_aux_loss_coeff)
    tp, pp, cp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size, args.context_parallel_size
    assert world_size % (tp * pp * cp) == 0, "world size must divide by tp x pp x cp"
    pcfg = ParallelConfig(tp=tp, pp=pp, cp=cp, ep=args.expert_model_parallel_size, dp=world_size // (tp * pp * cp),
                          sequence_parallel=bool(args.sequence_parallel) or tp == 1)
    train = TrainConfig(
        micro_batch_size=args.micro_batch_size, global_batch_size=args.global_batch_size, lr=args.lr, min_lr=args.min_lr,
        weight_decay=args.weight_decay, adam_beta1=args.adam_beta1, adam_beta2=args.adam_beta2, clip_grad=args.clip_grad,
        dtype="bf16" if (args.bf16 or args.fp16) else "fp32", seed=args.seed, fused_comm=not args.no_fused_comm,
        schedule_config=args.schedule_config, dhellam=bool(args.dhellam), compute_streams=args.compute_streams,
        train_iters=args.train_iters, log_interval=args.log_interval, save=args.save, load=args.load,
        save_interval=args.save_interval, distributed_timeout_minutes=args.distributed_timeout_minutes,
        # Megatron semantics: --loss-scale fixes the factor; --fp16 without it turns the dynamic scaler on
        loss_scale=args.loss_scale if args.loss_scale is not None else 1.0,
        dynamic_loss_scale=bool(args.fp16) and args.loss_scale is None, initial_loss_scale=args.initial_loss_scale,
        loss_scale_window=args.loss_scale_window, hysteresis=args.hysteresis, min_loss_scale=args.min_loss_scale,
        label_smoothing=args.label_smoothing_factor, deterministic=args.deterministic_mode)
    return cfg, pcfg, train


def get_args():
    if _ARGS is None:
        raise RuntimeError("initialize_dhellam_megatron() has not been called")
    return _ARGS


def initialize_dhellam_megatron(megapath: Optional[str] = None, extra_args_provider: Optional[Callable] = None, argv=None,
                                init_distributed: bool = True):
    """Parses arguments, brings up torch.distributed + the parallel mesh, returns ``args``.

    The namespace additionally carries ``model_config``, ``parallel_config`` and
    ``train_config`` (this framework's dataclasses) and ``parallel_state``."""
    global _ARGS
    check_megatron_available(megapath)
    parser = build_parser(extra_args_provider)
    args = parser.parse_args(argv)
    import torch.distributed as dist
    from ..parallel import state as PS
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if init_distributed and world > 1 and not dist.is_initialized():
        PS.init_distributed(args.distributed_backend, args.distributed_timeout_minutes)
    if dist.is_initialized():
        world = dist.get_world_size()
    cfg, pcfg, train = configs_from_args(args, world)
    args.model_config, args.parallel_config, args.train_config = cfg, pcfg, train
    args.world_size = world
    args.rank = dist.get_rank() if dist.is_initialized() else 0
    args.parallel_state = PS.initialize_model_parallel(pcfg) if (init_distributed or world == 1) else None
    _ARGS = args
    return args
