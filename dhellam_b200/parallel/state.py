"""Process-group mesh: DP x PP x CP x TP with EP carved out of DP.

Supplies what the reference takes from ``megatron.core.parallel_state`` and from its own
TP shim (dhellam/adaptor/parallel_state.py:10-38): group objects, ranks and sizes for
every axis, plus the global ranks of a context-parallel ring
(``get_context_parallel_global_ranks``; dhellam/core/dsllm.py:51-57).

Rank order follows Megatron: TP varies fastest, then CP, then DP, then PP.
One process per GPU; the backend is NCCL on GPUs and gloo on CPU ranks.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config import ParallelConfig


@dataclass
class ParallelState:
    cfg: ParallelConfig
    rank: int = 0
    world: int = 1
    tp_rank: int = 0
    cp_rank: int = 0
    dp_rank: int = 0
    pp_rank: int = 0
    ep_rank: int = 0
    tp_group: object = None
    cp_group: object = None
    dp_group: object = None
    pp_group: object = None
    ep_group: object = None
    edp_group: object = None       # ranks that hold the same experts (across EP blocks and CP ranks)
    edp_ranks: List[int] = field(default_factory=lambda: [0])
    dp_cp_group: object = None            # gradient reduction group (DP x CP)
    tp_ranks: List[int] = field(default_factory=lambda: [0])
    cp_ranks: List[int] = field(default_factory=lambda: [0])
    dp_ranks: List[int] = field(default_factory=lambda: [0])
    pp_ranks: List[int] = field(default_factory=lambda: [0])
    ep_ranks: List[int] = field(default_factory=lambda: [0])
    dp_cp_ranks: List[int] = field(default_factory=lambda: [0])

    # ---- sizes
    @property
    def tp(self): return self.cfg.tp
    @property
    def cp(self): return self.cfg.cp
    @property
    def dp(self): return self.cfg.dp
    @property
    def pp(self): return self.cfg.pp
    @property
    def ep(self): return self.cfg.ep

    @property
    def sp(self) -> bool:
        return self.cfg.sequence_parallel and self.cfg.tp > 1

    def is_first_stage(self): return self.pp_rank == 0
    def is_last_stage(self): return self.pp_rank == self.cfg.pp - 1
    def pp_next(self): return self.pp_ranks[(self.pp_rank + 1) % self.cfg.pp]
    def pp_prev(self): return self.pp_ranks[(self.pp_rank - 1) % self.cfg.pp]


_STATE: Optional[ParallelState] = None


def coords(rank: int, cfg: ParallelConfig):
    tp = rank % cfg.tp
    cp = (rank // cfg.tp) % cfg.cp
    dp = (rank // (cfg.tp * cfg.cp)) % cfg.dp
    pp = rank // (cfg.tp * cfg.cp * cfg.dp)
    return tp, cp, dp, pp


def rank_of(tp, cp, dp, pp, cfg: ParallelConfig) -> int:
    return tp + cfg.tp * (cp + cfg.cp * (dp + cfg.dp * pp))


def init_distributed(backend: Optional[str] = None, timeout_minutes: float = 2.0):
    """Initialises torch.distributed from the torchrun environment if it is not yet up."""
    if dist.is_initialized():
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    kwargs = {}
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", str(rank % max(torch.cuda.device_count(), 1))))
        torch.cuda.set_device(local)
        kwargs["device_id"] = torch.device("cuda", local)
    dist.init_process_group(backend, rank=rank, world_size=world,
                            timeout=datetime.timedelta(minutes=timeout_minutes), **kwargs)


def initialize_model_parallel(cfg: ParallelConfig, backend: Optional[str] = None) -> ParallelState:
    """Creates all groups.  Every rank must call this with the same ``cfg``."""
    global _STATE
    if cfg.world == 1 and not dist.is_initialized():
        _STATE = ParallelState(cfg=cfg)
        return _STATE
    world = dist.get_world_size()
    rank = dist.get_rank()
    assert world == cfg.world, f"world size {world} != tp*cp*dp*pp = {cfg.world}"
    assert cfg.dp % cfg.ep == 0, "expert parallelism must divide data parallelism"
    tp, cp, dp, pp = coords(rank, cfg)
    st = ParallelState(cfg=cfg, rank=rank, world=world, tp_rank=tp, cp_rank=cp, dp_rank=dp, pp_rank=pp)

    def make(groups_of_ranks, attr_group, attr_ranks):
        for ranks in groups_of_ranks:
            g = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
            if rank in ranks:
                setattr(st, attr_group, g)
                setattr(st, attr_ranks, list(ranks))

    make([[rank_of(t, c, d, p, cfg) for t in range(cfg.tp)] for p in range(cfg.pp) for d in range(cfg.dp) for c in range(cfg.cp)],
         "tp_group", "tp_ranks")
    make([[rank_of(t, c, d, p, cfg) for c in range(cfg.cp)] for p in range(cfg.pp) for d in range(cfg.dp) for t in range(cfg.tp)],
         "cp_group", "cp_ranks")
    make([[rank_of(t, c, d, p, cfg) for d in range(cfg.dp)] for p in range(cfg.pp) for c in range(cfg.cp) for t in range(cfg.tp)],
         "dp_group", "dp_ranks")
    make([[rank_of(t, c, d, p, cfg) for p in range(cfg.pp)] for d in range(cfg.dp) for c in range(cfg.cp) for t in range(cfg.tp)],
         "pp_group", "pp_ranks")
    make([[rank_of(t, c, d, p, cfg) for d in range(cfg.dp) for c in range(cfg.cp)] for p in range(cfg.pp) for t in range(cfg.tp)],
         "dp_cp_group", "dp_cp_ranks")
    # EP: consecutive blocks of `ep` data-parallel ranks
    ep_groups = []
    for p in range(cfg.pp):
        for c in range(cfg.cp):
            for t in range(cfg.tp):
                for blk in range(cfg.dp // cfg.ep):
                    ep_groups.append([rank_of(t, c, blk * cfg.ep + e, p, cfg) for e in range(cfg.ep)])
    make(ep_groups, "ep_group", "ep_ranks")
    st.ep_rank = dp % cfg.ep
    # expert-data-parallel: the replicas of one expert shard, whose gradients are summed
    make([[rank_of(t, c, blk * cfg.ep + e, p, cfg) for blk in range(cfg.dp // cfg.ep) for c in range(cfg.cp)]
          for p in range(cfg.pp) for t in range(cfg.tp) for e in range(cfg.ep)], "edp_group", "edp_ranks")
    _STATE = st
    return st


def get_state() -> ParallelState:
    if _STATE is None:
        raise RuntimeError("model parallel state is not initialised")
    return _STATE


def set_state(st: Optional[ParallelState]):
    global _STATE
    _STATE = st


def destroy_model_parallel():
    global _STATE
    _STATE = None


# ---- Megatron-style getters (names used by the reference) -------------------
def get_tensor_model_parallel_group(): return get_state().tp_group
def get_tensor_model_parallel_rank(): return get_state().tp_rank
def get_tensor_model_parallel_world_size(): return get_state().tp
def get_context_parallel_group(): return get_state().cp_group
def get_context_parallel_rank(): return get_state().cp_rank
def get_context_parallel_world_size(): return get_state().cp
def get_context_parallel_global_ranks(): return get_state().cp_ranks
def get_data_parallel_group(): return get_state().dp_group
def get_data_parallel_rank(): return get_state().dp_rank
def get_data_parallel_world_size(): return get_state().dp
def get_pipeline_model_parallel_group(): return get_state().pp_group
def get_pipeline_model_parallel_rank(): return get_state().pp_rank
def get_pipeline_model_parallel_world_size(): return get_state().pp
def get_expert_model_parallel_group(): return get_state().ep_group
def get_expert_model_parallel_rank(): return get_state().ep_rank
def get_expert_model_parallel_world_size(): return get_state().ep
def is_pipeline_first_stage(): return get_state().is_first_stage()
def is_pipeline_last_stage(): return get_state().is_last_stage()
