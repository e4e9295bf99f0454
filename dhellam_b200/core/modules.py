"""Folded model modules: ``DSTB`` (a pair of transformer layers), ``DSHB`` (embedding +
loss head) and ``DSLLM`` (the stage's stack), with the reference's class and parameter
names (dhellam/core/dstb.py:1366-1468, dhellam/core/dshb.py:244-289,
dhellam/core/dsllm.py:43-106).

Parameters are views into one flat buffer per stage and ``main_grad`` attributes are views
into one flat fp32 gradient buffer, so the optimizer and the data-parallel reduction work on
two contiguous tensors instead of a list of parameters.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..config import ModelConfig, ParallelConfig, TrainConfig
from ..models.head import HeadParams
from ..models.transformer import LayerParams, layer_param_shapes
from ..parallel.state import ParallelState

_ALIGN = 128   # elements; keeps every parameter 256-byte aligned for TMA


def _dtype_of(train: TrainConfig):
    return torch.bfloat16 if train.dtype == "bf16" else torch.float32


def _is_norm(name: str) -> bool:
    return name.startswith("ln_") or name.startswith("final_ln")


class DSTB(nn.Module):
    """Block pair: the weights of layer ``i`` ("first") and of layer ``L-1-i`` ("second")."""

    def __init__(self, cfg: ModelConfig, ps: ParallelState, first_index: int, second_index: int):
        super().__init__()
        self.cfg, self.first_index, self.second_index = cfg, first_index, second_index
        self.shapes = layer_param_shapes(cfg, ps.tp, ps.ep)
        self._order = [(n, sfx) for sfx in ("first", "second") for n in self.shapes]

    def param_specs(self):
        """``[(attribute name, shape, layer index, base name)]`` in storage order."""
        out = []
        for n, sfx in self._order:
            idx = self.first_index if sfx == "first" else self.second_index
            out.append((f"{n}_{sfx}", self.shapes[n], idx, n))
        return out

    def layer_params(self, which: str) -> LayerParams:
        return LayerParams({n: getattr(self, f"{n}_{which}") for n in self.shapes})


class DSHB(nn.Module):
    """Head block on the first pipeline stage: word embedding (tied LM head), final norm."""

    def __init__(self, cfg: ModelConfig, ps: ParallelState):
        super().__init__()
        self.cfg = cfg
        vl = cfg.vocab_size // ps.tp
        assert cfg.vocab_size % ps.tp == 0, "vocabulary must divide by the tensor-parallel size"
        self.shapes = {"word_embeddings": (vl, cfg.hidden_size), "final_ln_weight": (cfg.hidden_size,)}
        if cfg.norm == "layernorm":
            self.shapes["final_ln_bias"] = (cfg.hidden_size,)
        if not cfg.tie_embeddings:
            self.shapes["output_weight"] = (vl, cfg.hidden_size)
        if cfg.position == "learned":
            self.shapes["position_embeddings"] = (cfg.seq_length, cfg.hidden_size)

    def param_specs(self):
        return [(n, s, -1, n) for n, s in self.shapes.items()]

    def head_params(self) -> HeadParams:
        return HeadParams({n: getattr(self, n) for n in self.shapes})


class DSLLM(nn.Module):
    """The folded model of one pipeline stage.

    ``num_layers`` must divide by ``2 * pp``; the stage owns ``num_layers / (2 pp)`` block
    pairs and, on the first stage, the head block.
    """

    def __init__(self, cfg: ModelConfig, ps: ParallelState, train: TrainConfig, device="cpu", seed: Optional[int] = None,
                 init: str = "random"):
        super().__init__()
        assert cfg.num_layers % (2 * ps.pp) == 0, "number of layers must divide by 2 x pipeline size"
        self.cfg, self.ps, self.train_cfg = cfg, ps, train
        self.device = torch.device(device)
        self.dtype = _dtype_of(train)
        c = cfg.num_layers // (2 * ps.pp)
        self.pre_process = ps.pp_rank == 0
        self.dctb = nn.ModuleList()
        for j in range(c):
            first = ps.pp_rank * c + j
            self.dctb.append(DSTB(cfg, ps, first, cfg.num_layers - 1 - first))
        self.dchb = DSHB(cfg, ps) if self.pre_process else None
        self._allocate(seed if seed is not None else train.seed, init)
        self.blocks = [(m.layer_params("first"), m.layer_params("second")) for m in self.dctb]
        self.head = self.dchb.head_params() if self.dchb is not None else None

    # ------------------------------------------------------------------ storage
    def _specs(self):
        specs = []
        for j, m in enumerate(self.dctb):
            for attr, shape, idx, base in m.param_specs():
                specs.append((m, f"dctb.{j}.{attr}", attr, shape, idx, base))
        if self.dchb is not None:
            for attr, shape, idx, base in self.dchb.param_specs():
                specs.append((self.dchb, f"dchb.{attr}", attr, shape, idx, base))
        return specs

    def _allocate(self, seed: int, init: str):
        specs = self._specs()
        offs, total = [], 0
        for _, _, _, shape, _, _ in specs:
            offs.append(total)
            n = math.prod(shape)
            total += (n + _ALIGN - 1) // _ALIGN * _ALIGN
        self.flat_param = torch.zeros(total, dtype=self.dtype, device=self.device)
        self.flat_grad = torch.zeros(total, dtype=torch.float32, device=self.device)
        self.param_index: Dict[str, Tuple[int, tuple]] = {}
        for (mod, full, attr, shape, idx, base), off in zip(specs, offs):
            n = math.prod(shape)
            view = self.flat_param[off:off + n].view(shape)
            p = nn.Parameter(view, requires_grad=False)
            p.main_grad = self.flat_grad[off:off + n].view(shape)
            p.sequence_parallel = _is_norm(base)
            p.layer_index = idx
            p.base_name = base
            p.is_expert = base.startswith("expert_")
            setattr(mod, attr, p)
            self.param_index[full] = (off, tuple(shape))
            if init != "none":
                self._init_param(p, base, idx, seed)

    def _init_param(self, p, base: str, layer_idx: int, seed: int):
        cfg, ps = self.cfg, self.ps
        with torch.no_grad():
            if _is_norm(base):
                p.fill_(0.0 if base.endswith("bias") else 1.0)
                return
            g = torch.Generator(device="cpu")
            key = sum(ord(ch) * (i + 1) for i, ch in enumerate(base)) % 9973
            rank_key = ps.tp_rank if not base.startswith("expert_") else ps.tp_rank + 131 * ps.ep_rank
            if base == "router_weight":
                rank_key = 0
            g.manual_seed(seed * 1000003 + (layer_idx + 2) * 10007 + key * 101 + rank_key)
            if self.device.type == "cuda":
                gd = torch.Generator(device=self.device)
                gd.manual_seed(g.initial_seed())
                p.copy_(torch.empty(p.shape, dtype=torch.float32, device=self.device).normal_(0.0, cfg.init_std, generator=gd))
            else:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, cfg.init_std, generator=g))

    # ------------------------------------------------------------------ API kept from the reference
    def set_input_tensor(self, input_tensor):
        """Receives ``[backward tensor, forward tensor]`` on stages after the first
        (dhellam/core/dsllm.py:75-83)."""
        if input_tensor is None:
            self.input_tensor = [None, None]
            return
        if not isinstance(input_tensor, (list, tuple)):
            input_tensor = [input_tensor]
        assert len(input_tensor) == 2, "the folded stage exchanges exactly two tensors"
        self.input_tensor = list(input_tensor)

    def zero_grad_buffer(self):
        self.flat_grad.zero_()

    def named_main_grads(self):
        for name, p in self.named_parameters():
            yield name, p.main_grad

    def load_full_layer_weights(self, layer_index: int, full: Dict[str, torch.Tensor]):
        """Loads one layer from unsharded tensors (see ``models.sharding``)."""
        from ..models.sharding import shard_layer
        shards = shard_layer(full, self.cfg, self.ps.tp, self.ps.tp_rank, self.ps.ep, self.ps.ep_rank)
        for m in self.dctb:
            for which, idx in (("first", m.first_index), ("second", m.second_index)):
                if idx == layer_index:
                    with torch.no_grad():
                        for n, t in shards.items():
                            getattr(m, f"{n}_{which}").copy_(t.to(self.dtype))
                    return True
        return False

    def load_full_head_weights(self, full: Dict[str, torch.Tensor]):
        from ..models.sharding import shard_head
        if self.dchb is None:
            return
        shards = shard_head(full, self.cfg, self.ps.tp, self.ps.tp_rank)
        with torch.no_grad():
            for n, t in shards.items():
                getattr(self.dchb, n).copy_(t.to(self.dtype))
