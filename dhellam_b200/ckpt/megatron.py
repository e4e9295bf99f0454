"""Checkpoints in the Megatron distributed-checkpoint layout, with the fold map.

Directory layout (Megatron-core ``dist_checkpointing`` with the ``torch_dist`` backend)::

    <save>/latest_checkpointed_iteration.txt
    <save>/iter_0000010/metadata.json      sharded_backend / common_backend descriptors
    <save>/iter_0000010/common.pt          iteration, arguments, RNG of rank 0, optimizer step
    <save>/iter_0000010/.metadata          ``torch.distributed.checkpoint`` metadata (pickled ``Metadata``:
                                           key -> global size, dtype and the chunks that tile it)
    <save>/iter_0000010/__{rank}_0.distcp  the chunks written by one rank, in the format of
                                           ``torch.distributed.checkpoint.FileSystemWriter``
    <save>/iter_0000010/optim_{rank}.pt    this rank's optimizer shard + its CPU / CUDA RNG state
                                           (a ``torch.save`` file; same parallel layout on resume)

The weight files are genuine ``torch.distributed.checkpoint`` (DCP) files: they are written by
``dcp.save`` through a planner that emits one write item per tensor-parallel piece, so
``dcp.load`` (and therefore Megatron-core's ``torch_dist`` reader, which is built on it) can
open them under the canonical keys below.

Tensors are stored under Megatron-core's canonical GPT keys
(``decoder.layers.{i}.self_attention.linear_qkv.weight`` ...), indexed by the *model* layer,
not by the folded slot: the reference's ``DSLLM`` has folded parameter names
(``dctb.{j}.column_attn_weight_first`` ..., dhellam/core/dstb.py:1373-1389) and defines no
sharded state dict, so its checkpoints could not be exchanged with an unfolded model; here
``fold map``: slot (stage p, pair j, first|second) <-> layer index is applied on save and
load, and the packed QKV rows are converted to Megatron's per-group interleave
``[q heads of group g | k_g | v_g]``.  Because every piece records its offset in the global
tensor, a checkpoint written with one tensor/pipeline/expert-parallel layout loads into
another.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config import ModelConfig, to_dict

# ----------------------------------------------------------------------------- names
LAYER_KEYS = {
    "ln_attn_weight": "self_attention.linear_qkv.layer_norm_weight",
    "ln_attn_bias": "self_attention.linear_qkv.layer_norm_bias",
    "column_attn_weight": "self_attention.linear_qkv.weight",
    "linear_attn_weight": "self_attention.linear_proj.weight",
    "ln_mlp_weight": "mlp.linear_fc1.layer_norm_weight",
    "ln_mlp_bias": "mlp.linear_fc1.layer_norm_bias",
    "column_mlp_weight": "mlp.linear_fc1.weight",
    "linear_mlp_weight": "mlp.linear_fc2.weight",
    "router_weight": "mlp.router.weight",
}
HEAD_KEYS = {
    "word_embeddings": "embedding.word_embeddings.weight",
    "position_embeddings": "embedding.position_embeddings.weight",
    "final_ln_weight": "decoder.final_layernorm.weight",
    "final_ln_bias": "decoder.final_layernorm.bias",
    "output_weight": "output_layer.weight",
}


def fold_map(num_layers: int, pp: int) -> Dict[Tuple[int, int, str], int]:
    """``(stage, pair index, "first"|"second") -> model layer index``."""
    c = num_layers // (2 * pp)
    m = {}
    for p in range(pp):
        for j in range(c):
            first = p * c + j
            m[(p, j, "first")] = first
            m[(p, j, "second")] = num_layers - 1 - first
    return m


# ----------------------------------------------------------------------------- QKV packing
def qkv_shard_to_megatron(w, cfg: ModelConfig, tp: int):
    """``[q heads | k heads | v heads]`` rows of one rank -> per-group interleave."""
    d = cfg.head_dim
    nq, nkv = cfg.num_attention_heads // tp, max(cfg.num_query_groups // tp, 1)
    g = nq // nkv
    q, k, v = w[: nq * d], w[nq * d:(nq + nkv) * d], w[(nq + nkv) * d:]
    parts = []
    for i in range(nkv):
        parts += [q[i * g * d:(i + 1) * g * d], k[i * d:(i + 1) * d], v[i * d:(i + 1) * d]]
    return torch.cat(parts, 0)


def qkv_megatron_to_shard(w, cfg: ModelConfig, tp: int):
    d = cfg.head_dim
    nq, nkv = cfg.num_attention_heads // tp, max(cfg.num_query_groups // tp, 1)
    g = nq // nkv
    rows = (g + 2) * d
    qs, ks, vs = [], [], []
    for i in range(nkv):
        blk = w[i * rows:(i + 1) * rows]
        qs.append(blk[: g * d]); ks.append(blk[g * d:(g + 1) * d]); vs.append(blk[(g + 1) * d:])
    return torch.cat(qs + ks + vs, 0)


# ----------------------------------------------------------------------------- pieces
def _pieces_for(base: str, t: torch.Tensor, cfg: ModelConfig, ps):
    """Returns ``(global shape, [(offsets tuple, tensor)], writer?)`` for one local tensor."""
    tp, r = ps.tp, ps.tp_rank
    shape = list(t.shape)
    writer_rep = ps.tp_rank == 0            # replicated tensors are written once
    if base == "column_attn_weight":
        m = qkv_shard_to_megatron(t, cfg, tp)
        return [shape[0] * tp, shape[1]], [((r * shape[0], 0), m)], True
    if base in ("linear_attn_weight", "linear_mlp_weight"):
        return [shape[0], shape[1] * tp], [((0, r * shape[1]), t)], True
    if base == "column_mlp_weight":
        if cfg.gated:
            f = shape[0] // 2
            return [shape[0] * tp, shape[1]], [((r * f, 0), t[:f]), ((f * tp + r * f, 0), t[f:])], True
        return [shape[0] * tp, shape[1]], [((r * shape[0], 0), t)], True
    if base in ("word_embeddings", "output_weight"):
        return [shape[0] * tp, shape[1]], [((r * shape[0], 0), t)], True
    return shape, [((0,) * len(shape), t)], writer_rep


def canonical_items(model, tensors_of=lambda p: p.data):
    """Yields ``(key, global shape, pieces, is_writer)`` for every parameter of this rank's
    stage, under canonical names.  ``tensors_of`` picks what to store for a parameter (its
    value, its fp32 master, a moment ...)."""
    cfg, ps = model.cfg, model.ps
    for m in model.dctb:
        for which, idx in (("first", m.first_index), ("second", m.second_index)):
            for base in m.shapes:
                p = getattr(m, f"{base}_{which}")
                t = tensors_of(p)
                if base in ("expert_column_weight", "expert_linear_weight"):
                    el = t.shape[0]
                    for e in range(el):
                        ge = ps.ep_rank * el + e
                        sub = "linear_fc1" if base == "expert_column_weight" else "linear_fc2"
                        key = f"decoder.layers.{idx}.mlp.experts.local_experts.{ge}.{sub}.weight"
                        b2 = "column_mlp_weight" if base == "expert_column_weight" else "linear_mlp_weight"
                        gshape, pieces, w = _pieces_for(b2, t[e], cfg, ps)
                        yield key, gshape, pieces, w
                    continue
                key = f"decoder.layers.{idx}.{LAYER_KEYS[base]}"
                gshape, pieces, w = _pieces_for(base, t, cfg, ps)
                yield key, gshape, pieces, w
    if model.dchb is not None:
        for base in model.dchb.shapes:
            p = getattr(model.dchb, base)
            gshape, pieces, w = _pieces_for(base, tensors_of(p), cfg, ps)
            yield HEAD_KEYS[base], gshape, pieces, w


# ----------------------------------------------------------------------------- save
def _iter_dir(root: str, iteration: int) -> str:
    return os.path.join(root, f"iter_{iteration:07d}")


def _dcp_save(d: str, pieces):
    """Writes ``pieces`` = ``[(key, global shape, offsets, cpu tensor)]`` of this rank as
    ``torch.distributed.checkpoint`` files.  Every rank of the job calls it (ranks without
    pieces take part in the planning collectives with an empty plan); the coordinator writes
    ``.metadata`` with, per key, the global size and all ranks' chunks."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import DefaultSavePlanner, FileSystemWriter
    from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
    from torch.distributed.checkpoint.planner import SavePlan, TensorWriteData, WriteItem, WriteItemType

    table = {(k, offs): t for k, _, offs, t in pieces}

    class PiecePlanner(DefaultSavePlanner):
        def create_local_plan(self):
            items = []
            for k, gshape, offs, t in pieces:
                chunk = ChunkStorageMetadata(offsets=torch.Size(offs), sizes=t.size())
                items.append(WriteItem(index=MetadataIndex(k, torch.Size(offs)), type=WriteItemType.SHARD,
                                       tensor_data=TensorWriteData(chunk=chunk, properties=TensorProperties.create_from_tensor(t),
                                                                   size=torch.Size(gshape))))
            self.plan = SavePlan(items, planner_data=dict(getattr(self, "mappings", None) or {}))
            return self.plan

        def resolve_data(self, write_item):
            return table[(write_item.index.fqn, tuple(write_item.index.offset))]

    no_dist = not (dist.is_initialized() and dist.get_world_size() > 1)
    dcp.save({}, storage_writer=FileSystemWriter(d, single_file_per_rank=True, sync_files=False),
             planner=PiecePlanner(), no_dist=no_dist)


def save_checkpoint(save_dir: str, iteration: int, model, optimizer=None, args: Optional[dict] = None):
    """Writes one checkpoint.  Every rank calls this; ranks that hold a data-parallel or
    context-parallel replica of the weights write nothing but their optimizer shard."""
    ps = model.ps
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    d = _iter_dir(save_dir, iteration)
    os.makedirs(d, exist_ok=True)
    # data-parallel rank 0 writes the dense weights; the first `ep` data-parallel ranks each write their experts
    weight_writer = ps.dp_rank < max(ps.ep, 1) and ps.cp_rank == 0
    pieces = []                        # (key, global shape, offsets, tensor)
    if weight_writer:
        dense_writer = ps.dp_rank == 0
        for key, gshape, pcs, writer in canonical_items(model):
            is_expert = ".experts.local_experts." in key
            if not writer or (not is_expert and not dense_writer):
                continue
            for offs, t in pcs:
                pieces.append((key, tuple(gshape), tuple(offs), t.detach().to("cpu").contiguous()))
    _dcp_save(d, pieces)
    if optimizer is not None:
        osd = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in optimizer.state_dict().items()}
        osd["rng_state"] = {"cpu": torch.get_rng_state(),
                            "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}
        torch.save(osd, os.path.join(d, f"optim_{rank}.pt"))
    if rank == 0:
        with open(os.path.join(d, "metadata.json"), "w") as fp:
            json.dump({"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch",
                       "common_backend_version": 1, "writer": "dhellam_b200"}, fp)
        common = {"iteration": iteration, "args": args or {}, "model_config": to_dict(model.cfg),
                  "parallel": {"tp": ps.tp, "pp": ps.pp, "cp": ps.cp, "dp": ps.dp, "ep": ps.ep},
                  "fold_map": {f"{p}.{j}.{w}": l for (p, j, w), l in fold_map(model.cfg.num_layers, ps.pp).items()},
                  "rng_state": torch.get_rng_state(), "optimizer_step": getattr(optimizer, "step_count", 0),
                  "checkpoint_version": 3.0}
        torch.save(common, os.path.join(d, "common.pt"))
        with open(os.path.join(save_dir, "latest_checkpointed_iteration.txt"), "w") as fp:
            fp.write(str(iteration))
    if dist.is_initialized() and world > 1:
        dist.barrier()
    return d


# ----------------------------------------------------------------------------- load
def read_latest_iteration(load_dir: str) -> Optional[int]:
    p = os.path.join(load_dir, "latest_checkpointed_iteration.txt")
    if not os.path.exists(p):
        return None
    return int(open(p).read().strip())


class _Reader:
    """Reads whole tensors out of a DCP checkpoint directory (each rank reads for itself)."""

    def __init__(self, d: str):
        from torch.distributed.checkpoint import FileSystemReader
        self.d = d
        self.meta = FileSystemReader(d).read_metadata()
        self.index = {k: v for k, v in self.meta.state_dict_metadata.items() if hasattr(v, "chunks")}

    def shape(self, key: str):
        return list(self.index[key].size)

    def full(self, key: str) -> torch.Tensor:
        """Assembles the whole tensor of ``key`` from its chunks."""
        return self.full_many([key])[key]

    def full_many(self, keys) -> Dict[str, torch.Tensor]:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint import FileSystemReader
        sd = {k: torch.empty(tuple(self.index[k].size), dtype=self.index[k].properties.dtype) for k in keys}
        if sd:
            dcp.load(sd, storage_reader=FileSystemReader(self.d), no_dist=True)
        return sd


def load_checkpoint(load_dir: str, model, optimizer=None, iteration: Optional[int] = None, strict: bool = True) -> int:
    """Loads weights (re-sharding them for this rank's layout) and, when the parallel layout
    matches, the optimizer shard.  Returns the iteration."""
    from ..models.sharding import shard_head, shard_layer
    if iteration is None:
        iteration = read_latest_iteration(load_dir)
        if iteration is None:
            raise FileNotFoundError(f"no latest_checkpointed_iteration.txt under {load_dir}")
    d = _iter_dir(load_dir, iteration)
    rd = _Reader(d)
    cfg, ps = model.cfg, model.ps
    # canonical (Megatron) full tensors -> this framework's full layout -> this rank's shards
    def full_layer(idx):
        want = {base: f"decoder.layers.{idx}.{sub}" for base, sub in LAYER_KEYS.items() if f"decoder.layers.{idx}.{sub}" in rd.index}
        ekeys = []
        if cfg.is_moe:
            for e in range(cfg.num_experts):
                ekeys += [f"decoder.layers.{idx}.mlp.experts.local_experts.{e}.linear_fc1.weight",
                          f"decoder.layers.{idx}.mlp.experts.local_experts.{e}.linear_fc2.weight"]
        got = rd.full_many(list(want.values()) + ekeys)
        full = {}
        for base, key in want.items():
            t = got[key]
            if base == "column_attn_weight":
                t = qkv_megatron_to_shard(t, cfg, 1)
            full[base] = t
        if cfg.is_moe:
            full["expert_column_weight"] = torch.stack([got[k] for k in ekeys[0::2]])
            full["expert_linear_weight"] = torch.stack([got[k] for k in ekeys[1::2]])
        return full
    for m in model.dctb:
        for which, idx in (("first", m.first_index), ("second", m.second_index)):
            shards = shard_layer(full_layer(idx), cfg, ps.tp, ps.tp_rank, ps.ep, ps.ep_rank)
            with torch.no_grad():
                for base in m.shapes:
                    if base not in shards:
                        if strict:
                            raise KeyError(f"layer {idx}: {base} missing from the checkpoint")
                        continue
                    getattr(m, f"{base}_{which}").copy_(shards[base].to(model.dtype))
    if model.dchb is not None:
        want = {base: key for base, key in HEAD_KEYS.items() if key in rd.index}
        got = rd.full_many(list(want.values()))
        shards = shard_head({base: got[key] for base, key in want.items()}, cfg, ps.tp, ps.tp_rank)
        with torch.no_grad():
            for base in model.dchb.shapes:
                getattr(model.dchb, base).copy_(shards[base].to(model.dtype))
    common = torch.load(os.path.join(d, "common.pt"), map_location="cpu", weights_only=False)
    if optimizer is not None:
        rank = dist.get_rank() if dist.is_initialized() else 0
        same = common["parallel"] == {"tp": ps.tp, "pp": ps.pp, "cp": ps.cp, "dp": ps.dp, "ep": ps.ep}
        p = os.path.join(d, f"optim_{rank}.pt")
        if same and os.path.exists(p):
            sd = torch.load(p, map_location="cpu", weights_only=False)
            rng = sd.pop("rng_state", None)
            optimizer.load_state_dict({k: (v.to(optimizer.master.device) if torch.is_tensor(v) else v) for k, v in sd.items()})
            if rng is not None:                   # every rank continues its own random streams
                torch.set_rng_state(rng["cpu"])
                if rng.get("cuda") is not None and torch.cuda.is_available():
                    torch.cuda.set_rng_state(rng["cuda"])
        else:
            # different layout: moments restart, master weights follow the loaded parameters
            import warnings
            warnings.warn(f"checkpoint {d} was written with parallel layout {common['parallel']}, this run uses "
                          f"tp={ps.tp} pp={ps.pp} cp={ps.cp} dp={ps.dp} ep={ps.ep}: weights were re-sharded, but the Adam "
                          "moments restart from zero (the optimizer shards are only reloadable in the layout that wrote them)")
            optimizer.master.copy_(model.flat_param[optimizer.lo:optimizer.hi].float())
            optimizer.step_count = int(common.get("optimizer_step", 0))
    return int(common["iteration"])
