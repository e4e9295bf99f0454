"""Synthetic token data of a named shape, and micro-batch construction.

The reference's dataset blob is not part of its repository and its demo run only needs
token ids of the right shape (script/run.sh:60-75); its head block can also fabricate a
batch on the device (``initialize_pre_process_data``, dhellam/core/dshb.py:53-73).  Here
every rank derives its micro-batches from ``(seed, step, micro-batch index, dp rank)``, so
no broadcast over the tensor-parallel group is needed (the reference broadcasts tokens,
labels and masks: megatron.patch:827-910).

Rows are sequence-first (row = s * batch + b).  With context parallelism a rank holds
sequence chunks ``r`` and ``2c-1-r`` of ``2c`` (the load-balanced causal split of
dhellam/core/dstb.py:167-169).
"""
from __future__ import annotations

from typing import List

import torch

from .config import ModelConfig, TrainConfig
from .core.engine import MicroBatch


def cp_chunk_positions(seq: int, cp: int, r: int) -> torch.Tensor:
    """Sequence positions held by context-parallel rank ``r`` (ascending)."""
    if cp == 1:
        return torch.arange(seq, dtype=torch.int32)
    assert seq % (2 * cp) == 0, "sequence must divide by 2 x context-parallel size"
    c = seq // (2 * cp)
    a = torch.arange(r * c, (r + 1) * c, dtype=torch.int32)
    b = torch.arange((2 * cp - 1 - r) * c, (2 * cp - r) * c, dtype=torch.int32)
    return torch.cat([a, b])


def synthetic_tokens(cfg: ModelConfig, batch: int, seed: int) -> torch.Tensor:
    """``[batch, seq+1]`` ids uniform in ``[0, vocab)`` from ``seed`` (CPU generator, so the
    stream is identical on every rank and device)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (batch, cfg.seq_length + 1), generator=g, dtype=torch.int64)


def make_microbatch(cfg: ModelConfig, ps, sample: torch.Tensor, index: int, seed: int, device, pin: bool = False) -> MicroBatch:
    """Builds this rank's micro-batch from ``sample [B, S+1]`` (tokens; labels are the shift by one)."""
    B = sample.shape[0]
    pos = cp_chunk_positions(cfg.seq_length, ps.cp, ps.cp_rank)
    tok = sample[:, :-1][:, pos.long()]          # [B, S_local]
    lab = sample[:, 1:][:, pos.long()]
    tokens = tok.t().contiguous().reshape(-1).to(torch.int32)       # sequence-first rows
    labels = lab.t().contiguous().reshape(-1).to(torch.int32)
    positions = pos[:, None].expand(-1, B).contiguous().reshape(-1)
    mask = torch.ones(tokens.numel(), dtype=torch.float32)
    T = tokens.numel()
    lo, hi = ps.tp_rank * (T // ps.tp), (ps.tp_rank + 1) * (T // ps.tp)
    dev = torch.device(device)
    if dev.type == "cuda":
        host = [tokens, labels, mask, positions]
        if pin:
            host = [t.pin_memory() for t in host]
        tokens, labels, mask, positions = [t.to(dev, non_blocking=True) for t in host]
    return MicroBatch(index=index, tokens=tokens, labels=labels, loss_mask=mask, positions=positions, batch=B, seed=seed,
                      positions_local=positions[lo:hi])


def synthetic_step_batches(cfg: ModelConfig, train: TrainConfig, ps, step: int, device) -> List[MicroBatch]:
    """All micro-batches of one optimizer step for this rank."""
    n = train.num_microbatches(ps.dp)
    out = []
    for i in range(n):
        seed = (train.seed * 1000003 + step * 8191 + ps.dp_rank * 127 + i) & 0x7FFFFFFF
        sample = synthetic_tokens(cfg, train.micro_batch_size, seed)
        out.append(make_microbatch(cfg, ps, sample, i, seed, device))
    return out
