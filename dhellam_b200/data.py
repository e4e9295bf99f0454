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


# --------------------------------------------------------------------------- real token data
class TokenFileDataset:
    """Samples ``[seq+1]`` windows from a flat file of token ids (``uint16`` / ``int32`` /
    ``int64``, the payload of a Megatron ``.bin`` file or any ``numpy`` memmap-able dump).

    Sample ``i`` of epoch ``e`` starts at a position drawn from a permutation seeded with
    ``(seed, e)``; the file is memory-mapped, nothing is read up front.  This covers what the
    reference gets from Megatron's ``GPTDataset`` for its demo run (script/run.sh:60-75,
    ``--data-path``); document boundaries and blending are not modelled."""

    def __init__(self, path: str, seq_length: int, dtype: str = "int32", seed: int = 1234):
        import numpy as np
        self.np = np
        self.tokens = np.memmap(path, dtype=np.dtype(dtype), mode="r")
        self.seq = seq_length
        self.n = (len(self.tokens) - 1) // seq_length
        if self.n <= 0:
            raise ValueError(f"{path}: {len(self.tokens)} tokens are fewer than one sample of {seq_length + 1}")
        self.seed = seed
        self._perm_epoch, self._perm = -1, None

    def __len__(self):
        return self.n

    def sample(self, index: int) -> torch.Tensor:
        epoch, i = divmod(index, self.n)
        if epoch != self._perm_epoch:
            self._perm = self.np.random.default_rng((self.seed, epoch)).permutation(self.n)
            self._perm_epoch = epoch
        start = int(self._perm[i]) * self.seq
        return torch.from_numpy(self.np.asarray(self.tokens[start:start + self.seq + 1]).astype(self.np.int64))

    def batch(self, first_index: int, batch: int) -> torch.Tensor:
        """``[batch, seq+1]`` of consecutive sample indices."""
        return torch.stack([self.sample(first_index + j) for j in range(batch)])


def broadcast_batch_on_tp_group(ps, sample, batch: int, seq_plus_one: int, device="cpu") -> torch.Tensor:
    """Hands the ``[batch, seq+1]`` token sample that only the first rank of each
    tensor-parallel group read from disk to the rest of the group (``sample`` is ``None``
    on the others).  Same purpose as the reference's patched ``get_batch_on_this_tp_rank``
    (megatron.patch:827-910), which broadcasts tokens, labels, loss mask and position ids;
    labels, mask and positions are derived on every rank here (``make_microbatch``), so one
    tensor crosses the group instead of four."""
    import torch.distributed as dist
    if ps.tp == 1 or ps.tp_group is None:
        return sample
    dev = torch.device(device)
    if ps.tp_rank == 0:
        buf = sample.to(device=dev, dtype=torch.int64).contiguous()
        assert tuple(buf.shape) == (batch, seq_plus_one)
    else:
        buf = torch.empty((batch, seq_plus_one), dtype=torch.int64, device=dev)
    dist.broadcast(buf, src=ps.tp_ranks[0], group=ps.tp_group)
    return buf


def file_step_batches(ds: TokenFileDataset, cfg: ModelConfig, train: TrainConfig, ps, step: int, device) -> List[MicroBatch]:
    """All micro-batches of one optimizer step for this rank from a token file: data-parallel
    rank ``d`` takes every ``dp``-th micro-batch, the first rank of each tensor-parallel group
    reads and the group receives a broadcast."""
    n = train.num_microbatches(ps.dp)
    B = train.micro_batch_size
    out = []
    dev = torch.device(device)
    bdev = dev if dev.type == "cuda" else torch.device("cpu")
    for i in range(n):
        first = ((step * n + i) * ps.dp + ps.dp_rank) * B
        sample = ds.batch(first, B) if ps.tp_rank == 0 else None
        sample = broadcast_batch_on_tp_group(ps, sample, B, cfg.seq_length + 1, bdev)
        seed = (train.seed * 1000003 + step * 8191 + ps.dp_rank * 127 + i) & 0x7FFFFFFF
        out.append(make_microbatch(cfg, ps, sample.cpu() if sample.is_cuda else sample, i, seed, device))
    return out
