"""Token-file dataset, the broadcast of a batch inside a tensor-parallel group, the blackboard
and the launch templates."""
import numpy as np
import torch

from dhellam_b200.config import ParallelConfig, TrainConfig, preset
from dhellam_b200.data import TokenFileDataset, broadcast_batch_on_tp_group, file_step_batches

from dist_utils import run_ranks


def _token_file(tmp_path, n=5000, vocab=256):
    path = str(tmp_path / "tokens.bin")
    np.arange(n, dtype=np.int32).__mod__(vocab).astype(np.int32).tofile(path)
    return path


def test_token_file_dataset_windows_and_epochs(tmp_path):
    path = _token_file(tmp_path, vocab=1 << 30)          # ids = positions: every window is recognisable
    ds = TokenFileDataset(path, 64, "int32", seed=7)
    assert len(ds) == (5000 - 1) // 64
    seen = set()
    for i in range(len(ds)):
        s = ds.sample(i)
        assert s.shape == (65,) and s.dtype == torch.int64
        # a window of consecutive ids (mod vocab): label = next token
        assert torch.equal(s[:-1] + 1, s[1:])
        seen.add(int(s[0]))
    assert len(seen) == len(ds)                          # a permutation: every window exactly once per epoch
    first_epoch0, first_epoch1 = ds.sample(0), ds.sample(len(ds))
    assert ds.batch(3, 4).shape == (4, 65)
    again = TokenFileDataset(path, 64, "int32", seed=7)
    assert torch.equal(again.sample(0), first_epoch0) and torch.equal(again.sample(len(ds)), first_epoch1)


def _bcast_worker(rank, world, path):
    from dhellam_b200.parallel import state as PS
    cfg = preset("tiny-llama", seq_length=64, vocab_size=256)
    ps = PS.initialize_model_parallel(ParallelConfig(tp=2))
    ds = TokenFileDataset(path, 64, "int32", seed=7)
    ref = ds.batch(0, 2)
    got = broadcast_batch_on_tp_group(ps, ref if ps.tp_rank == 0 else None, 2, 65)
    assert torch.equal(got, ref)
    train = TrainConfig(micro_batch_size=2, global_batch_size=4, dtype="fp32")
    mbs = file_step_batches(ds, cfg, train, ps, 0, "cpu")
    assert len(mbs) == 2
    # both ranks hold the same full micro-batch (sequence-first rows), labels shifted by one
    tok = ds.batch(0, 2)[:, :-1].t().reshape(-1).to(torch.int32)
    assert torch.equal(mbs[0].tokens, tok)
    assert torch.equal(mbs[0].labels, ds.batch(0, 2)[:, 1:].t().reshape(-1).to(torch.int32))


def test_batch_broadcast_inside_tensor_parallel_group(tmp_path):
    run_ranks(_bcast_worker, 2, _token_file(tmp_path))


def test_blackboard_and_launch_templates():
    from dhellam_b200.common import GLOBAL_VARIABLES, launch_on_stream, launch_with_event
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama")
    train = TrainConfig(micro_batch_size=1, global_batch_size=2, dtype="fp32")
    tr = Trainer(cfg, ParallelConfig(), train, device=torch.device("cpu"), ps=PS.initialize_model_parallel(ParallelConfig()))
    assert GLOBAL_VARIABLES["loss_scale_func"] == tr.optimizer.scale_loss
    mbs = [make_microbatch(cfg, tr.ps, synthetic_tokens(cfg, 1, 3 + i), i, 3 + i, tr.device) for i in range(2)]
    loss = tr.train_step(mbs)
    assert GLOBAL_VARIABLES["loss"] is loss
    out, ms = launch_on_stream(lambda a, b: a + b, 2, 3, profiling=True)
    assert out == 5 and ms >= 0.0
    out, ev = launch_with_event(lambda a: a * 2, 4)
    assert out == 8 and (ev is None or hasattr(ev, "record"))


def _chunk_worker(rank, world):
    import torch.distributed as dist
    from dhellam_b200.ops import comm as C
    from dhellam_b200.parallel import state as PS
    ps = PS.initialize_model_parallel(ParallelConfig(tp=world))
    g = torch.Generator().manual_seed(5)
    shards = [torch.randn(6, 16, generator=g) for _ in range(world)]
    w = torch.randn(24, 16, generator=g)
    out, full = C.chunk_allgather_gemm(w, shards[rank], world, rank, ps.tp_group, ps.tp_ranks)
    ref_full = torch.cat(shards)
    assert torch.equal(full, ref_full)
    assert torch.allclose(out, ref_full @ w.t(), rtol=1e-5, atol=1e-5)
    xs = [torch.randn(4 * world, 16, generator=g) for _ in range(world)]      # each rank's partial-product input
    total = sum(x @ w.t() for x in xs)
    got = C.chunk_gemm_reduce_scatter(xs[rank], w, world, rank, ps.tp_group, chunks=3)
    assert torch.allclose(got, total[rank * 4:(rank + 1) * 4], rtol=1e-5, atol=1e-5)
    assert C.get_distributed_world_size(ps.tp_group) == world


def test_host_level_chunked_overlap_prototypes_match_plain_composition():
    run_ranks(_chunk_worker, 2)
    run_ranks(_chunk_worker, 4)
