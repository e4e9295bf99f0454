"""The distributed optimizer (each data-parallel rank owns 1/dp of the master weights and Adam
state: gradients are reduce-scattered, the owned slice is updated, parameters are gathered
again) must produce the parameters of the replicated optimizer."""
import torch

from dist_utils import run_ranks


def _worker(rank, world, out_dir):
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama", seq_length=32)
    pcfg = ParallelConfig(dp=world)
    train = TrainConfig(micro_batch_size=1, global_batch_size=2 * world, dtype="fp32", lr=1e-3)
    ps = PS.initialize_model_parallel(pcfg)
    results = []
    for distributed in (False, True):
        torch.manual_seed(11)
        tr = Trainer(cfg, pcfg, train, device="cpu", ps=ps, distributed_optimizer=distributed)
        if results:
            tr.model.flat_param.data.copy_(start)
            tr.optimizer.master.copy_(start[tr.optimizer.lo:tr.optimizer.hi])
        else:
            start = tr.model.flat_param.detach().clone()
        assert tr.optimizer.distributed == distributed
        if distributed:
            assert tr.optimizer.master.numel() < tr.model.flat_param.numel()      # a shard, not a replica
        for step in range(2):
            mbs = [make_microbatch(cfg, ps, synthetic_tokens(cfg, 1, 100 * step + 10 * ps.dp_rank + i), i, 7 + i, "cpu") for i in range(2)]
            tr.train_step(mbs)
        results.append(tr.model.flat_param.detach().clone())
        sd = tr.optimizer.state_dict()
        tr.optimizer.load_state_dict(sd)                                           # round trip of the shard layout
    assert torch.allclose(results[0], results[1], rtol=1e-5, atol=1e-6), float((results[0] - results[1]).abs().max())
    assert not torch.equal(results[0], start)


def test_distributed_optimizer_matches_replicated(tmp_path):
    run_ranks(_worker, 2, str(tmp_path))
