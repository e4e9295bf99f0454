"""Failure detection with host-made failures on CPU ranks (no GPU is faulted anywhere):
a rank that stops between steps, a rank that hangs on the host, a stale restart epoch."""
import time

import pytest
import torch

from dist_utils import run_ranks


def _dead_rank(rank, world):
    import torch.distributed as dist
    from dhellam_b200.runtime.watchdog import Heartbeat, RankFailure, StepGate
    hb = Heartbeat(interval=0.05, timeout=0.6)
    gate = StepGate(timeout=3.0, heartbeat=hb)
    gate.agree(0)
    t = torch.ones(4) * rank
    dist.all_reduce(t)                       # step 0 completes on every rank
    if rank == world - 1:
        hb.pause()                           # this rank "dies" between steps: no beat, no further announcement
        time.sleep(2.0)
        hb.resume()
        gate.announce(10**6)                 # let the survivors' final barrier in the harness pass
        hb.stop()
        return
    t0 = time.time()
    with pytest.raises(RankFailure) as ei:
        gate.agree(1)                        # checked on the host BEFORE launching step 1
    assert ei.value.ranks == [world - 1]
    assert time.time() - t0 < 2.5
    time.sleep(1.5)
    hb.stop()


def test_rank_that_stops_between_steps_is_detected_before_the_next_launch():
    run_ranks(_dead_rank, 3)


def _late_rank(rank, world):
    from dhellam_b200.runtime.watchdog import Heartbeat, RankFailure, StepGate
    hb = Heartbeat(interval=0.05, timeout=5.0)
    gate = StepGate(timeout=0.5, heartbeat=hb)
    if rank == 1:
        time.sleep(1.2)                      # alive (heartbeat runs) but far too late
        gate.announce(0)
        hb.stop()
        return
    with pytest.raises(RankFailure) as ei:
        gate.agree(0)
    assert ei.value.ranks == [1] and "within" in str(ei.value)
    time.sleep(1.0)
    hb.stop()


def test_delayed_rank_times_out_with_a_typed_error():
    run_ranks(_late_rank, 2)


def _stale_epoch(rank, world):
    from dhellam_b200.runtime.watchdog import RankFailure, StepGate
    gate = StepGate(timeout=2.0)
    if rank == 1:
        gate.announce(5, epoch=0)            # a rank that did not take part in the restart
        time.sleep(0.8)
        return
    time.sleep(0.2)
    with pytest.raises(RankFailure) as ei:
        gate.agree(5, epoch=1)
    assert "epoch" in str(ei.value)


def test_stale_restart_epoch_is_rejected():
    run_ranks(_stale_epoch, 2)


def _exception_rank(rank, world, path):
    """A rank raises in its step function: the others see it through the gate, save nothing
    new, and a fresh run resumes from the last checkpoint with the same losses."""
    from dhellam_b200.ckpt import load_checkpoint, save_checkpoint
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.data import synthetic_step_batches
    from dhellam_b200.runtime.watchdog import Heartbeat, RankFailure, StepGate
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama", seq_length=32)
    train = TrainConfig(micro_batch_size=1, global_batch_size=2, dtype="fp32", lr=1e-3)
    tr = Trainer(cfg, ParallelConfig(dp=2), train, device="cpu")
    hb = Heartbeat(interval=0.05, timeout=0.6)
    gate = StepGate(timeout=3.0, heartbeat=hb)
    losses = []
    failed = False
    for step in range(4):
        try:
            if rank == 1 and step == 2:
                raise RuntimeError("injected host failure")
            gate.agree(step)
        except RuntimeError as e:
            if isinstance(e, RankFailure) or "injected" in str(e):
                failed = True
                if rank == 1:
                    hb.pause()
                break
            raise
        losses.append(float(tr.train_step(synthetic_step_batches(cfg, train, tr.ps, step, "cpu"))))
        if step == 0:
            save_checkpoint(path, 1, tr.model, tr.optimizer)
    assert failed and len(losses) == 2
    if rank == 0:
        torch.save(losses, path + "/losses.pt")
    time.sleep(1.5)
    hb.resume()
    hb.stop()


def _resume_rank(rank, world, path):
    from dhellam_b200.ckpt import load_checkpoint
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.data import synthetic_step_batches
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama", seq_length=32)
    train = TrainConfig(micro_batch_size=1, global_batch_size=2, dtype="fp32", lr=1e-3)
    tr = Trainer(cfg, ParallelConfig(dp=2), train, device="cpu")
    it = load_checkpoint(path, tr.model, tr.optimizer)
    loss = float(tr.train_step(synthetic_step_batches(cfg, train, tr.ps, it, "cpu")))
    if rank == 0:
        before = torch.load(path + "/losses.pt")
        assert loss == before[1], (loss, before)


def test_injected_exception_aborts_the_step_and_resume_matches(tmp_path):
    run_ranks(_exception_rank, 2, str(tmp_path))
    run_ranks(_resume_rank, 2, str(tmp_path))


def _never_joins(rank, world):
    from dhellam_b200.runtime.watchdog import Heartbeat, RankFailure
    if rank == 1:
        time.sleep(1.0)                      # never creates its heartbeat
        return
    with pytest.raises(RankFailure) as ei:
        Heartbeat(interval=0.05, timeout=0.5, startup_timeout=0.4)
    assert ei.value.ranks == [1] and "never joined" in str(ei.value)
    time.sleep(0.8)


def test_rank_that_never_joins_is_reported():
    run_ranks(_never_joins, 2)


def test_train_loop_stops_before_the_next_launch_and_saves_nothing_after_a_host_failure(tmp_path):
    """``train.py`` on two CPU ranks: rank 1 stops beating and hangs on the host at step 1 (a
    host-made failure, no GPU involved).  Rank 0 must raise ``RankFailure`` from the step gate
    before launching step 1, and no checkpoint newer than step 1's predecessor may exist."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, DHELLAM_INJECT_HOST_FAILURE="1:1:6")
    save = tmp_path / "ck"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(root, "train.py"),
           "--num-layers", "2", "--hidden-size", "64", "--ffn-hidden-size", "128", "--num-attention-heads", "4",
           "--group-query-attention", "--num-query-groups", "2", "--seq-length", "32", "--vocab-size", "128", "--swiglu",
           "--micro-batch-size", "1", "--global-batch-size", "2", "--lr", "1e-3", "--dhellam",
           "--tensor-model-parallel-size", "2", "--sequence-parallel", "--train-iters", "3",
           "--save", str(save), "--save-interval", "1",
           "--step-gate-timeout", "3", "--heartbeat-interval", "0.1", "--heartbeat-timeout", "1.0"]
    p = subprocess.run(cmd, cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode != 0
    assert "RankFailure" in p.stderr and "[1]" in p.stderr, p.stderr[-3000:]
    assert (save / "iter_0000001").exists()
    assert not (save / "iter_0000002").exists() and not (save / "iter_0000003").exists()
    assert (save / "latest_checkpointed_iteration.txt").read_text() == "1"
