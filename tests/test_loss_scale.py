"""Loss scaling: a constant factor must not change the update, and the dynamic scaler skips
overflowing steps, backs off after ``hysteresis`` overflows and grows after its window."""
import math

import torch

from dhellam_b200.config import ParallelConfig, TrainConfig, preset
from dhellam_b200.data import make_microbatch, synthetic_tokens
from dhellam_b200.optim.adam import DynamicLossScaler
from dhellam_b200.parallel import state as PS
from dhellam_b200.trainer import Trainer


def _trainer(**kw):
    cfg = preset("tiny-llama")
    train = TrainConfig(micro_batch_size=1, global_batch_size=2, dtype="fp32", **kw)
    tr = Trainer(cfg, ParallelConfig(), train, device=torch.device("cpu"), ps=PS.initialize_model_parallel(ParallelConfig()))
    mbs = [make_microbatch(cfg, tr.ps, synthetic_tokens(cfg, 1, 3 + i), i, 3 + i, tr.device) for i in range(2)]
    return tr, mbs


def test_constant_loss_scale_leaves_the_update_unchanged():
    a, mbs = _trainer()
    b, _ = _trainer(loss_scale=1024.0)
    b.model.flat_param.data.copy_(a.model.flat_param.data)
    b.optimizer.master.copy_(a.optimizer.master)
    la, lb = a.train_step(mbs), b.train_step(mbs)
    assert torch.allclose(la, lb)
    # gradients carry the factor, the reported norm and the parameters do not
    assert torch.allclose(b.model.flat_grad, a.model.flat_grad * 1024.0, rtol=1e-4, atol=1e-6)
    assert math.isclose(float(a.last_grad_norm), float(b.last_grad_norm), rel_tol=1e-4)
    assert torch.allclose(a.model.flat_param, b.model.flat_param, rtol=1e-5, atol=1e-7)


def test_dynamic_scaler_schedule():
    s = DynamicLossScaler(initial=1024.0, min_scale=256.0, window=3, hysteresis=2)
    s.update(True)
    assert s.scale == 1024.0                 # first overflow is tolerated
    s.update(True)
    assert s.scale == 512.0
    s.update(True)
    s.update(True)
    assert s.scale == 256.0                  # floor
    for _ in range(3):
        s.update(False)
    assert s.scale == 512.0                  # a full window of good steps doubles it
    again = DynamicLossScaler()
    again.load_state_dict(s.state_dict())
    assert again.scale == s.scale


def test_overflowing_step_is_skipped_and_scale_backs_off():
    tr, mbs = _trainer(dynamic_loss_scale=True, initial_loss_scale=4096.0, hysteresis=1, loss_scale_window=2)
    before = tr.model.flat_param.clone()
    # first step: poison a gradient after the backward pass
    tr.optimizer.zero_grad()
    tr.engine.loss_scale = tr.optimizer.loss_scale
    tr.engine.run_step(mbs)
    tr.model.flat_grad[5] = float("inf")
    tr.optimizer.step()
    assert tr.optimizer.skipped_steps == 1 and tr.optimizer.step_count == 0
    assert torch.equal(tr.model.flat_param, before)
    assert tr.optimizer.loss_scale == 2048.0
    # two clean steps: parameters move, the scale grows back
    tr.train_step(mbs)
    assert not torch.equal(tr.model.flat_param, before) and tr.optimizer.step_count == 1
    tr.train_step(mbs)
    assert tr.optimizer.loss_scale == 4096.0
    sd = tr.optimizer.state_dict()
    assert sd["scaler"]["scale"] == 4096.0
