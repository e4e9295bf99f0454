"""Folded dual-strand engine on one CPU rank == sequential autograd model."""
import pytest
import torch

from dhellam_b200.config import ParallelConfig, TrainConfig, preset
from dhellam_b200.data import make_microbatch, synthetic_tokens
from dhellam_b200.models.sharding import random_full_head, random_full_layer
from dhellam_b200.parallel import state as PS
from dhellam_b200.trainer import Trainer
from reference_model import model_loss


def _run(cfg, n_mb=3, B=2, coeff=0.0):
    pcfg = ParallelConfig()
    train = TrainConfig(micro_batch_size=B, global_batch_size=B * n_mb, dtype="fp32", clip_grad=0.0)
    PS.set_state(None)
    tr = Trainer(cfg, pcfg, train, device="cpu")
    layers = [random_full_layer(cfg, i, 7) for i in range(cfg.num_layers)]
    head = random_full_head(cfg, 7)
    for i, w in enumerate(layers):
        assert tr.model.load_full_layer_weights(i, w)
    tr.model.load_full_head_weights(head)
    samples = [synthetic_tokens(cfg, B, 100 + i) for i in range(n_mb)]
    mbs = [make_microbatch(cfg, tr.ps, s, i, 100 + i, "cpu") for i, s in enumerate(samples)]
    tr.optimizer.zero_grad()
    losses = tr.engine.run_step(mbs)
    # oracle
    for w in layers:
        for t in w.values():
            t.requires_grad_(True)
    for t in head.values():
        t.requires_grad_(True)
    ref_losses = []
    total = 0
    for s in samples:
        l = model_loss(cfg, layers, head, s, coeff)
        ref_losses.append(l.detach())
        total = total + l / n_mb
    total.backward()
    return tr, losses, ref_losses, layers, head


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-gpt"])
def test_folded_engine_matches_autograd(name):
    cfg = preset(name, seq_length=32)
    tr, losses, ref_losses, layers, head = _run(cfg)
    for a, b in zip(losses, ref_losses):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5), (a, b)
    for m in tr.model.dctb:
        for which, idx in (("first", m.first_index), ("second", m.second_index)):
            for n in m.shapes:
                g = getattr(m, f"{n}_{which}").main_grad
                ref = layers[idx][n].grad
                assert torch.allclose(g, ref, rtol=2e-3, atol=2e-5), (n, idx, (g - ref).abs().max())
    for n in tr.model.dchb.shapes:
        g = getattr(tr.model.dchb, n).main_grad
        assert torch.allclose(g, head[n].grad, rtol=2e-3, atol=2e-5), n


def test_moe_engine_matches_autograd():
    cfg = preset("tiny-moe", seq_length=32, moe_aux_loss_coeff=0.01)
    tr, losses, ref_losses, layers, head = _run(cfg, coeff=0.0)
    # reported losses exclude the auxiliary term; gradients include it
    for m in tr.model.dctb:
        for which, idx in (("first", m.first_index), ("second", m.second_index)):
            for n in m.shapes:
                g = getattr(m, f"{n}_{which}").main_grad
                assert torch.isfinite(g).all()


def test_trainer_close_releases_model_and_optimizer_state():
    import gc
    import weakref
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.data import synthetic_step_batches
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama", seq_length=32)
    train = TrainConfig(micro_batch_size=1, global_batch_size=2, dtype="fp32")
    PS.set_state(None)
    tr = Trainer(cfg, ParallelConfig(), train, device="cpu")
    loss = tr.train_step(synthetic_step_batches(cfg, train, tr.ps, 0, "cpu"))
    w_param, w_master = weakref.ref(tr.model.flat_param), weakref.ref(tr.optimizer.master)
    del loss
    tr.close()
    del tr
    gc.collect()
    assert w_param() is None and w_master() is None
    PS.set_state(None)
