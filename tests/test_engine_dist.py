"""Multi-rank plumbing on CPU (gloo): the folded dual-strand engine under TP+SP, PP, CP, EP
and DP reproduces the losses and gradients of the unsharded sequential autograd model."""
import pytest
import torch

from dist_utils import run_ranks


def _worker(rank, world, name, par, n_mb, B, seq, overrides):
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.models.sharding import random_full_head, random_full_layer, shard_head, shard_layer
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    from reference_model import model_loss

    cfg = preset(name, seq_length=seq, **overrides)
    pcfg = ParallelConfig(**par)
    train = TrainConfig(micro_batch_size=B, global_batch_size=B * n_mb * pcfg.dp, dtype="fp32", clip_grad=0.0)
    tr = Trainer(cfg, pcfg, train, device="cpu")
    ps = tr.ps
    layers = [random_full_layer(cfg, i, 11) for i in range(cfg.num_layers)]
    head = random_full_head(cfg, 11)
    loaded = sum(bool(tr.model.load_full_layer_weights(i, w)) for i, w in enumerate(layers))
    assert loaded == cfg.num_layers // pcfg.pp
    tr.model.load_full_head_weights(head)
    samples = {(d, i): synthetic_tokens(cfg, B, 500 + 17 * d + i) for d in range(pcfg.dp) for i in range(n_mb)}
    mbs = [make_microbatch(cfg, ps, samples[(ps.dp_rank, i)], i, 500 + i, "cpu") for i in range(n_mb)]
    tr.optimizer.zero_grad()
    losses = tr.engine.run_step(mbs)
    tr.optimizer.reduce_gradients()

    for w in layers:
        for t in w.values():
            t.requires_grad_(True)
    for t in head.values():
        t.requires_grad_(True)
    total = 0
    ref = {}
    for key, s in samples.items():
        l = model_loss(cfg, layers, head, s, cfg.moe_aux_loss_coeff if cfg.is_moe else 0.0)
        ref[key] = l.detach()
        total = total + l / len(samples)
    total.backward()

    if ps.pp_rank == 0 and not cfg.is_moe:
        assert len(losses) == n_mb
        for i, l in enumerate(losses):
            assert torch.allclose(l, ref[(ps.dp_rank, i)], rtol=1e-4, atol=1e-5), (i, l, ref[(ps.dp_rank, i)])
    tol = dict(rtol=5e-3, atol=3e-5)
    for m in tr.model.dctb:
        for which, idx in (("first", m.first_index), ("second", m.second_index)):
            gfull = {n: t.grad for n, t in layers[idx].items()}
            gsh = shard_layer(gfull, cfg, ps.tp, ps.tp_rank, ps.ep, ps.ep_rank)
            for n in m.shapes:
                g = getattr(m, f"{n}_{which}").main_grad
                assert torch.allclose(g, gsh[n], **tol), (rank, n, idx, float((g - gsh[n]).abs().max()))
    if tr.model.dchb is not None:
        gsh = shard_head({n: t.grad for n, t in head.items()}, cfg, ps.tp, ps.tp_rank)
        for n in tr.model.dchb.shapes:
            g = getattr(tr.model.dchb, n).main_grad
            assert torch.allclose(g, gsh[n], **tol), (rank, n, float((g - gsh[n]).abs().max()))


CASES = [
    # name, world, parallel config, micro-batches, batch, seq
    ("tiny-llama", 2, dict(tp=2), 4, 2, 128, {}),                      # BASELINE config 1: TP2 + SP, 4 micro-batches
    ("tiny-llama", 2, dict(pp=2), 3, 2, 32, {"num_layers": 4}),
    ("tiny-llama", 2, dict(cp=2), 2, 2, 32, {}),
    ("tiny-llama", 2, dict(dp=2), 2, 1, 32, {}),
    ("tiny-gpt", 2, dict(tp=2), 2, 2, 32, {}),
    ("tiny-moe", 2, dict(dp=2, ep=2), 2, 2, 32, {"moe_aux_loss_coeff": 0.0}),
    ("tiny-llama", 4, dict(tp=2, pp=2), 3, 1, 32, {"num_layers": 4}),
    ("tiny-llama", 4, dict(cp=4), 2, 1, 64, {}),
    ("tiny-gpt", 4, dict(pp=2, cp=2), 3, 1, 32, {"num_layers": 4}),
    ("tiny-moe", 4, dict(dp=4, ep=2), 2, 1, 32, {"moe_aux_loss_coeff": 0.0}),    # two replicas of every expert shard
    ("tiny-moe", 4, dict(dp=2, ep=2, cp=2), 2, 1, 32, {"moe_aux_loss_coeff": 0.0}),   # experts replicated over CP ranks
]


@pytest.mark.parametrize("name,world,par,n_mb,B,seq,ov", CASES, ids=[f"{c[0]}-{'x'.join(f'{k}{v}' for k, v in c[2].items())}" for c in CASES])
def test_parallel_engine_matches_autograd(name, world, par, n_mb, B, seq, ov):
    run_ranks(_worker, world, name, par, n_mb, B, seq, ov)


GATHER_CASES = [("tiny-llama", 2, dict(cp=2), 2, 2, 32, {}), ("tiny-llama", 4, dict(cp=4), 2, 1, 64, {}),
                ("tiny-gpt", 4, dict(tp=2, cp=2), 2, 1, 32, {})]


@pytest.mark.parametrize("name,world,par,n_mb,B,seq,ov", GATHER_CASES, ids=[f"gather-{c[0]}-{'x'.join(f'{k}{v}' for k, v in c[2].items())}" for c in GATHER_CASES])
def test_context_parallel_gather_form_matches_autograd(name, world, par, n_mb, B, seq, ov, monkeypatch):
    """The gather form of context parallelism (what GPUs run over peer memory) on CPU ranks through the
    simulator of the exchange: chunk placement in global order, one bottom-right aligned causal call per
    query chunk, zero rows for unseen keys, owner reduction of dK|dV."""
    monkeypatch.setenv("DHELLAM_CP_GATHER_SIM", "1")
    run_ranks(_worker, world, name, par, n_mb, B, seq, ov)


def _pp_bubble_worker(rank, world):
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama", num_layers=4, seq_length=32)
    pcfg = ParallelConfig(pp=2)
    train = TrainConfig(micro_batch_size=1, global_batch_size=3, dtype="fp32")
    tr = Trainer(cfg, pcfg, train, device="cpu")
    tr.engine.time_pp = True
    mbs = [make_microbatch(cfg, tr.ps, synthetic_tokens(cfg, 1, 9 + i), i, 9 + i, "cpu") for i in range(3)]
    tr.optimizer.zero_grad()
    tr.engine.run_step(mbs)
    ms = tr.engine.pp_bubble_ms()
    assert ms > 0.0                       # every tick but the last exchanges with the neighbour stage
    assert tr.engine.pp_bubble_ms() == 0.0  # reading clears the record


def test_pipeline_exchange_time_is_recorded():
    run_ranks(_pp_bubble_worker, 2)
