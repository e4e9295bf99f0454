"""Checkpoint layout, fold map, re-sharding on load, and resume."""
import json
import os

import torch

from dist_utils import run_ranks


def test_fold_map_is_a_bijection():
    from dhellam_b200.ckpt import fold_map
    for L, P in ((8, 1), (8, 2), (12, 3), (40, 2)):
        m = fold_map(L, P)
        assert sorted(m.values()) == list(range(L))
        assert m[(0, 0, "first")] == 0 and m[(0, 0, "second")] == L - 1
        # the two halves of a stage are mirror images
        for (p, j, w), l in m.items():
            if w == "first":
                assert m[(p, j, "second")] == L - 1 - l


def test_qkv_interleave_round_trip():
    from dhellam_b200.ckpt.megatron import qkv_megatron_to_shard, qkv_shard_to_megatron
    from dhellam_b200.config import preset
    cfg = preset("tiny-llama")
    w = torch.randn((cfg.num_attention_heads + 2 * cfg.num_query_groups) * cfg.head_dim, cfg.hidden_size)
    assert torch.equal(qkv_megatron_to_shard(qkv_shard_to_megatron(w, cfg, 1), cfg, 1), w)
    m = qkv_shard_to_megatron(w, cfg, 1)
    d, g = cfg.head_dim, cfg.num_attention_heads // cfg.num_query_groups
    # first group: its query heads, then its key head, then its value head
    assert torch.equal(m[: g * d], w[: g * d])
    assert torch.equal(m[g * d:(g + 1) * d], w[cfg.num_attention_heads * d: cfg.num_attention_heads * d + d])


def _save_worker(rank, world, path, par):
    from dhellam_b200.ckpt import save_checkpoint
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.models.sharding import random_full_head, random_full_layer
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama", num_layers=4, seq_length=32)
    tr = Trainer(cfg, ParallelConfig(**par), TrainConfig(micro_batch_size=1, global_batch_size=2 * par.get("dp", 1), dtype="fp32"), device="cpu")
    for i in range(cfg.num_layers):
        tr.model.load_full_layer_weights(i, random_full_layer(cfg, i, 21))
    tr.model.load_full_head_weights(random_full_head(cfg, 21))
    save_checkpoint(path, 7, tr.model, tr.optimizer, {"note": "test"})


def test_save_tp2_pp2_load_single_rank_reshards(tmp_path):
    from dhellam_b200.ckpt import load_checkpoint, read_latest_iteration
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.models.sharding import random_full_head, random_full_layer
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    path = str(tmp_path / "ck")
    run_ranks(_save_worker, 4, path, dict(tp=2, pp=2))
    assert read_latest_iteration(path) == 7
    d = os.path.join(path, "iter_0000007")
    for f in ("metadata.json", "common.pt", ".metadata", "__0_0.distcp", "__3_0.distcp"):
        assert os.path.exists(os.path.join(d, f)), f
    meta = json.load(open(os.path.join(d, "metadata.json")))
    assert meta["sharded_backend"] == "torch_dist"
    # the weight files are real torch.distributed.checkpoint files: any DCP reader opens them
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader
    idx = FileSystemReader(d).read_metadata().state_dict_metadata
    for key in ("embedding.word_embeddings.weight", "decoder.final_layernorm.weight",
                "decoder.layers.0.self_attention.linear_qkv.weight", "decoder.layers.3.mlp.linear_fc2.weight",
                "decoder.layers.2.self_attention.linear_qkv.layer_norm_weight"):
        assert key in idx, key
    cfg = preset("tiny-llama", num_layers=4, seq_length=32)
    assert list(idx["decoder.layers.1.mlp.linear_fc1.weight"].size) == [2 * cfg.ffn_hidden_size, cfg.hidden_size]
    assert len(idx["decoder.layers.1.mlp.linear_fc1.weight"].chunks) == 4          # gate and up halves of two TP ranks
    sd = {"decoder.layers.3.mlp.linear_fc2.weight": torch.empty(cfg.hidden_size, cfg.ffn_hidden_size),
          "decoder.final_layernorm.weight": torch.empty(cfg.hidden_size)}
    dcp.load(sd, checkpoint_id=d, no_dist=True)
    assert torch.equal(sd["decoder.layers.3.mlp.linear_fc2.weight"], random_full_layer(cfg, 3, 21)["linear_mlp_weight"])
    assert torch.equal(sd["decoder.final_layernorm.weight"], random_full_head(cfg, 21)["final_ln_weight"])
    PS.set_state(None)
    tr = Trainer(cfg, ParallelConfig(), TrainConfig(micro_batch_size=1, global_batch_size=2, dtype="fp32"), device="cpu")
    it = load_checkpoint(path, tr.model, tr.optimizer)
    assert it == 7
    for m in tr.model.dctb:
        for which, li in (("first", m.first_index), ("second", m.second_index)):
            full = random_full_layer(cfg, li, 21)
            for n in m.shapes:
                assert torch.equal(getattr(m, f"{n}_{which}").data, full[n]), (li, n)
    head = random_full_head(cfg, 21)
    assert torch.equal(tr.model.dchb.word_embeddings.data, head["word_embeddings"])
    PS.set_state(None)


def test_resume_reproduces_the_loss_curve(tmp_path):
    from dhellam_b200.ckpt import load_checkpoint, save_checkpoint
    from dhellam_b200.config import ParallelConfig, TrainConfig, preset
    from dhellam_b200.data import synthetic_step_batches
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama", seq_length=32)
    train = TrainConfig(micro_batch_size=1, global_batch_size=2, dtype="fp32", lr=1e-3)
    PS.set_state(None)
    a = Trainer(cfg, ParallelConfig(), train, device="cpu")
    losses = []
    for step in range(4):
        if step == 2:
            save_checkpoint(str(tmp_path), 2, a.model, a.optimizer)
        losses.append(float(a.train_step(synthetic_step_batches(cfg, train, a.ps, step, "cpu"))))
    PS.set_state(None)
    b = Trainer(cfg, ParallelConfig(), train, device="cpu")
    it = load_checkpoint(str(tmp_path), b.model, b.optimizer)
    resumed = [float(b.train_step(synthetic_step_batches(cfg, train, b.ps, step, "cpu"))) for step in range(it, 4)]
    assert resumed == losses[2:], (resumed, losses)
    PS.set_state(None)
