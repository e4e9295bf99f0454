"""Unsharded ("full") layer weights and their tensor/expert-parallel shards.

Full layouts used by this framework:

* ``column_attn_weight [(nq + 2 nkv) d, h]`` = all query heads, then all key heads, then all
  value heads; a rank takes its query heads, its key heads and its value heads;
* ``linear_attn_weight [h, nq d]`` is split by columns (query heads);
* ``column_mlp_weight [2f, h]`` = gate rows then up rows; a rank takes its slice of each;
* ``linear_mlp_weight [h, f]`` is split by columns;
* expert weights ``[E, ...]`` are split over experts (EP) and, inside an expert, like the
  dense MLP (TP);
* ``word_embeddings [V, h]`` is split by rows.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config import ModelConfig


def full_layer_shapes(cfg: ModelConfig):
    h, d, f = cfg.hidden_size, cfg.head_dim, cfg.ffn_hidden_size
    nq, nkv = cfg.num_attention_heads, cfg.num_query_groups
    g = 2 if cfg.gated else 1
    s = {"ln_attn_weight": (h,), "column_attn_weight": ((nq + 2 * nkv) * d, h), "linear_attn_weight": (h, nq * d),
         "ln_mlp_weight": (h,)}
    if cfg.norm == "layernorm":
        s["ln_attn_bias"] = (h,)
        s["ln_mlp_bias"] = (h,)
    if cfg.is_moe:
        s["router_weight"] = (cfg.num_experts, h)
        s["expert_column_weight"] = (cfg.num_experts, g * f, h)
        s["expert_linear_weight"] = (cfg.num_experts, h, f)
    else:
        s["column_mlp_weight"] = (g * f, h)
        s["linear_mlp_weight"] = (h, f)
    return s


def random_full_layer(cfg: ModelConfig, layer_index: int, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed * 7919 + layer_index)
    out = {}
    for n, shape in full_layer_shapes(cfg).items():
        if n.startswith("ln_"):
            base = torch.zeros(shape) if n.endswith("bias") else torch.ones(shape)
            out[n] = (base + 0.1 * torch.randn(shape, generator=gen)).to(dtype)
        else:
            out[n] = (torch.randn(shape, generator=gen) * cfg.init_std).to(dtype)
    return out


def random_full_head(cfg: ModelConfig, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed * 7919 + 100003)
    out = {"word_embeddings": (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=gen) * cfg.init_std).to(dtype),
           "final_ln_weight": (torch.ones(cfg.hidden_size) + 0.1 * torch.randn(cfg.hidden_size, generator=gen)).to(dtype)}
    if cfg.norm == "layernorm":
        out["final_ln_bias"] = (0.1 * torch.randn(cfg.hidden_size, generator=gen)).to(dtype)
    if not cfg.tie_embeddings:
        out["output_weight"] = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=gen) * cfg.init_std).to(dtype)
    if cfg.position == "learned":
        out["position_embeddings"] = (torch.randn(cfg.seq_length, cfg.hidden_size, generator=gen) * cfg.init_std).to(dtype)
    return out


def _rows(t, n, r):
    k = t.shape[0] // n
    return t[r * k:(r + 1) * k]


def _cols(t, n, r):
    k = t.shape[-1] // n
    return t[..., r * k:(r + 1) * k]


def shard_qkv(w, cfg: ModelConfig, tp: int, r: int):
    d = cfg.head_dim
    nq, nkv = cfg.num_attention_heads, cfg.num_query_groups
    q, k, v = w[:nq * d], w[nq * d:(nq + nkv) * d], w[(nq + nkv) * d:]
    return torch.cat([_rows(q, tp, r), _rows(k, tp, r), _rows(v, tp, r)], dim=0)


def unshard_qkv(shards, cfg: ModelConfig):
    d = cfg.head_dim
    tp = len(shards)
    nq, nkv = cfg.num_attention_heads // tp, cfg.num_query_groups // tp
    q = torch.cat([s[:nq * d] for s in shards], 0)
    k = torch.cat([s[nq * d:(nq + nkv) * d] for s in shards], 0)
    v = torch.cat([s[(nq + nkv) * d:] for s in shards], 0)
    return torch.cat([q, k, v], 0)


def _shard_fc1(w, cfg, tp, r):
    if cfg.gated:
        f = w.shape[-2] // 2
        gate, up = w[..., :f, :], w[..., f:, :]
        k = f // tp
        return torch.cat([gate[..., r * k:(r + 1) * k, :], up[..., r * k:(r + 1) * k, :]], dim=-2)
    k = w.shape[-2] // tp
    return w[..., r * k:(r + 1) * k, :]


def unshard_fc1(shards, cfg):
    if cfg.gated:
        f = shards[0].shape[-2] // 2
        return torch.cat([s[..., :f, :] for s in shards] + [s[..., f:, :] for s in shards], dim=-2)
    return torch.cat(shards, dim=-2)


def shard_layer(full: Dict[str, torch.Tensor], cfg: ModelConfig, tp: int, r: int, ep: int = 1, er: int = 0):
    out = {}
    for n, w in full.items():
        if n == "column_attn_weight":
            out[n] = shard_qkv(w, cfg, tp, r)
        elif n == "linear_attn_weight" or n == "linear_mlp_weight":
            out[n] = _cols(w, tp, r)
        elif n == "column_mlp_weight":
            out[n] = _shard_fc1(w, cfg, tp, r)
        elif n == "expert_column_weight":
            out[n] = _shard_fc1(_rows(w, ep, er), cfg, tp, r)
        elif n == "expert_linear_weight":
            out[n] = _cols(_rows(w, ep, er), tp, r)
        else:
            out[n] = w
    return {k: v.contiguous() for k, v in out.items()}


def shard_head(full: Dict[str, torch.Tensor], cfg: ModelConfig, tp: int, r: int):
    out = {}
    for n, w in full.items():
        out[n] = _rows(w, tp, r).contiguous() if n in ("word_embeddings", "output_weight") else w
    return out
