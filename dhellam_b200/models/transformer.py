"""Transformer layer as two strands of ops (Llama, GPT and Mixtral families).

The op names, their order and their dependencies follow the reference's static graphs
(dhellam/core/dstb.py:698-843) and its per-op functions ``DCFunc`` (dstb.py:64-425), so
that strategy files written for the reference drive this engine.  What differs:

* activations are sequence-first ``[S*B, h]`` rows, so the sequence all-gather /
  reduce-scatter keeps token order for any micro-batch size;
* RMSNorm / RoPE / grouped-query attention / SwiGLU for Llama, LayerNorm / GeLU for GPT,
  a routed expert MLP for Mixtral (new ops with ids >= 35);
* ring steps for any context-parallel size, not only 2;
* with ``env.fused_comm`` the collective is performed inside the GEMM kernel: the
  ``allgather_*`` / ``reduce_scatter_*`` ops stay in the graph under their names (so the
  same strategy files are legal) but only hand their operand to the fused GEMM op.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..config import ModelConfig
from ..ops import activation as A
from ..ops import attention as ATT
from ..ops import bda as BDA
from ..ops import comm as C
from ..ops import gemm as G
from ..ops import norm as N
from ..ops import rope as R
from ..sched.ir import BWD, COMM, COMPUTE, FWD, MEM, MMA, NVL, LayerProgram, LayerRun, Op
from ..sched.optable import OP_TABLE_IDX


# --------------------------------------------------------------------------- parameters
PARAM_NAMES = ["ln_attn_weight", "ln_attn_bias", "column_attn_weight", "linear_attn_weight",
               "ln_mlp_weight", "ln_mlp_bias", "column_mlp_weight", "linear_mlp_weight"]
MOE_PARAM_NAMES = ["router_weight", "expert_column_weight", "expert_linear_weight"]


def layer_param_shapes(cfg: ModelConfig, tp: int, ep: int = 1):
    """Per-rank parameter shapes of one layer.  Names follow the reference's ``DSTB``
    parameters (dhellam/core/dstb.py:1373-1389)."""
    h, d = cfg.hidden_size, cfg.head_dim
    nq, nkv = cfg.num_attention_heads // tp, max(cfg.num_query_groups // tp, 1)
    f = cfg.ffn_hidden_size // tp
    shapes = {
        "ln_attn_weight": (h,),
        "column_attn_weight": ((nq + 2 * nkv) * d, h),
        "linear_attn_weight": (h, nq * d),
        "ln_mlp_weight": (h,),
    }
    if cfg.norm == "layernorm":
        shapes["ln_attn_bias"] = (h,)
        shapes["ln_mlp_bias"] = (h,)
    if cfg.is_moe:
        el = cfg.num_experts // ep
        shapes["router_weight"] = (cfg.num_experts, h)
        shapes["expert_column_weight"] = (el, (2 if cfg.gated else 1) * f, h)
        shapes["expert_linear_weight"] = (el, h, f)
    else:
        shapes["column_mlp_weight"] = ((2 if cfg.gated else 1) * f, h)
        shapes["linear_mlp_weight"] = (h, f)
    return shapes


class LayerParams:
    """Tensors of one layer.  Every tensor ``p`` has ``p.main_grad`` (fp32) attached by the
    owner; norm weights carry ``sequence_parallel = True`` (dstb.py:1414-1421)."""

    def __init__(self, tensors: dict):
        self.__dict__.update(tensors)
        self._names = list(tensors.keys())

    def named(self):
        return [(n, getattr(self, n)) for n in self._names]

    def get(self, name, default=None):
        return self.__dict__.get(name, default)


# --------------------------------------------------------------------------- helpers
def _use(run: LayerRun, t):
    """Marks ``t`` as used on the stream that executes the current op, so the caching
    allocator does not recycle it while that stream still reads it."""
    s = getattr(run.env, "cur_stream", None)
    if s is not None and t is not None and t.is_cuda:
        t.record_stream(s)
    return t


def _heads(env):
    cfg, tp = env.cfg, env.ps.tp
    return cfg.num_attention_heads // tp, max(cfg.num_query_groups // tp, 1), cfg.head_dim


def _norm_fwd(env, x, w, b, budget):
    if env.cfg.norm == "rmsnorm":
        y, rstd = N.rmsnorm_fwd(x, w, env.cfg.norm_eps, sm_budget=budget)
        return y, (rstd,)
    y, mu, rstd = N.layernorm_fwd(x, w, b, env.cfg.norm_eps, sm_budget=budget)
    return y, (mu, rstd)


def _norm_bwd(env, dy, x, w, b, stat, residual_grad, budget):
    if env.cfg.norm == "rmsnorm":
        dx, _ = N.rmsnorm_bwd(dy, x, w, stat[0], weight_main_grad=w.main_grad, residual_grad=residual_grad, sm_budget=budget)
        return dx
    dx, _, _ = N.layernorm_bwd(dy, x, w, stat[0], stat[1], weight_main_grad=w.main_grad, bias_main_grad=b.main_grad,
                               residual_grad=residual_grad, sm_budget=budget)
    return dx


def _seed(run: LayerRun, site: int) -> int:
    return (run.mb.seed * 1000003 + run.layer_index * 16 + site) & 0x7FFFFFFFFFFFFFFF


# --------------------------------------------------------------------------- forward ops
def f_ln_attn(run):
    x = _use(run, run.v["x"])
    p = run.params
    y, stat = _norm_fwd(run.env, x, p.ln_attn_weight, p.get("ln_attn_bias"), run.budget("ln_attn"))
    run.acts["x0"], run.acts["ln1_stat"] = x, stat
    run.v["ln1"] = y


def _split_site(env, w, transpose_w=False):
    """True when the collective beside the GEMM with weight ``w`` runs as its own kernel on the
    communication stream (decided per site by ``FusedTP.split``), False when it is fused into
    the GEMM kernel."""
    n, k = (w.shape[1], w.shape[0]) if transpose_w else (w.shape[0], w.shape[1])
    return env.fused.split(env.fused.rows, n, k)


def f_allgather_attn(run):
    env = run.env
    if env.fused_tp:
        if _split_site(env, run.params.column_attn_weight):
            env.fused.gather_start(_use(run, run.v["ln1"]), "attn_c")
        run.v["ln1_shard"] = run.v.pop("ln1")
    else:
        run.v["ln1_full"], _ = C.gather_along_first_dim(_use(run, run.v.pop("ln1")), env.ps.tp_group)


def f_gemm_attn_c(run):
    env, p = run.env, run.params
    if env.fused_tp:
        # the gathered operand is not kept: the backward re-gathers the (8x smaller) shard
        shard = _use(run, run.v.pop("ln1_shard"))
        if _split_site(env, p.column_attn_weight):
            full, sync = env.fused.gather_consume("attn_c")
            qkv = G.gemm_nt(full, p.column_attn_weight, sm_budget=run.budget("gemm_attn_c"), sync=sync)
        else:
            qkv, _ = env.fused.ag_gemm(shard, p.column_attn_weight, "attn_c", sm_budget=run.budget("gemm_attn_c"))
        run.acts["ln1_shard"] = shard
    else:
        full = _use(run, run.v.pop("ln1_full"))
        qkv = G.gemm_nt(full, p.column_attn_weight, sm_budget=run.budget("gemm_attn_c"))
        run.acts["ln1_full"] = full
    run.v["qkv"] = qkv


def _qkv_views(env, qkv, B):
    nq, nkv, d = _heads(env)
    T = qkv.shape[0]
    S = T // B
    v4 = qkv.view(S, B, nq + 2 * nkv, d)
    return v4[:, :, :nq], v4[:, :, nq:nq + nkv], v4[:, :, nq + nkv:]


def _apply_rope(run, qkv, inverse=False):
    env = run.env
    if env.cfg.position != "rope":
        return
    nq, nkv, d = _heads(env)
    R.rope_apply_(qkv, run.mb.positions, env.rope_cos, env.rope_sin, nq, nkv, d, inverse=inverse)


def f_fl_attn(run):
    env = run.env
    qkv = _use(run, run.v.pop("qkv"))
    _apply_rope(run, qkv)
    q, k, v = _qkv_views(env, qkv, run.mb.batch)
    o, lse = ATT.attn_fwd(q, k, v, causal=True, scale=env.softmax_scale, sm_budget=run.budget("fl_attn"))
    run.acts["qkv"], run.acts["attn_out"], run.acts["lse"] = qkv, o, lse
    run.v["attn_out"] = o.view(qkv.shape[0], -1)


def f_gemm_attn_l(run):
    env, p = run.env, run.params
    a = _use(run, run.v.pop("attn_out"))
    if env.fused_tp and _split_site(env, p.linear_attn_weight):
        part, sync = env.fused.partial_produce("attn_l", a.shape[0], p.linear_attn_weight.shape[0])
        G.gemm_nt(a, p.linear_attn_weight, out=part, sm_budget=run.budget("gemm_attn_l"), sync=sync)
    elif env.fused_tp:
        run.v["proj"] = env.fused.gemm_rs(a, p.linear_attn_weight, "attn_l", sm_budget=run.budget("gemm_attn_l"))
    else:
        run.v["proj_partial"] = G.gemm_nt(a, p.linear_attn_weight, sm_budget=run.budget("gemm_attn_l"))


def f_reduce_scatter_attn(run):
    env = run.env
    if not env.fused_tp:
        run.v["proj"], _ = C.reduce_scatter_along_first_dim(_use(run, run.v.pop("proj_partial")), env.ps.tp_group)
    elif "proj" not in run.v:
        run.v["proj"] = env.fused.rs_reduce("attn_l")


def f_bda_attn(run):
    env = run.env
    h1 = BDA.bda_fwd(_use(run, run.v.pop("proj")), run.acts["x0"], None, env.cfg.hidden_dropout, _seed(run, 1), env.training,
                     sm_budget=run.budget("bda_attn"))
    run.v["h1"] = h1


def f_ln_mlp(run):
    p = run.params
    h1 = _use(run, run.v.pop("h1"))
    y, stat = _norm_fwd(run.env, h1, p.ln_mlp_weight, p.get("ln_mlp_bias"), run.budget("ln_mlp"))
    run.acts["h1"], run.acts["ln2_stat"] = h1, stat
    run.v["ln2"] = y


def f_allgather_mlp(run):
    env = run.env
    if env.fused_tp:
        if _split_site(env, run.params.column_mlp_weight):
            env.fused.gather_start(_use(run, run.v["ln2"]), "mlp_c")
        run.v["ln2_shard"] = run.v.pop("ln2")
    else:
        run.v["ln2_full"], _ = C.gather_along_first_dim(_use(run, run.v.pop("ln2")), env.ps.tp_group)


def f_gemm_mlp_c(run):
    env, p = run.env, run.params
    if env.fused_tp:
        shard = _use(run, run.v.pop("ln2_shard"))
        if _split_site(env, p.column_mlp_weight):
            full, sync = env.fused.gather_consume("mlp_c")
            fc1 = G.gemm_nt(full, p.column_mlp_weight, sm_budget=run.budget("gemm_mlp_c"), sync=sync)
        else:
            fc1, _ = env.fused.ag_gemm(shard, p.column_mlp_weight, "mlp_c", sm_budget=run.budget("gemm_mlp_c"))
        run.acts["ln2_shard"] = shard
    else:
        full = _use(run, run.v.pop("ln2_full"))
        fc1 = G.gemm_nt(full, p.column_mlp_weight, sm_budget=run.budget("gemm_mlp_c"))
        run.acts["ln2_full"] = full
    run.acts["fc1"] = fc1
    run.v["fc1"] = fc1


def f_act_mlp(run):
    fc1 = _use(run, run.v.pop("fc1"))
    if run.env.cfg.gated:
        act = A.swiglu_fwd(fc1, sm_budget=run.budget("swiglu_mlp"))
    else:
        act = A.gelu_fwd(fc1, sm_budget=run.budget("gelu_mlp"))
    run.acts["act"] = act
    run.v["act"] = act


def f_gemm_mlp_l(run):
    env, p = run.env, run.params
    a = _use(run, run.v.pop("act"))
    if env.fused_tp and _split_site(env, p.linear_mlp_weight):
        part, sync = env.fused.partial_produce("mlp_l", a.shape[0], p.linear_mlp_weight.shape[0])
        G.gemm_nt(a, p.linear_mlp_weight, out=part, sm_budget=run.budget("gemm_mlp_l"), sync=sync)
    elif env.fused_tp:
        run.v["fc2"] = env.fused.gemm_rs(a, p.linear_mlp_weight, "mlp_l", sm_budget=run.budget("gemm_mlp_l"))
    else:
        run.v["fc2_partial"] = G.gemm_nt(a, p.linear_mlp_weight, sm_budget=run.budget("gemm_mlp_l"))


def f_reduce_scatter_mlp(run):
    env = run.env
    if not env.fused_tp:
        run.v["fc2"], _ = C.reduce_scatter_along_first_dim(_use(run, run.v.pop("fc2_partial")), env.ps.tp_group)
    elif "fc2" not in run.v:
        run.v["fc2"] = env.fused.rs_reduce("mlp_l")


def f_bda_mlp(run):
    env = run.env
    out = BDA.bda_fwd(_use(run, run.v.pop("fc2")), run.acts["h1"], None, env.cfg.hidden_dropout, _seed(run, 2), env.training,
                      sm_budget=run.budget("bda_mlp"))
    run.v["out"] = out


# --------------------------------------------------------------------------- backward ops
def b_bda_mlp_bwd(run):
    env = run.env
    dout = _use(run, run.v["dout"])
    if env.fused_tp and "ln2_shard" in run.acts:
        # re-gather the inputs of the two column-parallel layers for their weight gradients;
        # the pushes run on the communication stream under the first backward GEMMs
        comm = env.streams.s3 if getattr(env, "streams", None) is not None and env.streams.cuda else None
        env.fused.gather_start(run.acts["ln2_shard"], "regather_mlp", stream=comm)
        env.fused.gather_start(run.acts["ln1_shard"], "regather_attn", stream=comm)
    run.v["d_fc2"] = BDA.bda_bwd(dout, env.cfg.hidden_dropout, _seed(run, 2), env.training, sm_budget=run.budget("bda_mlp_bwd"))
    run.v["res_grad"] = dout


def b_allgather_mlp_bwd(run):
    env = run.env
    if env.fused_tp:
        if _split_site(env, run.params.linear_mlp_weight, True):
            env.fused.gather_start(_use(run, run.v["d_fc2"]), "mlp_l_bwd")
        run.v["d_fc2_shard"] = run.v.pop("d_fc2")
    else:
        run.v["d_fc2_full"], _ = C.gather_along_first_dim(_use(run, run.v.pop("d_fc2")), env.ps.tp_group)


def b_gemm_dgrad_mlp_l(run):
    env, p = run.env, run.params
    if env.fused_tp and _split_site(env, p.linear_mlp_weight, True):
        _use(run, run.v.pop("d_fc2_shard"))
        full, sync = env.fused.gather_consume("mlp_l_bwd")
        d_act = G.gemm_nn(full, p.linear_mlp_weight, sm_budget=run.budget("gemm_dgrad_mlp_l"), sync=sync)
        run.v["d_fc2_full"] = full
    elif env.fused_tp:
        d_act, full = env.fused.ag_gemm(_use(run, run.v.pop("d_fc2_shard")), p.linear_mlp_weight, "mlp_l_bwd", transpose_w=True,
                                        sm_budget=run.budget("gemm_dgrad_mlp_l"))
        run.v["d_fc2_full"] = full
    else:
        d_act = G.gemm_nn(_use(run, run.v["d_fc2_full"]), p.linear_mlp_weight, sm_budget=run.budget("gemm_dgrad_mlp_l"))
    run.v["d_act"] = d_act


def b_gemm_wgrad_mlp_l(run):
    p = run.params
    G.gemm_tn_acc(_use(run, run.v["d_fc2_full"]), _use(run, run.acts.pop("act")), p.linear_mlp_weight.main_grad,
                  sm_budget=run.budget("gemm_wgrad_mlp_l"))


def b_act_bwd(run):
    d_act = _use(run, run.v.pop("d_act"))
    fc1 = _use(run, run.acts.pop("fc1"))
    if run.env.cfg.gated:
        run.v["d_fc1"] = A.swiglu_bwd(d_act, fc1, sm_budget=run.budget("swiglu_bwd"))
    else:
        run.v["d_fc1"] = A.gelu_bwd(d_act, fc1, sm_budget=run.budget("gelu_bwd"))


def b_gemm_dgrad_mlp_c(run):
    env, p = run.env, run.params
    d_fc1 = _use(run, run.v["d_fc1"])
    if env.fused_tp and _split_site(env, p.column_mlp_weight, True):
        part, sync = env.fused.partial_produce("mlp_c_bwd", d_fc1.shape[0], p.column_mlp_weight.shape[1])
        G.gemm_nn(d_fc1, p.column_mlp_weight, out=part, sm_budget=run.budget("gemm_dgrad_mlp_c"), sync=sync)
    elif env.fused_tp:
        run.v["d_ln2"] = env.fused.gemm_rs(d_fc1, p.column_mlp_weight, "mlp_c_bwd", transpose_w=True,
                                           sm_budget=run.budget("gemm_dgrad_mlp_c"))
    else:
        run.v["d_ln2_partial"] = G.gemm_nn(d_fc1, p.column_mlp_weight, sm_budget=run.budget("gemm_dgrad_mlp_c"))


def b_gemm_wgrad_mlp_c(run):
    p = run.params
    if run.env.fused_tp:
        run.acts.pop("ln2_shard")
        full = run.env.fused.gather_wait("regather_mlp")
    else:
        full = _use(run, run.acts.pop("ln2_full"))
    G.gemm_tn_acc(_use(run, run.v["d_fc1"]), full, p.column_mlp_weight.main_grad, sm_budget=run.budget("gemm_wgrad_mlp_c"))


def b_reduce_scatter_mlp_c_bwd(run):
    env = run.env
    if not env.fused_tp:
        run.v["d_ln2"], _ = C.reduce_scatter_along_first_dim(_use(run, run.v.pop("d_ln2_partial")), env.ps.tp_group)
    elif "d_ln2" not in run.v:
        run.v["d_ln2"] = env.fused.rs_reduce("mlp_c_bwd")


def b_ln_mlp_bwd(run):
    p = run.params
    d_h1 = _norm_bwd(run.env, _use(run, run.v.pop("d_ln2")), _use(run, run.acts.pop("h1")), p.ln_mlp_weight, p.get("ln_mlp_bias"),
                     run.acts.pop("ln2_stat"), run.v.pop("res_grad"), run.budget("ln_mlp_bwd"))
    run.v["d_h1"] = d_h1


def b_bda_attn_bwd(run):
    env = run.env
    d_h1 = run.v["d_h1"]
    run.v["d_proj"] = BDA.bda_bwd(d_h1, env.cfg.hidden_dropout, _seed(run, 1), env.training, sm_budget=run.budget("bda_attn_bwd"))
    run.v["res_grad2"] = d_h1


def b_allgather_attn_bwd(run):
    env = run.env
    if env.fused_tp:
        if _split_site(env, run.params.linear_attn_weight, True):
            env.fused.gather_start(_use(run, run.v["d_proj"]), "attn_l_bwd")
        run.v["d_proj_shard"] = run.v.pop("d_proj")
    else:
        run.v["d_proj_full"], _ = C.gather_along_first_dim(_use(run, run.v.pop("d_proj")), env.ps.tp_group)


def b_gemm_dgrad_attn_l(run):
    env, p = run.env, run.params
    if env.fused_tp and _split_site(env, p.linear_attn_weight, True):
        _use(run, run.v.pop("d_proj_shard"))
        full, sync = env.fused.gather_consume("attn_l_bwd")
        d_o = G.gemm_nn(full, p.linear_attn_weight, sm_budget=run.budget("gemm_dgrad_attn_l"), sync=sync)
        run.v["d_proj_full"] = full
    elif env.fused_tp:
        d_o, full = env.fused.ag_gemm(_use(run, run.v.pop("d_proj_shard")), p.linear_attn_weight, "attn_l_bwd", transpose_w=True,
                                      sm_budget=run.budget("gemm_dgrad_attn_l"))
        run.v["d_proj_full"] = full
    else:
        d_o = G.gemm_nn(_use(run, run.v["d_proj_full"]), p.linear_attn_weight, sm_budget=run.budget("gemm_dgrad_attn_l"))
    run.v["d_attn_out"] = d_o


def b_gemm_wgrad_attn_l(run):
    p = run.params
    o = _use(run, run.acts["attn_out"])
    G.gemm_tn_acc(_use(run, run.v["d_proj_full"]), o.view(o.shape[0] * o.shape[1], -1), p.linear_attn_weight.main_grad,
                  sm_budget=run.budget("gemm_wgrad_attn_l"))


def b_attn_bwd(run):
    env = run.env
    nq, nkv, d = _heads(env)
    qkv = _use(run, run.acts.pop("qkv"))
    o = _use(run, run.acts["attn_out"])
    lse = _use(run, run.acts.pop("lse"))
    B = run.mb.batch
    q, k, v = _qkv_views(env, qkv, B)
    d_o = _use(run, run.v.pop("d_attn_out")).view(o.shape)
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = _qkv_views(env, dqkv, B)
    ATT.attn_bwd(d_o, q, k, v, o, lse, causal=True, scale=env.softmax_scale, dq=dq, dk=dk, dv=dv,
                 sm_budget=run.budget("attn_bwd"))
    _apply_rope(run, dqkv, inverse=True)
    run.v["d_qkv"] = dqkv


def b_gemm_dgrad_attn_c(run):
    env, p = run.env, run.params
    d_qkv = _use(run, run.v["d_qkv"])
    if env.fused_tp and _split_site(env, p.column_attn_weight, True):
        part, sync = env.fused.partial_produce("attn_c_bwd", d_qkv.shape[0], p.column_attn_weight.shape[1])
        G.gemm_nn(d_qkv, p.column_attn_weight, out=part, sm_budget=run.budget("gemm_dgrad_attn_c"), sync=sync)
    elif env.fused_tp:
        run.v["d_ln1"] = env.fused.gemm_rs(d_qkv, p.column_attn_weight, "attn_c_bwd", transpose_w=True,
                                           sm_budget=run.budget("gemm_dgrad_attn_c"))
    else:
        run.v["d_ln1_partial"] = G.gemm_nn(d_qkv, p.column_attn_weight, sm_budget=run.budget("gemm_dgrad_attn_c"))


def b_gemm_wgrad_attn_c(run):
    p = run.params
    if run.env.fused_tp:
        run.acts.pop("ln1_shard")
        full = run.env.fused.gather_wait("regather_attn")
    else:
        full = _use(run, run.acts.pop("ln1_full"))
    G.gemm_tn_acc(_use(run, run.v["d_qkv"]), full, p.column_attn_weight.main_grad, sm_budget=run.budget("gemm_wgrad_attn_c"))


def b_reduce_scatter_attn_c_bwd(run):
    env = run.env
    if not env.fused_tp:
        run.v["d_ln1"], _ = C.reduce_scatter_along_first_dim(_use(run, run.v.pop("d_ln1_partial")), env.ps.tp_group)
    elif "d_ln1" not in run.v:
        run.v["d_ln1"] = env.fused.rs_reduce("attn_c_bwd")


def b_ln_attn_bwd(run):
    p = run.params
    dx = _norm_bwd(run.env, _use(run, run.v.pop("d_ln1")), _use(run, run.acts.pop("x0")), p.ln_attn_weight, p.get("ln_attn_bias"),
                   run.acts.pop("ln1_stat"), run.v.pop("res_grad2"), run.budget("ln_attn_bwd"))
    run.v["dx"] = dx


# --------------------------------------------------------------------------- symmetric-buffer effects
# What each op of the dense layer does to the double-buffered symmetric-memory sites of
# ``FusedTP`` when the collectives run as their own kernels (the default).  The schedule checker
# (``sched.checker.check_buffer_reuse``) uses it to prove that no rank can overwrite a slot that
# another rank still reads; keep it next to the op functions above, which are the ground truth.
FUSED_BUFFER_EFFECTS = {
    "allgather_attn": [("push", "attn_c")],
    "gemm_attn_c": [("wait_read", "attn_c")],
    "allgather_mlp": [("push", "mlp_c")],
    "gemm_mlp_c": [("wait_read", "mlp_c")],
    "gemm_attn_l": [("write", "attn_l")],
    "reduce_scatter_attn": [("reduce", "attn_l")],
    "gemm_mlp_l": [("write", "mlp_l")],
    "reduce_scatter_mlp": [("reduce", "mlp_l")],
    "bda_mlp_bwd": [("push_s3", "regather_mlp"), ("push_s3", "regather_attn")],
    "allgather_mlp_bwd": [("push", "mlp_l_bwd")],
    "gemm_dgrad_mlp_l": [("wait_read", "mlp_l_bwd")],
    "gemm_wgrad_mlp_l": [("read", "mlp_l_bwd")],
    "gemm_dgrad_mlp_c": [("write", "mlp_c_bwd")],
    "gemm_wgrad_mlp_c": [("wait_read", "regather_mlp")],
    "reduce_scatter_mlp_c_bwd": [("reduce", "mlp_c_bwd")],
    "allgather_attn_bwd": [("push", "attn_l_bwd")],
    "gemm_dgrad_attn_l": [("wait_read", "attn_l_bwd")],
    "gemm_wgrad_attn_l": [("read", "attn_l_bwd")],
    "gemm_dgrad_attn_c": [("write", "attn_c_bwd")],
    "gemm_wgrad_attn_c": [("wait_read", "regather_attn")],
    "reduce_scatter_attn_c_bwd": [("reduce", "attn_c_bwd")],
}


# --------------------------------------------------------------------------- program builder
def _id(name: str) -> int:
    return OP_TABLE_IDX.get(name, -1)


def build_layer_program(cfg: ModelConfig, cp: int = 1) -> LayerProgram:
    """Builds the op graph of one layer for the given model family."""
    from . import moe as MOE
    from ..parallel import cp as CP

    P = LayerProgram(cfg.name)
    act_f, act_b = ("swiglu_mlp", "swiglu_bwd") if cfg.gated else ("gelu_mlp", "gelu_bwd")

    # A reduce-scatter reads its GEMM's partial product row block by row block behind per-block counters,
    # so it only needs the GEMM to have been LAUNCHED, not finished (the executor honours this when the
    # engine runs the row-block-wise reduction; otherwise it is an ordinary dependency).
    pipelined = {"reduce_scatter_attn": ("gemm_attn_l",), "reduce_scatter_mlp": ("gemm_mlp_l",),
                 "reduce_scatter_mlp_c_bwd": ("gemm_dgrad_mlp_c",), "reduce_scatter_attn_c_bwd": ("gemm_dgrad_attn_c",)}

    def add(name, strand, kind, fn, deps, res, deferrable=False):
        P.add(Op(name, strand, kind, fn, tuple(deps), res, _id(name), deferrable, pipelined.get(name, ())))

    # ------------------------------ forward strand
    add("ln_attn", FWD, COMPUTE, f_ln_attn, [], MEM)
    add("allgather_attn", FWD, COMM, f_allgather_attn, ["ln_attn"], NVL)
    add("gemm_attn_c", FWD, COMPUTE, f_gemm_attn_c, ["allgather_attn"], MMA)
    last = "gemm_attn_c"
    if cp > 1:
        for i in range(cp):
            name = f"cp_attn_block_fwd_{i + 1}"
            add(name, FWD, COMM if i < cp - 1 else COMPUTE, CP.make_ring_fwd_step(i, cp), [last], NVL if i < cp - 1 else MMA)
            last = name
    else:
        add("fl_attn", FWD, COMPUTE, f_fl_attn, [last], MMA)
        last = "fl_attn"
    add("gemm_attn_l", FWD, COMPUTE, f_gemm_attn_l, [last], MMA)
    add("reduce_scatter_attn", FWD, COMM, f_reduce_scatter_attn, ["gemm_attn_l"], NVL)
    add("bda_attn", FWD, COMPUTE, f_bda_attn, ["reduce_scatter_attn"], MEM)
    add("ln_mlp", FWD, COMPUTE, f_ln_mlp, ["bda_attn"], MEM)
    if cfg.is_moe:
        add("router_mlp", FWD, COMPUTE, MOE.f_router, ["ln_mlp"], MEM)
        add("dispatch_mlp", FWD, COMM, MOE.f_dispatch, ["router_mlp"], NVL)
        add("gemm_expert_c", FWD, COMPUTE, MOE.f_expert_c, ["dispatch_mlp"], MMA)
        add("act_expert", FWD, COMPUTE, MOE.f_expert_act, ["gemm_expert_c"], MEM)
        add("gemm_expert_l", FWD, COMPUTE, MOE.f_expert_l, ["act_expert"], MMA)
        add("combine_mlp", FWD, COMM, MOE.f_combine, ["gemm_expert_l"], NVL)
        add("bda_mlp", FWD, COMPUTE, f_bda_mlp, ["combine_mlp"], MEM)
    else:
        add("allgather_mlp", FWD, COMM, f_allgather_mlp, ["ln_mlp"], NVL)
        add("gemm_mlp_c", FWD, COMPUTE, f_gemm_mlp_c, ["allgather_mlp"], MMA)
        add(act_f, FWD, COMPUTE, f_act_mlp, ["gemm_mlp_c"], MEM)
        add("gemm_mlp_l", FWD, COMPUTE, f_gemm_mlp_l, [act_f], MMA)
        add("reduce_scatter_mlp", FWD, COMM, f_reduce_scatter_mlp, ["gemm_mlp_l"], NVL)
        add("bda_mlp", FWD, COMPUTE, f_bda_mlp, ["reduce_scatter_mlp"], MEM)

    # ------------------------------ backward strand
    add("bda_mlp_bwd", BWD, COMPUTE, b_bda_mlp_bwd, [], MEM)
    if cfg.is_moe:
        add("combine_mlp_bwd", BWD, COMM, MOE.b_combine_bwd, ["bda_mlp_bwd"], NVL)
        add("gemm_dgrad_expert_l", BWD, COMPUTE, MOE.b_dgrad_expert_l, ["combine_mlp_bwd"], MMA)
        add("gemm_wgrad_expert_l", BWD, COMPUTE, MOE.b_wgrad_expert_l, ["combine_mlp_bwd"], MMA, True)
        add("act_expert_bwd", BWD, COMPUTE, MOE.b_expert_act_bwd, ["gemm_dgrad_expert_l"], MEM)
        add("gemm_dgrad_expert_c", BWD, COMPUTE, MOE.b_dgrad_expert_c, ["act_expert_bwd"], MMA)
        add("gemm_wgrad_expert_c", BWD, COMPUTE, MOE.b_wgrad_expert_c, ["act_expert_bwd"], MMA, True)
        add("dispatch_mlp_bwd", BWD, COMM, MOE.b_dispatch_bwd, ["gemm_dgrad_expert_c"], NVL)
        add("router_mlp_bwd", BWD, COMPUTE, MOE.b_router_bwd, ["dispatch_mlp_bwd"], MEM)
        add("ln_mlp_bwd", BWD, COMPUTE, b_ln_mlp_bwd, ["router_mlp_bwd"], MEM)
    else:
        add("allgather_mlp_bwd", BWD, COMM, b_allgather_mlp_bwd, ["bda_mlp_bwd"], NVL)
        add("gemm_dgrad_mlp_l", BWD, COMPUTE, b_gemm_dgrad_mlp_l, ["allgather_mlp_bwd"], MMA)
        add("gemm_wgrad_mlp_l", BWD, COMPUTE, b_gemm_wgrad_mlp_l, ["gemm_dgrad_mlp_l"], MMA, True)
        add(act_b, BWD, COMPUTE, b_act_bwd, ["gemm_dgrad_mlp_l"], MEM)
        add("gemm_dgrad_mlp_c", BWD, COMPUTE, b_gemm_dgrad_mlp_c, [act_b], MMA)
        add("gemm_wgrad_mlp_c", BWD, COMPUTE, b_gemm_wgrad_mlp_c, [act_b], MMA, True)
        add("reduce_scatter_mlp_c_bwd", BWD, COMM, b_reduce_scatter_mlp_c_bwd, ["gemm_dgrad_mlp_c"], NVL)
        add("ln_mlp_bwd", BWD, COMPUTE, b_ln_mlp_bwd, ["reduce_scatter_mlp_c_bwd"], MEM)
    add("bda_attn_bwd", BWD, COMPUTE, b_bda_attn_bwd, ["ln_mlp_bwd"], MEM)
    add("allgather_attn_bwd", BWD, COMM, b_allgather_attn_bwd, ["bda_attn_bwd"], NVL)
    add("gemm_dgrad_attn_l", BWD, COMPUTE, b_gemm_dgrad_attn_l, ["allgather_attn_bwd"], MMA)
    add("gemm_wgrad_attn_l", BWD, COMPUTE, b_gemm_wgrad_attn_l, ["gemm_dgrad_attn_l"], MMA, True)
    last = "gemm_dgrad_attn_l"
    if cp > 1:
        for i in range(cp + 1):
            name = f"cp_attn_block_bwd_{i + 1}"
            add(name, BWD, COMM if i < cp else COMPUTE, CP.make_ring_bwd_step(i, cp), [last], NVL if i < cp else MMA)
            last = name
    else:
        add("attn_bwd", BWD, COMPUTE, b_attn_bwd, [last], MMA)
        last = "attn_bwd"
    add("gemm_dgrad_attn_c", BWD, COMPUTE, b_gemm_dgrad_attn_c, [last], MMA)
    add("gemm_wgrad_attn_c", BWD, COMPUTE, b_gemm_wgrad_attn_c, [last], MMA, True)
    add("reduce_scatter_attn_c_bwd", BWD, COMM, b_reduce_scatter_attn_c_bwd, ["gemm_dgrad_attn_c"], NVL)
    add("ln_attn_bwd", BWD, COMPUTE, b_ln_attn_bwd, ["reduce_scatter_attn_c_bwd"], MEM)
    return P
