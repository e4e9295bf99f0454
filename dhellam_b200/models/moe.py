"""Routed expert MLP (Mixtral family) as forward/backward strand ops.

The reference advertises expert parallelism (README.md:8) but has no router, dispatch or
expert GEMM in its op set (dhellam/core/dstb.py:24-58); the only trace is an
``all_to_all_single`` entry in its micro-benchmark (micro_benchmark/overlap.py:141-145).
These ops are therefore new: softmax top-k router with the load-balancing auxiliary loss,
dropless token dispatch (permute by expert, variable-size all-to-all over the expert
parallel group), per-expert GEMMs on the tcgen05 kernel over contiguous row groups,
SwiGLU, and the weighted combine; every op has an explicit backward.

Tensor parallelism inside an expert is not combined with expert parallelism here
(``tp`` must be 1 for MoE layers).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import activation as A
from ..ops import comm as C
from ..ops import gemm as G
from ..ops import moe as M


def _use(run, t):
    s = getattr(run.env, "cur_stream", None)
    if s is not None and t is not None and t.is_cuda:
        t.record_stream(s)
    return t


def _dev(run):
    """The device-resident exchange (``ops.moe_native.DeviceMoE``) when this run is on a GPU with the native
    kernels, else None (CPU ranks and the library backend take the host-driven path)."""
    return getattr(run.env, "moe_dev", None)


# --------------------------------------------------------------------------- forward
def f_router(run):
    env, p = run.env, run.params
    assert env.ps.tp == 1, "expert layers need tp = 1"
    x = _use(run, run.v.pop("ln2"))
    probs, topi, gates = M.router_topk_fwd(x, p.router_weight, env.cfg.moe_top_k)
    run.acts["moe_x"], run.acts["moe_probs"], run.acts["moe_topi"], run.acts["moe_gates"] = x, probs, topi, gates
    if env.training and env.cfg.moe_aux_loss_coeff > 0:
        env.moe_aux.append(M.aux_loss(probs, topi, env.cfg.num_experts))
    run.v["moe_x"] = x


def f_dispatch(run):
    env = run.env
    x = _use(run, run.v.pop("moe_x"))
    dev = _dev(run)
    if dev is not None:
        plan = dev.plan(run.acts["moe_topi"].to(torch.int32).contiguous())
        run.acts["moe_plan"] = plan
        slot, _ = dev.dispatch(plan, x, "xe", record=True)
        run.v["moe_xe"] = ("xe", slot)
        return
    plan = M.make_plan(run.acts["moe_topi"], env.cfg.num_experts, env.ps.ep, env.ps.ep_group)
    run.acts["moe_plan"] = plan
    xp = M.permute_rows(x, plan.src_row)                        # rows grouped by (destination rank, expert)
    xr = C.all_to_all_rows(xp, plan.send_counts, plan.recv_counts, env.ps.ep_group)
    xe = M.permute_rows(xr, plan.recv_sort) if plan.recv_sort is not None else xr   # expert-major on the owner
    run.acts["moe_xe"] = xe
    run.v["moe_xe"] = xe


def _expert_loop(plan, fn):
    o = 0
    for e, n in enumerate(plan.expert_rows):
        if n > 0:
            fn(e, o, o + n)
        o += n


def f_expert_c(run):
    p = run.params
    dev = _dev(run)
    if dev is not None:
        site, slot = run.v.pop("moe_xe")
        xe = dev.landed(site, slot)
        z = dev.grouped_nt(xe, p.expert_column_weight, run.acts["moe_plan"], sm_budget=run.budget("gemm_expert_c"))
        run.acts["moe_z"] = z
        run.v["moe_z"] = z
        return
    xe = _use(run, run.v.pop("moe_xe"))
    plan = run.acts["moe_plan"]
    w = p.expert_column_weight
    z = torch.empty((xe.shape[0], w.shape[1]), dtype=xe.dtype, device=xe.device)
    _expert_loop(plan, lambda e, a, b: G.gemm_nt(xe[a:b], w[e], out=z[a:b], sm_budget=run.budget("gemm_expert_c")))
    run.acts["moe_z"] = z
    run.v["moe_z"] = z


def f_expert_act(run):
    z = _use(run, run.v.pop("moe_z"))
    dev = _dev(run)
    if dev is not None and run.env.cfg.gated:
        a = dev.swiglu_fwd(z, run.acts["moe_plan"])          # only the rows in use (count read on the device)
    else:
        a = A.swiglu_fwd(z) if run.env.cfg.gated else A.gelu_fwd(z)
    run.acts["moe_a"] = a
    run.v["moe_a"] = a


def f_expert_l(run):
    p = run.params
    a = _use(run, run.v.pop("moe_a"))
    plan = run.acts["moe_plan"]
    dev = _dev(run)
    if dev is not None:
        y, slot = dev.output_buffer("y")
        dev.grouped_nt(a, p.expert_linear_weight, plan, out=y, sm_budget=run.budget("gemm_expert_l"))
        dev.publish("y", slot)
        run.v["moe_y"] = ("y", slot)
        return
    w = p.expert_linear_weight
    y = torch.empty((a.shape[0], w.shape[1]), dtype=a.dtype, device=a.device)
    _expert_loop(plan, lambda e, lo, hi: G.gemm_nt(a[lo:hi], w[e], out=y[lo:hi], sm_budget=run.budget("gemm_expert_l")))
    run.v["moe_y"] = y


def f_combine(run):
    env = run.env
    dev = _dev(run)
    if dev is not None:
        site, slot = run.v.pop("moe_y")
        out, yb = dev.combine(run.acts["moe_plan"], site, slot, gates=run.acts["moe_gates"].contiguous(), keep_copies=True)
        run.acts["moe_yb"] = yb
        run.v["fc2"] = out
        return
    y = _use(run, run.v.pop("moe_y"))
    plan = run.acts["moe_plan"]
    yr = M.unpermute_rows(y, plan.recv_sort) if plan.recv_sort is not None else y
    yb = C.all_to_all_rows(yr, plan.recv_counts, plan.send_counts, env.ps.ep_group)
    run.acts["moe_yb"] = yb                                     # per (token, k) expert outputs, dispatch order
    run.v["fc2"] = M.combine_rows(yb, plan, run.acts["moe_gates"])


# --------------------------------------------------------------------------- backward
def b_combine_bwd(run):
    env = run.env
    d_out = _use(run, run.v.pop("d_fc2"))                       # [T, h]
    plan = run.acts["moe_plan"]
    gates = run.acts["moe_gates"]
    yb = _use(run, run.acts.pop("moe_yb"))
    dev = _dev(run)
    if dev is not None:
        # d(copy) = gate * d_out[token] pushed to the owners; the gate gradient <d_out[token], copy> on the side;
        # the token rows are pushed again for the expert weight gradient (instead of keeping the landing buffer alive)
        slot, dots = dev.dispatch(plan, d_out, "dy", scale=gates.contiguous(), other=yb)
        run.v["d_gates"] = dots.view_as(gates)
        slot_x, _ = dev.dispatch(plan, _use(run, run.acts["moe_x"]), "xeb")
        run.v["d_y"] = ("dy", slot)
        run.v["moe_xeb"] = ("xeb", slot_x)
        return
    d_yb, d_gates = M.combine_rows_bwd(d_out, yb, plan, gates)
    run.v["d_gates"] = d_gates
    d_yr = C.all_to_all_rows(d_yb, plan.send_counts, plan.recv_counts, env.ps.ep_group)
    run.v["d_y"] = M.permute_rows(d_yr, plan.recv_sort) if plan.recv_sort is not None else d_yr


def _landed_dy(run):
    """Device path: the first consumer of the pushed output gradients waits for their arrival."""
    d_y = run.v["d_y"]
    if isinstance(d_y, tuple):
        d_y = _dev(run).landed(*d_y)
        run.v["d_y"] = d_y
    return d_y


def b_dgrad_expert_l(run):
    p = run.params
    plan = run.acts["moe_plan"]
    dev = _dev(run)
    if dev is not None:
        d_y = _landed_dy(run)
        run.v["d_a"] = dev.grouped_nn(d_y, p.expert_linear_weight, plan, sm_budget=run.budget("gemm_dgrad_expert_l"))
        return
    d_y = _use(run, run.v["d_y"])
    w = p.expert_linear_weight
    d_a = torch.empty((d_y.shape[0], w.shape[2]), dtype=d_y.dtype, device=d_y.device)
    _expert_loop(plan, lambda e, lo, hi: G.gemm_nn(d_y[lo:hi], w[e], out=d_a[lo:hi], sm_budget=run.budget("gemm_dgrad_expert_l")))
    run.v["d_a"] = d_a


def b_wgrad_expert_l(run):
    p = run.params
    d_y = _landed_dy(run) if _dev(run) is not None else _use(run, run.v["d_y"])
    a = _use(run, run.acts.pop("moe_a"))
    plan = run.acts["moe_plan"]
    mg = p.expert_linear_weight.main_grad
    dev = _dev(run)
    if dev is not None and mg.shape[1] % 256 == 0:
        dev.grouped_tn_acc(d_y, a, mg, plan, sm_budget=run.budget("gemm_wgrad_expert_l"))
        return
    if dev is not None:
        raise NotImplementedError("grouped expert weight gradients need the expert output width to be a multiple of 256")
    _expert_loop(plan, lambda e, lo, hi: G.gemm_tn_acc(d_y[lo:hi], a[lo:hi], mg[e], sm_budget=run.budget("gemm_wgrad_expert_l")))


def b_expert_act_bwd(run):
    d_a = _use(run, run.v.pop("d_a"))
    z = _use(run, run.acts.pop("moe_z"))
    dev = _dev(run)
    if dev is not None and run.env.cfg.gated:
        run.v["d_z"] = dev.swiglu_bwd(d_a, z, run.acts["moe_plan"])
        return
    run.v["d_z"] = A.swiglu_bwd(d_a, z) if run.env.cfg.gated else A.gelu_bwd(d_a, z)


def b_dgrad_expert_c(run):
    p = run.params
    d_z = _use(run, run.v["d_z"])
    plan = run.acts["moe_plan"]
    dev = _dev(run)
    if dev is not None:
        d_xe, slot = dev.output_buffer("dxe")
        dev.grouped_nn(d_z, p.expert_column_weight, plan, out=d_xe, sm_budget=run.budget("gemm_dgrad_expert_c"))
        dev.publish("dxe", slot)
        run.v["d_xe"] = ("dxe", slot)
        return
    w = p.expert_column_weight
    d_xe = torch.empty((d_z.shape[0], w.shape[2]), dtype=d_z.dtype, device=d_z.device)
    _expert_loop(plan, lambda e, lo, hi: G.gemm_nn(d_z[lo:hi], w[e], out=d_xe[lo:hi], sm_budget=run.budget("gemm_dgrad_expert_c")))
    run.v["d_xe"] = d_xe


def b_wgrad_expert_c(run):
    p = run.params
    d_z = _use(run, run.v["d_z"])
    plan = run.acts["moe_plan"]
    mg = p.expert_column_weight.main_grad
    dev = _dev(run)
    if dev is not None:
        if mg.shape[1] % 256 != 0:
            raise NotImplementedError("grouped expert weight gradients need the expert FFN width to be a multiple of 256")
        site, slot = run.v.pop("moe_xeb")
        dev.grouped_tn_acc(d_z, dev.landed(site, slot), mg, plan, sm_budget=run.budget("gemm_wgrad_expert_c"))
        return
    xe = _use(run, run.acts.pop("moe_xe"))
    _expert_loop(plan, lambda e, lo, hi: G.gemm_tn_acc(d_z[lo:hi], xe[lo:hi], mg[e], sm_budget=run.budget("gemm_wgrad_expert_c")))


def b_dispatch_bwd(run):
    env = run.env
    plan = run.acts["moe_plan"]
    dev = _dev(run)
    if dev is not None:
        site, slot = run.v.pop("d_xe")
        run.v["d_moe_x"], _ = dev.combine(plan, site, slot)            # plain sum over the k copies of a token
        return
    d_xe = _use(run, run.v.pop("d_xe"))
    d_xr = M.unpermute_rows(d_xe, plan.recv_sort) if plan.recv_sort is not None else d_xe
    d_xp = C.all_to_all_rows(d_xr, plan.recv_counts, plan.send_counts, env.ps.ep_group)
    run.v["d_moe_x"] = M.scatter_add_rows(d_xp, plan.src_row, plan.num_tokens)      # sum over the k copies of a token


def b_router_bwd(run):
    env, p = run.env, run.params
    x = _use(run, run.acts.pop("moe_x"))
    probs, topi, gates = run.acts.pop("moe_probs"), run.acts.pop("moe_topi"), run.acts.pop("moe_gates")
    run.acts.pop("moe_plan")
    aux_scale = env.cfg.moe_aux_loss_coeff * getattr(env, "grad_scale", 1.0) if env.training else 0.0
    d_logits = M.router_topk_bwd(run.v.pop("d_gates"), probs, topi, gates, env.cfg.num_experts, aux_scale)
    dl = d_logits.to(x.dtype)
    d_x = run.v.pop("d_moe_x")
    E = dl.shape[1]
    if dl.is_cuda and E % 8 != 0:
        # the tensor-core GEMM needs 16-byte rows: pad the expert dimension with zeros
        pad = (-E) % 8
        dl = torch.nn.functional.pad(dl, (0, pad))
        w_pad = torch.nn.functional.pad(p.router_weight, (0, 0, 0, pad))
        g_pad = torch.zeros((E + pad, x.shape[1]), dtype=torch.float32, device=x.device)
        d_x = d_x + G.gemm_nn(dl, w_pad).to(d_x.dtype)
        G.gemm_tn_acc(dl, x, g_pad, accumulate=False)
        p.router_weight.main_grad.add_(g_pad[:E])
    else:
        d_x = d_x + G.gemm_nn(dl, p.router_weight).to(d_x.dtype)
        G.gemm_tn_acc(dl, x, p.router_weight.main_grad)
    run.v["d_ln2"] = d_x.to(x.dtype)
