"""Mixture-of-experts primitives: router, dispatch plan, row permutations, combine.

New relative to the reference (it has no MoE ops; see ``models/moe.py``).  The router runs
as one sm_100a kernel on CUDA tensors (csrc/head_optim.cu, ``router_kernel``: logits, softmax, top-k and gate
normalisation in one pass over the token row); the plan and the permutations use index
arithmetic on the device, and the only host read is the per-expert row count that sizes
the expert GEMMs (dropless routing has data-dependent shapes).
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import kernels as K
from .comm import group_size


# --------------------------------------------------------------------------- router
def router_topk_fwd(x, w, k: int):
    """``x [T,h]``, ``w [E,h]`` -> ``(probs [T,E] fp32, topi [T,k] int64, gates [T,k] fp32)``
    with ``gates`` the selected probabilities renormalised to sum to one."""
    T, h = x.shape
    E = w.shape[0]
    if x.is_cuda and E <= 64 and k <= 8:
        probs = torch.empty((T, E), dtype=torch.float32, device=x.device)
        topi32 = torch.empty((T, k), dtype=torch.int32, device=x.device)
        gates = torch.empty((T, k), dtype=torch.float32, device=x.device)
        fn = K.proto("dh_router_topk", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        K.check(fn(x.data_ptr(), w.data_ptr(), probs.data_ptr(), topi32.data_ptr(), gates.data_ptr(), T, h, E, k,
                   K.stream_ptr(None)), "dh_router_topk")
        return probs, topi32.long(), gates
    logits = x.float() @ w.float().t()
    probs = torch.softmax(logits, dim=-1)
    topv, topi = probs.topk(k, dim=-1)
    gates = topv / topv.sum(-1, keepdim=True)
    return probs, topi, gates


def aux_loss(probs, topi, E: int):
    """Load-balancing loss ``E * sum_e f_e * P_e`` (fraction routed x mean probability)."""
    frac = torch.zeros(E, dtype=torch.float32, device=probs.device)
    frac.index_add_(0, topi.reshape(-1), torch.ones(topi.numel(), dtype=torch.float32, device=probs.device))
    frac = frac / topi.numel()
    return E * (frac * probs.mean(0)).sum()


def router_topk_bwd(d_gates, probs, topi, gates, E: int, aux_scale: float = 0.0):
    """Gradient with respect to the router logits ``[T,E]`` (fp32)."""
    T = probs.shape[0]
    topv_sum = probs.gather(1, topi).sum(-1, keepdim=True)
    d_topv = (d_gates - (d_gates * gates).sum(-1, keepdim=True)) / topv_sum
    d_probs = torch.zeros_like(probs)
    d_probs.scatter_add_(1, topi, d_topv)
    if aux_scale:
        frac = torch.zeros(E, dtype=torch.float32, device=probs.device)
        frac.index_add_(0, topi.reshape(-1), torch.ones(topi.numel(), dtype=torch.float32, device=probs.device))
        frac = frac / topi.numel()
        d_probs = d_probs + aux_scale * E * frac[None, :] / T
    return probs * (d_probs - (d_probs * probs).sum(-1, keepdim=True))


# --------------------------------------------------------------------------- dispatch plan
@dataclass
class DispatchPlan:
    num_tokens: int
    src_row: torch.Tensor            # [T*k] token index of every dispatched copy, grouped by expert
    src_slot: torch.Tensor           # [T*k] flat (token * k + choice) index of every copy
    send_counts: List[int]           # rows sent to every expert-parallel rank
    recv_counts: List[int]           # rows received from every rank
    recv_sort: Optional[torch.Tensor]  # permutation (src-rank major -> expert major) on the receiver
    expert_rows: List[int]           # rows per local expert after the exchange


def make_plan(topi, E: int, ep: int, group) -> DispatchPlan:
    T, k = topi.shape
    flat = topi.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    src_slot = order
    src_row = torch.div(order, k, rounding_mode="floor")
    counts = torch.bincount(flat, minlength=E)                    # per global expert
    el = E // ep
    if ep == 1:
        c = counts.tolist()
        return DispatchPlan(T, src_row, src_slot, [int(sum(c))], [int(sum(c))], None, [int(v) for v in c])
    send_mat = counts.view(ep, el)                                # [dest rank, local expert]
    recv_mat = torch.empty_like(send_mat)                         # [src rank, local expert]
    dist.all_to_all_single(recv_mat, send_mat.contiguous(), group=group)
    rm = recv_mat.tolist()
    send_counts = [int(v) for v in send_mat.sum(1).tolist()]
    recv_counts = [int(sum(r)) for r in rm]
    # received rows are ordered (src rank, local expert); sort them expert-major
    seg_expert = torch.tensor([e for s in range(ep) for e in range(el)], device=topi.device)
    seg_len = recv_mat.reshape(-1)
    row_expert = torch.repeat_interleave(seg_expert, seg_len)
    recv_sort = torch.sort(row_expert, stable=True).indices
    expert_rows = [int(sum(rm[s][e] for s in range(ep))) for e in range(el)]
    return DispatchPlan(T, src_row, src_slot, send_counts, recv_counts, recv_sort, expert_rows)


# --------------------------------------------------------------------------- row movement
def permute_rows(x, index):
    """``out[i] = x[index[i]]``."""
    return x.index_select(0, index)


def unpermute_rows(x, index):
    """Inverse of ``permute_rows``: ``out[index[i]] = x[i]``."""
    out = torch.empty_like(x)
    out.index_copy_(0, index, x)
    return out


def scatter_add_rows(x, index, n_rows: int):
    """``out[index[i]] += x[i]`` with fp32 accumulation."""
    out = torch.zeros((n_rows, x.shape[1]), dtype=torch.float32, device=x.device)
    out.index_add_(0, index, x.float())
    return out


def combine_rows(yb, plan: DispatchPlan, gates):
    """Weighted un-permute: ``out[token] = sum_k gate[token,k] * y[copy(token,k)]``."""
    g = gates.reshape(-1).index_select(0, plan.src_slot)          # gate of every copy, dispatch order
    out = torch.zeros((plan.num_tokens, yb.shape[1]), dtype=torch.float32, device=yb.device)
    out.index_add_(0, plan.src_row, yb.float() * g[:, None])
    return out.to(yb.dtype)


def combine_rows_bwd(d_out, yb, plan: DispatchPlan, gates):
    """Returns ``(d_yb [T*k,h], d_gates [T,k] fp32)``."""
    g = gates.reshape(-1).index_select(0, plan.src_slot)
    d_rows = d_out.index_select(0, plan.src_row).float()
    d_yb = (d_rows * g[:, None]).to(yb.dtype)
    d_copy = (d_rows * yb.float()).sum(-1)
    d_gates = torch.zeros(gates.numel(), dtype=torch.float32, device=yb.device)
    d_gates.index_copy_(0, plan.src_slot, d_copy)
    return d_yb, d_gates.view_as(gates)
