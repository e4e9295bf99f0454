"""Small helpers kept from the reference's ``dhellam/common/common.py``: rank-0 printing
(:15-17), a workspace accessor (:2-13) and the QKV memory-layout probe (:19-123).

The reference allocates a fresh cuBLAS workspace tensor on every GEMM call; here the kernel
library needs no workspace, so ``get_workspace`` hands out one cached buffer per device for
callers that still ask for one.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_WORKSPACES = {}


def print_rank0(*args, **kwargs):
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*args, **kwargs, flush=True)


def get_workspace_size_bytes() -> int:
    """32 MiB, the size the reference uses on sm >= 90."""
    return 32 * 1024 * 1024


def get_workspace(device=None):
    dev = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
    key = (dev.type, dev.index)
    if key not in _WORKSPACES:
        _WORKSPACES[key] = torch.empty(get_workspace_size_bytes(), dtype=torch.uint8, device=dev)
    return _WORKSPACES[key]


def get_qkv_layout(q, k, v, qkv_format: str = "sbhd") -> str:
    """Names the memory layout of ``q, k, v`` in the TransformerEngine vocabulary.

    For format ``sbhd`` the answer is one of ``sb3hd`` (one buffer, q/k/v interleaved ahead
    of the head dimension), ``sbh3d`` (interleaved after it), ``sbhd_sb2hd`` / ``sbhd_sbh2d``
    (q separate, k/v sharing a buffer) or ``sbhd_sbhd_sbhd`` (three buffers or any other
    arrangement); likewise for ``bshd`` and ``thd``.  The packed QKV rows of this framework,
    ``[q heads | k heads | v heads]`` per token with grouped KV heads, are reported as the
    generic three-tensor layout because the strides inside one buffer are not uniform.
    """
    assert all(x.stride(-1) == 1 for x in (q, k, v)), "q, k and v must have stride 1 in their last dimension!"
    fmt = qkv_format
    pre = fmt[:-2]            # "sb", "bs" or "t"

    def same_storage(*ts):
        p = ts[0].untyped_storage().data_ptr()
        return all(t.untyped_storage().data_ptr() == p for t in ts)

    d = q.shape[-1]
    h = q.shape[-2]
    es = q.element_size()

    def off(t):
        return (t.data_ptr() - t.untyped_storage().data_ptr()) // es

    same_shape = q.shape == k.shape == v.shape
    same_stride = q.stride() == k.stride() == v.stride()
    if same_storage(q, k, v) and same_shape and same_stride:
        dk, dv = off(k) - off(q), off(v) - off(q)
        if dk == d and dv == 2 * d and q.stride(-2) == 3 * d:
            return f"{pre}h3d"
        if dk == h * d and dv == 2 * h * d and q.stride(-3) == 3 * h * d:
            return f"{pre}3hd"
    if same_storage(k, v) and not same_storage(q, k) and k.shape == v.shape and k.stride() == v.stride():
        dv = off(v) - off(k)
        hk = k.shape[-2]
        if dv == d and k.stride(-2) == 2 * d:
            return f"{fmt}_{pre}h2d"
        if dv == hk * d and k.stride(-3) == 2 * hk * d:
            return f"{fmt}_{pre}2hd"
    return f"{fmt}_{fmt}_{fmt}"


# name used by the reference package (dhellam/__init__.py:5)
_get_qkv_layout = get_qkv_layout
