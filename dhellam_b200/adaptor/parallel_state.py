"""Tensor-parallel state shim with the reference's function names
(dhellam/adaptor/parallel_state.py:10-38).  It forwards to ``dhellam_b200.parallel.state``
unless a group was set explicitly, so code written against either API sees one state."""
from __future__ import annotations

import torch.distributed as dist

from ..parallel import state as _state

_TENSOR_MODEL_PARALLEL_GROUP = None


def set_tensor_model_parallel_group(group):
    global _TENSOR_MODEL_PARALLEL_GROUP
    _TENSOR_MODEL_PARALLEL_GROUP = group


def get_tensor_model_parallel_group():
    if _TENSOR_MODEL_PARALLEL_GROUP is not None:
        return _TENSOR_MODEL_PARALLEL_GROUP
    return _state.get_tensor_model_parallel_group()


def get_tensor_model_parallel_world_size():
    g = _TENSOR_MODEL_PARALLEL_GROUP
    if g is not None:
        return dist.get_world_size(group=g)
    return _state.get_tensor_model_parallel_world_size()


def get_tensor_model_parallel_rank():
    g = _TENSOR_MODEL_PARALLEL_GROUP
    if g is not None:
        return dist.get_rank(group=g)
    return _state.get_tensor_model_parallel_rank()
