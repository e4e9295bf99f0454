"""dhellam_b200: a Blackwell-native double-strand LLM training engine.

The names below are the ones the reference package exports (dhellam/__init__.py:1-5), so
code written against it finds the same entry points here.
"""
from .ops.gemm import gemm_bwd, gemm_fwd, gemm_fwd_event  # noqa: F401
from .ops.norm import pylayernorm_bwd, pylayernorm_fwd  # noqa: F401
from .ops.comm import gather_along_first_dim, reduce_scatter_along_first_dim  # noqa: F401
from .ops.attention import pymha_varlen_bwd, pymha_varlen_fwd  # noqa: F401
from .common.common import _get_qkv_layout  # noqa: F401

__version__ = "0.1.0"
