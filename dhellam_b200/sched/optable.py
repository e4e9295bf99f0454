"""Op table: stable numeric ids of the schedulable ops.

Ids 0-34 are the reference's (search/op_table.py:1-37) and never change; ops that the
reference does not have (GeLU MLP, expert MLP, ring steps beyond context-parallel size 2)
get ids >= 35.
"""
from __future__ import annotations

OP_TABLE_IDX = {
    "allgather_attn": 0,
    "allgather_attn_bwd": 1,
    "allgather_mlp": 2,
    "allgather_mlp_bwd": 3,
    "reduce_scatter_attn": 4,
    "reduce_scatter_mlp": 5,
    "gemm_dgrad_attn_c": 6,
    "gemm_dgrad_mlp_c": 7,
    "gemm_wgrad_attn_c_reduce_scatter_attn_c_bwd": 8,
    "gemm_wgrad_mlp_c_reduce_scatter_mlp_c_bwd": 9,
    "attn_bwd": 10,
    "fl_attn": 11,
    "bda_attn": 12,
    "bda_mlp": 13,
    "bda_attn_bwd": 14,
    "bda_mlp_bwd": 15,
    "gemm_attn_c": 16,
    "gemm_attn_l": 17,
    "gemm_dgrad_attn_l": 18,
    "gemm_dgrad_mlp_l": 19,
    "gemm_mlp_c": 20,
    "gemm_mlp_l": 21,
    "gemm_wgrad_attn_l": 22,
    "gemm_wgrad_mlp_l": 23,
    "ln_attn": 24,
    "ln_mlp": 25,
    "ln_attn_bwd": 26,
    "ln_mlp_bwd": 27,
    "swiglu_bwd": 28,
    "swiglu_mlp": 29,
    "cp_attn_block_fwd_1": 30,
    "cp_attn_block_fwd_2": 31,
    "cp_attn_block_bwd_1": 32,
    "cp_attn_block_bwd_2": 33,
    "cp_attn_block_bwd_3": 34,
    # ---- extensions
    "gelu_mlp": 35,
    "gelu_bwd": 36,
    "router_mlp": 37,
    "dispatch_mlp": 38,
    "gemm_expert_c": 39,
    "act_expert": 40,
    "gemm_expert_l": 41,
    "combine_mlp": 42,
    "combine_mlp_bwd": 43,
    "gemm_dgrad_expert_l": 44,
    "gemm_wgrad_expert_l": 45,
    "act_expert_bwd": 46,
    "gemm_dgrad_expert_c": 47,
    "gemm_wgrad_expert_c": 48,
    "dispatch_mlp_bwd": 49,
    "router_mlp_bwd": 50,
    # unfused pieces of the two fused reference entries (ids 8, 9)
    "gemm_wgrad_attn_c": 51,
    "gemm_wgrad_mlp_c": 52,
    "reduce_scatter_attn_c_bwd": 53,
    "reduce_scatter_mlp_c_bwd": 54,
}
# ring steps for context-parallel sizes above 2
for _i in range(3, 17):
    OP_TABLE_IDX[f"cp_attn_block_fwd_{_i}"] = 100 + _i
for _i in range(4, 18):
    OP_TABLE_IDX[f"cp_attn_block_bwd_{_i}"] = 200 + _i

OP_TABLE_NAME = {v: k for k, v in OP_TABLE_IDX.items()}
