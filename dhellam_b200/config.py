"""Model / parallelism / training configuration and the named model presets.

The reference takes its configuration from Megatron's argparse namespace plus two flags
(dhellam/adaptor/megatron.py:33-38) and bash variables (script/run.sh:6-34); here the same
information lives in three dataclasses that the Megatron-style argument parser in
``adaptor/args.py`` fills.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Optional


@dataclass
class ModelConfig:
    name: str = "custom"
    num_layers: int = 2
    hidden_size: int = 256
    ffn_hidden_size: int = 688
    num_attention_heads: int = 4
    num_query_groups: int = 2            # KV heads
    head_dim: Optional[int] = None       # default hidden / heads
    vocab_size: int = 1024
    seq_length: int = 128
    norm: str = "rmsnorm"                # rmsnorm | layernorm
    activation: str = "swiglu"           # swiglu | gelu
    position: str = "rope"               # rope | learned
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    hidden_dropout: float = 0.0
    tie_embeddings: bool = True          # the reference ties the LM head to the embedding (core/dshb.py:256-262)
    init_std: float = 0.02
    # mixture of experts
    num_experts: int = 0
    moe_top_k: int = 2
    moe_aux_loss_coeff: float = 0.01

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def gated(self) -> bool:
        return self.activation == "swiglu"

    def layer_params(self) -> int:
        h, f, d = self.hidden_size, self.ffn_hidden_size, self.head_dim
        attn = h * (self.num_attention_heads + 2 * self.num_query_groups) * d + self.num_attention_heads * d * h
        mlp = (3 if self.gated else 2) * h * f
        if self.is_moe:
            mlp = mlp * self.num_experts + h * self.num_experts
        return attn + mlp + 2 * h

    def total_params(self) -> int:
        emb = self.vocab_size * self.hidden_size * (1 if self.tie_embeddings else 2)
        return self.num_layers * self.layer_params() + emb + self.hidden_size

    def flops_per_token(self, seq_length: Optional[int] = None, causal: bool = True) -> float:
        """Model FLOPs (forward + backward = 3x forward) per token, the usual 6N + attention form."""
        s = seq_length or self.seq_length
        h, f, d = self.hidden_size, self.ffn_hidden_size, self.head_dim
        nq, nkv = self.num_attention_heads, self.num_query_groups
        lin = 2 * h * (nq + 2 * nkv) * d + 2 * nq * d * h
        experts = self.moe_top_k if self.is_moe else 1
        lin += 2 * (3 if self.gated else 2) * h * f * experts
        if self.is_moe:
            lin += 2 * h * self.num_experts
        attn = 4 * nq * d * s * (0.5 if causal else 1.0)
        head = 2 * h * self.vocab_size
        return 3.0 * (self.num_layers * (lin + attn) + head)


@dataclass
class ParallelConfig:
    tp: int = 1
    cp: int = 1
    pp: int = 1
    ep: int = 1
    dp: int = 1
    sequence_parallel: bool = True

    def __post_init__(self):
        # Like the reference (its layer graph is LN -> all-gather -> GEMM ... GEMM -> reduce-scatter,
        # dhellam/core/dstb.py:700-757), this engine always shards the activations between
        # tensor-parallel regions along the sequence.  Tensor parallelism without it is not built,
        # so asking for it is an error rather than a silently different run.
        if self.tp > 1 and not self.sequence_parallel:
            raise ValueError("tensor parallelism here always uses sequence parallelism: pass --sequence-parallel "
                             "(ParallelConfig(sequence_parallel=True)) when tp > 1")

    @property
    def world(self) -> int:
        return self.tp * self.cp * self.pp * self.dp

    def describe(self) -> str:
        parts = []
        for k in ("dp", "tp", "cp", "pp", "ep"):
            v = getattr(self, k)
            if v > 1:
                parts.append(f"{k}{v}")
        s = "x".join(parts) or "single"
        return s + ("+sp" if self.tp > 1 and self.sequence_parallel else "")


@dataclass
class TrainConfig:
    micro_batch_size: int = 2
    global_batch_size: int = 8
    lr: float = 6.0e-5
    min_lr: float = 6.0e-6
    weight_decay: float = 0.1
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    dtype: str = "bf16"                  # bf16 | fp32
    seed: int = 1234
    fused_comm: bool = True              # in-kernel collectives (peer memory) instead of NCCL
    schedule_config: Optional[str] = None
    dhellam: bool = True                 # dual-strand scheduling on/off (the reference's --dhellam)
    compute_streams: int = 1             # 1: both strands' compute in schedule order on one stream; 2: co-run
    train_iters: int = 2
    log_interval: int = 1
    save: Optional[str] = None
    load: Optional[str] = None
    save_interval: int = 10000
    distributed_timeout_minutes: float = 2.0
    # loss scaling (Megatron's --loss-scale / --initial-loss-scale / --loss-scale-window / --hysteresis /
    # --min-loss-scale): a constant factor, or the dynamic scaler that halves on overflow and doubles after a
    # window of good steps.  bf16 needs neither; it is there for 16-bit runs configured the reference's way.
    loss_scale: float = 1.0
    dynamic_loss_scale: bool = False
    initial_loss_scale: float = 65536.0
    loss_scale_window: int = 1000
    hysteresis: int = 2
    min_loss_scale: float = 1.0
    label_smoothing: float = 0.0         # Megatron's --label-smoothing-factor
    # the two switches of the benchmark's composition arm: the reference's built-in 17-block schedule
    # (dhellam/core/dstb.py:1043-1059) and its device-wide synchronisation after every block (:1266)
    reference_schedule: bool = False
    sync_per_block: bool = False
    deterministic: bool = False          # Megatron's --deterministic-mode: fixed-order reductions, bitwise repeatable runs

    def num_microbatches(self, dp: int) -> int:
        assert self.global_batch_size % (self.micro_batch_size * dp) == 0, "global batch must divide by micro-batch x dp"
        return self.global_batch_size // (self.micro_batch_size * dp)


# --------------------------------------------------------------------------- presets
PRESETS = {
    # plumbing config (CPU / gloo)
    "tiny-llama": ModelConfig(name="tiny-llama", num_layers=2, hidden_size=256, ffn_hidden_size=688, num_attention_heads=4,
                              num_query_groups=2, vocab_size=1024, seq_length=128, rope_theta=10000.0),
    # headline: Llama-3.1-70B architecture truncated to 8 layers (script/run.sh:11-33 in the reference)
    "llama3.1-70b-8l": ModelConfig(name="llama3.1-70b-8l", num_layers=8, hidden_size=8192, ffn_hidden_size=28672,
                                   num_attention_heads=64, num_query_groups=8, vocab_size=128256, seq_length=4096,
                                   rope_theta=500000.0),
    "llama3-8b": ModelConfig(name="llama3-8b", num_layers=32, hidden_size=4096, ffn_hidden_size=14336,
                             num_attention_heads=32, num_query_groups=8, vocab_size=128256, seq_length=65536,
                             rope_theta=500000.0),
    "mixtral-8x7b-8l": ModelConfig(name="mixtral-8x7b-8l", num_layers=8, hidden_size=4096, ffn_hidden_size=14336,
                                   num_attention_heads=32, num_query_groups=8, vocab_size=32000, seq_length=16384,
                                   rope_theta=1000000.0, num_experts=8, moe_top_k=2, moe_aux_loss_coeff=0.01),
    "gpt-13b": ModelConfig(name="gpt-13b", num_layers=40, hidden_size=5120, ffn_hidden_size=20480, num_attention_heads=40,
                           num_query_groups=40, vocab_size=50304, seq_length=8192, norm="layernorm", activation="gelu",
                           position="rope", rope_theta=10000.0),
    "tiny-gpt": ModelConfig(name="tiny-gpt", num_layers=2, hidden_size=128, ffn_hidden_size=512, num_attention_heads=4,
                            num_query_groups=4, vocab_size=512, seq_length=64, norm="layernorm", activation="gelu"),
    "tiny-moe": ModelConfig(name="tiny-moe", num_layers=2, hidden_size=128, ffn_hidden_size=256, num_attention_heads=4,
                            num_query_groups=2, vocab_size=512, seq_length=64, num_experts=4, moe_top_k=2),
}


def preset(name: str, **overrides) -> ModelConfig:
    return replace(PRESETS[name], **overrides)


def to_dict(cfg) -> dict:
    return asdict(cfg)
