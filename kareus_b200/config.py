"""Model, GPU and parallelism configuration.

Covers the reference's model/GPU registry (``tests/bayesian/common/model_config.py:13-129``)
and the subset of Megatron's ``TransformerConfig`` / ``ModelParallelConfig`` that the
partition engine reads (``3rdparty/Megatron-LM/megatron/core/model_parallel_config.py:104-112``).
Unlike the reference, the model config and the parallel layout are plain dataclasses with no
dependency on Megatron.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


# --------------------------------------------------------------------------- GPUs
# ``p2p_power_w`` is the static ("blocked in a p2p wait") board power that the planner
# subtracts to get effective energy.  A100/A40 values are the reference's; the B200 value was measured
# with `kareus_b200.energy.p2p_probe` (20 s blocked in an NCCL receive, HGX B200, 1000 W limit: 251 W).
GPU_CONFIGS: Dict[str, dict] = {
    "A40": {"p2p_power_w": 70.0, "freq_range": (900, 1740, 30)},
    "A100": {"p2p_power_w": 85.0, "freq_range": (900, 1410, 30)},
    # B200: 1965 MHz max SM clock; under dense GEMM the part is power limited near 1.3 GHz,
    # so the useful search range ends well below the maximum.
    "B200": {"p2p_power_w": 251.0, "freq_range": (900, 1965, 75)},
}
DEFAULT_GPU = "B200"


def get_p2p_power(gpu_type: str) -> float:
    if gpu_type not in GPU_CONFIGS:
        raise ValueError(f"Unknown GPU type {gpu_type!r}; known: {sorted(GPU_CONFIGS)}")
    return float(GPU_CONFIGS[gpu_type]["p2p_power_w"])


def get_freq_grid(gpu_type: str) -> list:
    """Clock grid, highest first (reference: ``tests/bayesian/common/runner.py:192-196``)."""
    lo, hi, step = GPU_CONFIGS[gpu_type]["freq_range"]
    out = []
    f = hi
    while f >= lo:
        out.append(int(f))
        f -= step
    return out


# --------------------------------------------------------------------------- model
@dataclass(frozen=True)
class ModelConfig:
    """Llama-family decoder architecture."""

    name: str
    hidden_size: int
    num_attention_heads: int
    num_query_groups: int
    ffn_hidden_size: int
    num_layers: int
    vocab_size: int = 128256
    head_dim: Optional[int] = None
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    hidden_dropout: float = 0.0
    qk_layernorm: bool = False
    tie_embeddings: bool = False
    max_seq_len: int = 4096
    init_std: float = 0.02
    num_layers_in_first_pipeline_stage: Optional[int] = None

    @property
    def hd(self) -> int:
        return self.head_dim if self.head_dim is not None else self.hidden_size // self.num_attention_heads

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)

    def num_params(self) -> int:
        h, f, L, v = self.hidden_size, self.ffn_hidden_size, self.num_layers, self.vocab_size
        qkv = h * (self.num_attention_heads + 2 * self.num_query_groups) * self.hd
        proj = self.num_attention_heads * self.hd * h
        mlp = 3 * h * f
        per_layer = qkv + proj + mlp + 2 * h
        emb = v * h * (1 if self.tie_embeddings else 2)
        return L * per_layer + emb + h

    def flops_per_token(self, seq_len: int, recompute: bool = True) -> float:
        """Model FLOPs per token for fwd+bwd (+1 fwd when fully recomputing), causal attention."""
        h, f, L, v = self.hidden_size, self.ffn_hidden_size, self.num_layers, self.vocab_size
        qkv = h * (self.num_attention_heads + 2 * self.num_query_groups) * self.hd
        proj = self.num_attention_heads * self.hd * h
        dense = 2 * (qkv + proj + 3 * h * f)
        attn = 2 * 2 * self.num_attention_heads * self.hd * seq_len / 2  # QK^T and PV, causal half
        layer_fwd = dense + attn
        head_fwd = 2 * h * v
        mult_layer = 4.0 if recompute else 3.0
        return L * layer_fwd * mult_layer + head_fwd * 3.0


MODEL_REGISTRY: Dict[str, ModelConfig] = {
    "llama3.2_3b": ModelConfig(
        name="llama3.2_3b", hidden_size=3072, num_attention_heads=24, num_query_groups=8,
        ffn_hidden_size=8192, num_layers=28, vocab_size=128256, head_dim=128,
        rope_theta=500000.0, num_layers_in_first_pipeline_stage=15,
    ),
    "llama3.1_8b": ModelConfig(
        name="llama3.1_8b", hidden_size=4096, num_attention_heads=32, num_query_groups=8,
        ffn_hidden_size=14336, num_layers=32, vocab_size=128256, head_dim=128,
        rope_theta=500000.0,
    ),
    "llama_13b": ModelConfig(
        name="llama_13b", hidden_size=5120, num_attention_heads=40, num_query_groups=40,
        ffn_hidden_size=13824, num_layers=40, vocab_size=32000, head_dim=128,
        rope_theta=10000.0,
    ),
    "qwen3_1.7b": ModelConfig(
        name="qwen3_1.7b", hidden_size=2048, num_attention_heads=16, num_query_groups=8,
        ffn_hidden_size=6144, num_layers=28, vocab_size=151936, head_dim=128,
        rope_theta=1000000.0, norm_eps=1e-6, qk_layernorm=True, tie_embeddings=True,
        num_layers_in_first_pipeline_stage=15,
    ),
    # CPU plumbing model: 2 layers, hidden 256, 4 heads / 2 KV heads, SwiGLU 688, vocab 1024.
    "tiny": ModelConfig(
        name="tiny", hidden_size=256, num_attention_heads=4, num_query_groups=2,
        ffn_hidden_size=688, num_layers=2, vocab_size=1024, head_dim=64,
        rope_theta=10000.0, max_seq_len=128,
    ),
    # GPU smoke model with head_dim 128 so the sm_100a attention/GEMM kernels apply.
    "tiny128": ModelConfig(
        name="tiny128", hidden_size=512, num_attention_heads=4, num_query_groups=2,
        ffn_hidden_size=1024, num_layers=2, vocab_size=2048, head_dim=128,
        rope_theta=10000.0, max_seq_len=256,
    ),
}


def get_model_config(name: str) -> ModelConfig:
    if name not in MODEL_REGISTRY:
        raise ValueError(f"Unknown model {name!r}. Available: {sorted(MODEL_REGISTRY)}")
    return MODEL_REGISTRY[name]


# --------------------------------------------------------------------------- parallel layout
@dataclass
class ParallelConfig:
    """Parallel layout and engine switches.

    ``tp_comm``:
      * ``"allreduce"`` – the reference's layout: activations replicated over TP, one all-reduce
        after every row-parallel GEMM (fwd) and every column-parallel dgrad (bwd)
        (``kareus/megatron/core/extensions/ops/te_linear.py:319-329,391-401``).
      * ``"sp"`` – Megatron sequence parallelism: norm/residual on ``s/tp`` rows, all-gather before
        column-parallel GEMMs and reduce-scatter after row-parallel ones, as separate collectives.
      * ``"sp_fused"`` – the same dataflow with the collective fused into the GEMM kernel
        (all-gather→GEMM, GEMM→reduce-scatter over NVLink peer memory).
    ``comm_backend``: ``"nccl"`` (torch.distributed; gloo on CPU) or ``"kernel"`` (our all-pairs
    kernels over the symmetric heap, with the ``sm_num`` knob).
    """

    tp: int = 1
    cp: int = 1
    pp: int = 1
    dp: int = 1
    num_nanobatches: int = 2
    tp_comm: str = "allreduce"
    comm_backend: str = "nccl"
    recompute: bool = True
    nano_split_dim: str = "auto"  # "batch", "seq" or "auto" (batch when mbs >= N)
    cp_comm: str = "all_gather"  # "all_gather" (reference) or "ring"

    def __post_init__(self):
        if self.tp_comm not in ("allreduce", "sp", "sp_fused"):
            raise ValueError(f"bad tp_comm {self.tp_comm!r}")
        if self.comm_backend not in ("nccl", "kernel"):
            raise ValueError(f"bad comm_backend {self.comm_backend!r}")
        if self.num_nanobatches not in (1, 2, 4):
            raise ValueError("num_nanobatches must be 1, 2 or 4")
        if self.cp_comm not in ("all_gather", "ring"):
            raise ValueError(f"bad cp_comm {self.cp_comm!r}")

    @property
    def world_size(self) -> int:
        return self.tp * self.cp * self.pp * self.dp

    @property
    def sequence_parallel(self) -> bool:
        return self.tp_comm in ("sp", "sp_fused") and self.tp > 1


@dataclass
class TrainConfig:
    """Optimizer and batch settings (reference yaml ``tests/artifact/conf/*.yaml:17,180-191``)."""

    micro_batch_size: int = 8
    global_batch_size: int = 64
    seq_len: int = 4096
    lr: float = 2e-4
    min_lr: float = 2e-5
    weight_decay: float = 0.01
    betas: Tuple[float, float] = (0.9, 0.98)
    eps: float = 1e-8
    grad_clip: float = 1.0
    warmup_steps: int = 500
    max_steps: int = 100000
    seed: int = 42
    dtype: str = "bf16"

    def num_microbatches(self, dp: int) -> int:
        per = self.micro_batch_size * dp
        if self.global_batch_size % per:
            raise ValueError("global_batch_size must be divisible by micro_batch_size*dp")
        return self.global_batch_size // per
