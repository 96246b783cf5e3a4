"""Search space of one partition: (SM clock, CTAs given to the collective, launch slot[, nanobatches]).

Reference encoding: ``tests/bayesian/common/encoding.py:10-76`` (numeric clock and SM indices,
one-hot launch slot, block size fixed at 1024) and the per-partition spaces in
``tests/bayesian/partitions/*/bo_search.py``.  The optional fourth axis is this framework's
nanobatch split count {1, 2, 4}.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np

BLOCK_SIZE = 1024


@dataclass(frozen=True)
class Config:
    freq: int
    sm: int
    overlap: Tuple[str, str]
    block: int = BLOCK_SIZE
    nano: int = 2

    def key(self) -> tuple:
        return (self.freq, self.sm, self.overlap[0], self.overlap[1], self.block, self.nano)

    def cfg_string(self) -> str:
        return f"{self.overlap[0]}-{self.overlap[1]}-{self.sm}-{self.block}"


@dataclass
class SearchSpace:
    overlap_windows: List[Tuple[str, str]]
    sm_values: List[int]
    n_init: int = 96
    batches: int = 4
    acq_batch: int = 32
    real_fraction: float = 0.4
    dynamic_fraction: float = 0.2
    time_fraction: float = 0.2
    nano_values: List[int] = field(default_factory=lambda: [2])

    def grid(self, freqs: Sequence[int]) -> List[Config]:
        return [Config(f, sm, ow, BLOCK_SIZE, n) for f, sm, ow, n in
                itertools.product(freqs, self.sm_values, self.overlap_windows, self.nano_values)]

    def encode(self, configs: Sequence[Config], freqs: Sequence[int]) -> np.ndarray:
        """``[freq_idx, sm_idx, nano_idx, onehot(overlap)...]`` per config."""
        fi = {f: i for i, f in enumerate(freqs)}
        si = {s: i for i, s in enumerate(self.sm_values)}
        ni = {n: i for i, n in enumerate(self.nano_values)}
        oi = {tuple(o): i for i, o in enumerate(self.overlap_windows)}
        X = np.zeros((len(configs), 3 + len(self.overlap_windows)), dtype=float)
        for r, c in enumerate(configs):
            X[r, 0], X[r, 1], X[r, 2] = fi[c.freq], si[c.sm], ni[c.nano]
            X[r, 3 + oi[tuple(c.overlap)]] = 1.0
        return X


# The 14 partition kinds: 4 tensor-parallel ones and 10 that exist with context parallelism.
# ``comm`` names the collective carried by the partition; AR partitions sweep 3..30 CTAs, AG/RS
# partitions 1..20 (reference ``tests/bayesian/partitions/*/bo_search.py:18-37``).
_AR_SM = list(range(3, 31, 3))
_AG_SM = list(range(1, 21))
N = ("none",)


def _ow(*slots):
    return [(s, "none") for s in slots]


PARTITION_SPACES: Dict[str, Tuple[str, SearchSpace]] = {
    "fwd_attn": ("all_reduce", SearchSpace(_ow("norm_0", "linear_0", "rope_0", "attn_0"), _AR_SM)),
    "fwd_mlp": ("all_reduce", SearchSpace(_ow("norm_0", "linear_0", "activation_0"), _AR_SM)),
    "bwd_attn": ("all_reduce", SearchSpace(_ow("norm_0", "linear_0", "attn_0", "rope_0"), _AR_SM)),
    "bwd_mlp": ("all_reduce", SearchSpace(_ow("norm_0", "linear_0", "activation_0"), _AR_SM)),
    "fwd_qkv_ar": ("all_reduce", SearchSpace(_ow("norm_0", "linear_0"), _AR_SM, 48, 4, 16)),
    "fwd_qkv_ag": ("all_gather_kv", SearchSpace(_ow("norm_0", "linear_0", "rope_0"), _AG_SM, 48, 4, 16)),
    "fwd_ao_ag": ("all_gather_kv", SearchSpace(_ow("attn_0", "linear_0"), _AG_SM, 36, 3, 16)),
    "fwd_ao_ar": ("all_reduce", SearchSpace(_ow("attn_0"), _AR_SM, 36, 3, 16)),
    "bwd_qkv_ar": ("all_reduce", SearchSpace(_ow("rope_0", "linear_0"), _AR_SM, 48, 4, 16)),
    "bwd_qkv_rs": ("reduce_scatter_kv", SearchSpace(_ow("rope_0", "linear_0"), _AG_SM, 48, 4, 16)),
    "bwd_a_rs": ("reduce_scatter_kv", SearchSpace(_ow("attn_0"), _AG_SM, 36, 3, 16)),
    "bwd_a_ag": ("all_gather_kv", SearchSpace(_ow("attn_0"), _AG_SM, 36, 3, 16)),
    "bwd_o_ag": ("all_gather_kv", SearchSpace(_ow("norm_0", "linear_0"), _AG_SM, 36, 3, 16)),
    "bwd_o_ar": ("all_reduce", SearchSpace(_ow("norm_0"), _AR_SM, 36, 3, 16)),
}
# Partitions of the fused sequence-parallel path (``tp_comm="sp_fused"``): eight per layer, each the
# compute of one segment beside the fused GEMM+collective kernel of the other nanobatch.  ``sm``
# is the fused kernel's knob: copy-driver CTAs for all-gather→GEMM kernels, SMs the kernel leaves to
# the other nanobatch's compute for GEMM→reduce-scatter kernels (``csrc/fused_gemm_comm.cu``).  The
# reference has no such partitions (its TP collectives are all-reduces: ``tests/bayesian/partitions``).
# Both kinds sweep the same values: a plan file names ONE config per reference key (fwd_attn, ...), the
# "_ag" segment of that key inherits its sm, so the composer pairs the two partitions' points by sm.
_FUSED_AG_SM = [4, 8, 12, 16, 24, 32]
_FUSED_RS_SM = [4, 8, 12, 16, 24, 32]
SP_FUSED_SPACES: Dict[str, Tuple[str, SearchSpace]] = {
    "fwd_attn_ag": ("fused_ag_gemm", SearchSpace(_ow("norm_0"), _FUSED_AG_SM, 12, 2, 6)),
    "fwd_attn": ("fused_gemm_rs", SearchSpace(_ow("rope_0", "attn_0"), _FUSED_RS_SM, 16, 2, 8)),
    "fwd_mlp_ag": ("fused_ag_gemm", SearchSpace(_ow("norm_0"), _FUSED_AG_SM, 12, 2, 6)),
    "fwd_mlp": ("fused_gemm_rs", SearchSpace(_ow("activation_0"), _FUSED_RS_SM, 12, 2, 6)),
    "bwd_mlp_ag": ("fused_ag_dgrad", SearchSpace(_ow("norm_0"), _FUSED_AG_SM, 12, 2, 6)),
    "bwd_mlp": ("fused_dgrad_rs", SearchSpace(_ow("activation_0"), _FUSED_RS_SM, 12, 2, 6)),
    "bwd_attn_ag": ("fused_ag_dgrad", SearchSpace(_ow("norm_0"), _FUSED_AG_SM, 12, 2, 6)),
    "bwd_attn": ("fused_dgrad_rs", SearchSpace(_ow("attn_0", "rope_0"), _FUSED_RS_SM, 16, 2, 8)),
}
SP_FUSED_PARTITIONS = tuple(SP_FUSED_SPACES)


def partition_space(key: str, tp_comm: str = "allreduce") -> Tuple[str, SearchSpace]:
    """``(collective kind, search space)`` of a partition key for a tensor-parallel flavour."""
    if tp_comm in ("sp", "sp_fused") and key in SP_FUSED_SPACES:
        return SP_FUSED_SPACES[key]
    if key not in PARTITION_SPACES:
        raise KeyError(f"unknown partition {key!r}; known: {sorted(PARTITION_SPACES) + sorted(SP_FUSED_SPACES)}")
    return PARTITION_SPACES[key]


TP_PARTITIONS = ("fwd_attn", "fwd_mlp", "bwd_attn", "bwd_mlp")
CP_PARTITIONS = tuple(k for k in PARTITION_SPACES if k not in TP_PARTITIONS or k in ("fwd_mlp", "bwd_mlp"))
