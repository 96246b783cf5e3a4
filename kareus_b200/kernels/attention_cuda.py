"""Flash-attention entry points for bf16 CUDA tensors (hand-written sm_100a kernels).

``strict=True`` marks calls whose K/V may be views of another GPU's memory: they run the native
kernels or raise.  Other calls leave the native kernels only through
:func:`kareus_b200.kernels.cuda.attention_fallback_allowed` (an explicit opt-in, logged once).
"""
from __future__ import annotations

import torch

from . import cuda as KC


def have_native() -> bool:
    return hasattr(KC.lib(), "kb_flash_attn_fwd")


def forward(q, k, v, scale, causal=True, q_offset=0, kv_len=None, strict=False):
    if have_native():
        from . import attention_native
        return attention_native.forward(q, k, v, scale, causal, q_offset, kv_len, strict=strict)
    KC.attention_fallback_allowed("the library was built without the attention forward kernel", strict)
    return KC.attention_fwd_library(q, k, v, scale, causal, q_offset, kv_len)


def backward(do, q, k, v, o, lse, scale, causal=True, q_offset=0, kv_len=None, out=None, strict=False):
    if have_native() and hasattr(KC.lib(), "kb_flash_attn_bwd"):
        from . import attention_native
        return attention_native.backward(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out, strict=strict)
    KC.attention_fallback_allowed("the library was built without the attention backward kernel", strict)
    return KC.attention_bwd_library(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out)
