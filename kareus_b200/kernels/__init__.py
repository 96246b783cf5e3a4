"""Kernel entry points used by the operators.

Every function takes torch tensors.  CUDA tensors go to the hand-written sm_100a kernels in
``libkareus_b200.so`` (built from ``kernels/csrc`` and loaded through :mod:`.cuda`); CPU tensors
go to the PyTorch statements in :mod:`.ref`.  There is no silent fallback on a GPU: if the
library is missing the call raises, and bf16 attention shapes the hand-written kernels do not
cover (head dim other than 128, rows that are not 16-byte aligned) raise too unless
``KAREUS_B200_ATTENTION_FALLBACK=1`` opts into the flash-attention wheel, which is logged once.
``KAREUS_B200_LIBRARY_BASELINE=1`` switches GEMM and attention to the vendor libraries (cuBLAS
through ``torch.matmul``, the flash-attention wheel); that is the A/B baseline configured like the
reference, never the default.

Operands that live in another GPU's memory (peer views of the symmetric heap) must be announced
with ``peer=True``; such calls run this package's own kernels or raise, whatever the switches say:
a vendor-library kernel never receives a peer's memory.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import ref

_LAUNCHES = [0]


def launch_count() -> int:
    """Number of kernels of this package launched so far in this process."""
    return _LAUNCHES[0]


def _count(n: int = 1) -> None:
    _LAUNCHES[0] += n


def library_baseline() -> bool:
    return os.environ.get("KAREUS_B200_LIBRARY_BASELINE", "0") == "1"


def _cuda():
    from . import cuda
    return cuda


def is_cuda(t) -> bool:
    return isinstance(t, torch.Tensor) and t.is_cuda


# ----------------------------------------------------------------------------- norm
def rmsnorm_fwd(x, w, eps):
    if is_cuda(x):
        return _cuda().rmsnorm_fwd(x, w, eps)
    return ref.rmsnorm_fwd(x, w, eps)


def rmsnorm_bwd(dy, x, rstd, w, dw_accum=None):
    """``(dx, dw)``; with ``dw_accum`` the weight gradient is added into that buffer and ``dw`` is None."""
    if is_cuda(x):
        return _cuda().rmsnorm_bwd(dy, x, rstd, w, dw_accum)
    dx, dw = ref.rmsnorm_bwd(dy, x, rstd, w)
    if dw_accum is not None:
        dw_accum.add_(dw.reshape(dw_accum.shape).to(dw_accum.dtype))
        dw = None
    return dx, dw


# ----------------------------------------------------------------------------- rope
def rope_inplace(q, k, freqs, inverse=False):
    """Rotate ``q`` and ``k`` (views are fine) in place."""
    if is_cuda(q):
        return _cuda().rope_inplace(q, k, freqs, inverse)
    q.copy_(ref.rope_apply(q, freqs, inverse))
    if k is not None:
        k.copy_(ref.rope_apply(k, freqs, inverse))


# ----------------------------------------------------------------------------- swiglu
def swiglu_fwd(x):
    if is_cuda(x):
        return _cuda().swiglu_fwd(x)
    return ref.swiglu_fwd(x)


def swiglu_bwd(dy, x):
    if is_cuda(x):
        return _cuda().swiglu_bwd(dy, x)
    return ref.swiglu_bwd(dy, x)


# ----------------------------------------------------------------------------- dropout-add
def dropout_add_fwd(x, residual, p, seed):
    if is_cuda(x):
        return _cuda().dropout_add_fwd(x, residual, p, seed)
    return ref.dropout_add_fwd(x, residual, p, seed)


def dropout_add_bwd(dy, p, seed):
    if is_cuda(dy):
        return _cuda().dropout_add_bwd(dy, p, seed)
    return ref.dropout_add_bwd(dy, p, seed)


def add(a, b):
    if is_cuda(a):
        return _cuda().add(a, b)
    return a + b


# ----------------------------------------------------------------------------- GEMM
def gemm(a, b, trans_a=False, trans_b=True, out_dtype=None, accumulate=None, out=None, bias=None, activation=None):
    """``op(a) @ op(b)``.  ``accumulate`` is an fp32 tensor that receives ``+=``.  ``bias`` (per output
    feature) and ``activation`` (``"gelu"``) run in the GEMM's epilogue."""
    if is_cuda(a):
        if library_baseline():
            return _cuda().gemm_library(a, b, trans_a, trans_b, out_dtype, accumulate, out, bias, activation)
        return _cuda().gemm(a, b, trans_a, trans_b, out_dtype, accumulate, out, bias=bias, activation=activation)
    r = ref.gemm(a, b, trans_a, trans_b, out_dtype, accumulate)
    if bias is not None or activation:
        r = ref.bias_act(r, bias, activation)
    if out is not None:
        out.copy_(r)
        return out
    return r


# ----------------------------------------------------------------------------- attention
def _peer_guard(q, what: str) -> None:
    """A call that announces peer-memory operands may only reach this package's own kernels."""
    from .cuda import KernelError
    if not is_cuda(q):
        raise KernelError(f"{what}: peer-memory operands need CUDA tensors")
    if library_baseline():
        raise KernelError(f"{what}: KAREUS_B200_LIBRARY_BASELINE=1 would hand another GPU's memory to a "
                          "vendor-library kernel; refused")


def attention_fwd(q, k, v, scale, causal=True, q_offset=0, kv_len=None, peer=False):
    """``peer=True``: ``k``/``v`` may be views of another GPU's memory; only the native kernel may run."""
    if peer:
        _peer_guard(q, "attention_fwd")
        return _cuda().attention_fwd(q, k, v, scale, causal, q_offset, kv_len, strict=True)
    if is_cuda(q):
        if library_baseline():
            return _cuda().attention_fwd_library(q, k, v, scale, causal, q_offset, kv_len)
        return _cuda().attention_fwd(q, k, v, scale, causal, q_offset, kv_len)
    return ref.attention_fwd(q, k, v, scale, causal, q_offset, kv_len)


def attention_bwd(do, q, k, v, o, lse, scale, causal=True, q_offset=0, kv_len=None, out=None, peer=False):
    """Returns ``(dq, dk, dv)``; ``out`` may provide preallocated (strided) destinations.
    ``peer=True`` as in :func:`attention_fwd`."""
    if peer:
        _peer_guard(q, "attention_bwd")
        return _cuda().attention_bwd(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out, strict=True)
    if is_cuda(q):
        if library_baseline():
            return _cuda().attention_bwd_library(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out)
        return _cuda().attention_bwd(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out)
    dq, dk, dv = ref.attention_bwd(do, q, k, v, o, lse, scale, causal, q_offset, kv_len)
    if out is not None:
        out[0].copy_(dq.reshape(out[0].shape))
        out[1].copy_(dk)
        out[2].copy_(dv)
        return out
    return dq, dk, dv


def attention_fwd_chunked(q, sources, table, chunk_rows, q_positions, scale, causal=True, peer=False):
    """Attention over K/V stored as chunks in several buffers (``ref.attention_fwd_chunked`` states the
    math).  On GPUs this is ONE launch of the native kernel, which fetches each chunk's tiles from its
    buffer; with ``peer=True`` the buffers may be other GPUs' memory.  No library route exists."""
    if is_cuda(q):
        if library_baseline() or peer:
            _peer_guard(q, "attention_fwd_chunked")
        from . import attention_native
        return attention_native.forward_chunked(q, sources, table, chunk_rows, q_positions, scale, causal)
    if peer:
        _peer_guard(q, "attention_fwd_chunked")
    return ref.attention_fwd_chunked(q, sources, table, chunk_rows, q_positions, scale, causal)


def attention_bwd_chunked(do, q, sources, table, chunk_rows, q_positions, o, lse, scale, dq, dkv, dk_row_base,
                          dv_row_base, causal=True, peer=False):
    """Backward of :func:`attention_fwd_chunked`.  dQ goes to the view ``dq``; dK and dV of the logical key
    range go to the rows of ``dkv`` named by ``dk_row_base`` / ``dv_row_base`` (one entry per logical chunk)."""
    if is_cuda(q):
        if library_baseline() or peer:
            _peer_guard(q, "attention_bwd_chunked")
        from . import attention_bwd_native
        return attention_bwd_native.backward_chunked(do, q, sources, table, chunk_rows, q_positions, o, lse, scale,
                                                     dq, dkv, dk_row_base, dv_row_base, causal)
    if peer:
        _peer_guard(q, "attention_bwd_chunked")
    g_q, g_k, g_v = ref.attention_bwd_chunked(do, q, sources, table, chunk_rows, q_positions, o, lse, scale, causal)
    dq.copy_(g_q.reshape(dq.shape))
    for c, (bk, bv) in enumerate(zip(dk_row_base, dv_row_base)):
        dkv[bk:bk + chunk_rows].copy_(g_k[c * chunk_rows:(c + 1) * chunk_rows])
        dkv[bv:bv + chunk_rows].copy_(g_v[c * chunk_rows:(c + 1) * chunk_rows])
    return dq, dkv


# ----------------------------------------------------------------------------- cross entropy
def cross_entropy_local_stats(logits, targets, vocab_start):
    if is_cuda(logits):
        return _cuda().cross_entropy_local_stats(logits, targets, vocab_start)
    return ref.cross_entropy_local_stats(logits, targets, vocab_start)


def cross_entropy_finish(logits, targets, vocab_start, gmax, gsum, grad_scale):
    if is_cuda(logits):
        return _cuda().cross_entropy_finish(logits, targets, vocab_start, gmax, gsum, grad_scale)
    return ref.cross_entropy_finish(logits, targets, vocab_start, gmax, gsum, grad_scale)


# ----------------------------------------------------------------------------- embedding
def embedding_fwd(tokens, weight, vocab_start):
    if is_cuda(weight):
        return _cuda().embedding_fwd(tokens, weight, vocab_start)
    return ref.embedding_fwd(tokens, weight, vocab_start)


def embedding_bwd(dout, tokens, grad_weight, vocab_start):
    if is_cuda(dout):
        return _cuda().embedding_bwd(dout, tokens, grad_weight, vocab_start)
    return ref.embedding_bwd(dout, tokens, grad_weight, vocab_start)


# ----------------------------------------------------------------------------- optimizer
def adamw_step(p, g, m, v, master, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    if is_cuda(master):
        return _cuda().adamw_step(p, g, m, v, master, lr, beta1, beta2, eps, wd, step, grad_scale)
    return ref.adamw_step(p, g, m, v, master, lr, beta1, beta2, eps, wd, step, grad_scale)


def sumsq(t):
    if is_cuda(t):
        return _cuda().sumsq(t)
    return ref.sumsq(t)
