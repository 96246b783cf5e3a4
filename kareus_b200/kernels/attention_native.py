"""Wrappers of the hand-written sm_100a flash-attention kernels.

Inputs may be strided views: ``q`` is ``[sq, b, h, d]`` or ``[sq, b, g, rep, d]``, ``k``/``v`` are
``[skv, b, g, d]``, all with a contiguous head dimension of 128 and 16-byte aligned strides (views
of the packed QKV projection qualify).  ``q_offset`` is the absolute position of query row 0
relative to key 0 and ``kv_len`` limits the visible keys; together they express the causal masks of
context-parallel chunks.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import cuda as KC

_DECLARED = False


def _lib():
    global _DECLARED
    L = KC.lib()
    if not _DECLARED:
        P, I, LNG, F = c_void_p, c_int, c_long, c_float
        L.kb_flash_attn_fwd.argtypes = [P, LNG, LNG, LNG, LNG, P, LNG, LNG, LNG, P, LNG, LNG, LNG, P, P,
                                        I, I, I, I, I, I, F, I, I, P, P]
        L.kb_flash_attn_fwd.restype = c_int
        if hasattr(L, "kb_flash_attn_bwd"):
            L.kb_flash_attn_bwd.restype = c_int
        _DECLARED = True
    return L


def _q_geometry(q):
    if q.dim() == 5:
        s, b, g, rep, d = q.shape
        return s, b, g, rep, d, (q.stride(0), q.stride(1), q.stride(2), q.stride(3))
    s, b, h, d = q.shape
    return s, b, 1, h, d, (q.stride(0), q.stride(1), 0, q.stride(2))


def _usable(t) -> bool:
    return t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(st % 8 == 0 for st in t.stride()[:-1])


def unsupported_reason(d, g, kg, *tensors):
    """Why the native kernels cannot take a call, or ``None``."""
    if d != 128:
        return f"head dim {d} (the kernels are specialised for 128)"
    if g != kg:
        return f"query groups {g} do not match key groups {kg}"
    if not all(_usable(t) for t in tensors):
        return "an operand's head dim is not contiguous or a stride/base is not 16-byte aligned"
    return None


def forward(q, k, v, scale, causal=True, q_offset=0, kv_len=None, strict=False):
    sq, b, g, rep, d, qs = _q_geometry(q)
    kg = k.shape[2]
    if q.dim() == 4:
        # [s,b,h,d] with h = kg*rep heads laid out group-major: reinterpret as (g, rep)
        rep = q.shape[2] // kg
        g = kg
        qs = (q.stride(0), q.stride(1), q.stride(2) * rep, q.stride(2))
    why = unsupported_reason(d, g, kg, q, k, v)
    if why is not None:
        KC.attention_fallback_allowed(why, strict)
        return KC.attention_fwd_library(q, k, v, scale, causal, q_offset, kv_len)
    skv = k.shape[0] if kv_len is None else int(kv_len)
    out = torch.empty(sq, b, g * rep, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, g * rep, sq, dtype=torch.float32, device=q.device)
    st = KC.status_word(q.device)
    rc = _lib().kb_flash_attn_fwd(q.data_ptr(), *qs, k.data_ptr(), k.stride(0), k.stride(1), k.stride(2),
                                  v.data_ptr(), v.stride(0), v.stride(1), v.stride(2), out.data_ptr(),
                                  lse.data_ptr(), sq, skv, b, g, rep, d, float(scale), 1 if causal else 0,
                                  int(q_offset), st.data_ptr(), KC._stream())
    KC._check(rc, "flash_attn_fwd")
    KC._count()
    return out, lse


def _ptr_array(tensors):
    return (c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _int_array(values):
    return (c_int * len(values))(*[int(v) for v in values])


def check_chunked(q, sources, table, chunk_rows, q_positions):
    """Validate a chunked call (see ``ref.attention_fwd_chunked``); raises :class:`KernelError`.  These
    calls may read other GPUs' memory, so there is no fallback of any kind."""
    k0, v0 = sources[0]
    kg = k0.shape[2]
    sq, b, g, rep, d, qs = _q_geometry(q)
    if q.dim() == 4:
        rep, g = q.shape[2] // kg, kg
        qs = (q.stride(0), q.stride(1), q.stride(2) * rep, q.stride(2))
    why = unsupported_reason(d, g, kg, q, *[t for kv in sources for t in kv])
    if why is None and q.dtype != torch.bfloat16:
        why = f"dtype {q.dtype}"
    if why is None and any(tuple(k.stride()) != tuple(k0.stride()) or tuple(v.stride()) != tuple(v0.stride())
                           or k.shape != k0.shape for k, v in sources):
        why = "K/V sources differ in shape or strides"
    if why is None and (chunk_rows % 128 or sq % len(q_positions) or (sq // len(q_positions)) % 128):
        why = "chunks must be multiples of 128 rows"
    if why is not None:
        raise KC.KernelError(f"chunked attention cannot run ({why}); its operands may be peer memory, so no "
                             "library or PyTorch route exists")
    return sq, b, g, rep, d, qs


def forward_chunked(q, sources, table, chunk_rows, q_positions, scale, causal=True):
    """One launch over K/V chunks that live in several buffers (other GPUs' heaps through their peer
    mappings).  Returns ``(out [sq,b,h,d], lse [b,h,sq])``."""
    sq, b, g, rep, d, qs = check_chunked(q, sources, table, chunk_rows, q_positions)
    L = _lib()
    if not getattr(L, "_chunked_declared", False):
        P, I, LNG, F = c_void_p, c_int, c_long, c_float
        L.kb_flash_attn_fwd_chunked.argtypes = [P, LNG, LNG, LNG, LNG, P, P, I, I, LNG, LNG, LNG, LNG, LNG, LNG, P, P, I,
                                                I, I, P, P, P, I, I, I, I, I, F, I, P, P]
        L.kb_flash_attn_fwd_chunked.restype = c_int
        L._chunked_declared = True
    k0, v0 = sources[0]
    out = torch.empty(sq, b, g * rep, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, g * rep, sq, dtype=torch.float32, device=q.device)
    st = KC.status_word(q.device)
    rc = L.kb_flash_attn_fwd_chunked(
        q.data_ptr(), *qs, _ptr_array([k for k, _ in sources]), _ptr_array([v for _, v in sources]), len(sources),
        k0.shape[0], k0.stride(0), k0.stride(1), k0.stride(2), v0.stride(0), v0.stride(1), v0.stride(2),
        _int_array([t[0] for t in table]), _int_array([t[1] for t in table]), len(table), int(chunk_rows),
        sq // len(q_positions), _int_array(q_positions), out.data_ptr(), lse.data_ptr(), sq, b, g, rep, d,
        float(scale), 1 if causal else 0, st.data_ptr(), KC._stream())
    KC._check(rc, "flash_attn_fwd_chunked")
    KC._count()
    return out, lse


def backward(do, q, k, v, o, lse, scale, causal=True, q_offset=0, kv_len=None, out=None, strict=False):
    from . import attention_bwd_native
    return attention_bwd_native.backward(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out, strict=strict)
