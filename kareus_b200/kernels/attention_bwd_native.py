"""Wrapper of the sm_100a flash-attention backward kernel (see ``csrc/attention_bwd_sm100.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import cuda as KC

_DECLARED = False


def _lib():
    global _DECLARED
    L = KC.lib()
    if not _DECLARED:
        P, I, LNG, F = c_void_p, c_int, c_long, c_float
        L.kb_flash_attn_bwd.argtypes = ([P, LNG, LNG, LNG, LNG, P, LNG, LNG, LNG, P, LNG, LNG, LNG, P, P, P,
                                         P, LNG, LNG, LNG, LNG, P, LNG, LNG, LNG, P, LNG, LNG, LNG, P] +
                                        [I] * 6 + [F, I, I, P, P])
        L.kb_flash_attn_bwd.restype = c_int
        L.kb_flash_attn_bwd_scratch_floats.argtypes = [I] * 6
        L.kb_flash_attn_bwd_scratch_floats.restype = c_long
        _DECLARED = True
    return L


def _geom5(t, kg):
    """(s, b, g, rep, d, strides(s, b, g, r)) of a query-like view."""
    if t.dim() == 5:
        s, b, g, rep, d = t.shape
        return s, b, g, rep, d, (t.stride(0), t.stride(1), t.stride(2), t.stride(3))
    s, b, h, d = t.shape
    rep = h // kg
    return s, b, kg, rep, d, (t.stride(0), t.stride(1), t.stride(2) * rep, t.stride(2))


def _ok(t):
    return t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(st % 8 == 0 for st in t.stride()[:-1])


def backward(do, q, k, v, o, lse, scale, causal=True, q_offset=0, kv_len=None, out=None, strict=False):
    kg = k.shape[2]
    sq, b, g, rep, d, qs = _geom5(q, kg)
    from .attention_native import unsupported_reason
    why = unsupported_reason(d, g, kg, q, k, v)
    if why is not None:
        KC.attention_fallback_allowed(why, strict)
        return KC.attention_bwd_library(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out)
    skv = k.shape[0] if kv_len is None else int(kv_len)
    hq = g * rep
    o4, do4 = o.reshape(sq, b, hq, d), do.reshape(sq, b, hq, d)
    if not (o4.is_contiguous() and do4.is_contiguous()):
        KC._no_recording("making attention outputs contiguous")
        o4, do4 = o4.contiguous(), do4.contiguous()
    if out is None:
        dq = torch.empty(sq, b, g, rep, d, dtype=q.dtype, device=q.device)
        dk = torch.empty_like(k, memory_format=torch.contiguous_format)
        dv = torch.empty_like(v, memory_format=torch.contiguous_format)
    else:
        dq, dk, dv = out
    if skv < k.shape[0]:
        KC._no_recording("zero-filling the unseen keys' gradients")
        dk[skv:].zero_()
        dv[skv:].zero_()
    _, _, _, _, _, dqs = _geom5(dq, kg)
    L = _lib()
    work = torch.empty(L.kb_flash_attn_bwd_scratch_floats(sq, skv, b, g, rep, d), dtype=torch.float32, device=q.device)
    st = KC.status_word(q.device)
    rc = L.kb_flash_attn_bwd(q.data_ptr(), *qs, k.data_ptr(), k.stride(0), k.stride(1), k.stride(2),
                             v.data_ptr(), v.stride(0), v.stride(1), v.stride(2), o4.data_ptr(), do4.data_ptr(),
                             lse.data_ptr(), dq.data_ptr(), *dqs, dk.data_ptr(), dk.stride(0), dk.stride(1),
                             dk.stride(2), dv.data_ptr(), dv.stride(0), dv.stride(1), dv.stride(2), work.data_ptr(),
                             sq, skv, b, g, rep, d, float(scale), 1 if causal else 0, int(q_offset), st.data_ptr(),
                             KC._stream())
    KC._check(rc, "flash_attn_bwd")
    KC._count(6)
    if out is not None:
        return out
    return dq.reshape(q.shape), dk, dv


def backward_chunked(do, q, sources, table, chunk_rows, q_positions, o, lse, scale, dq, dkv, dk_row_base, dv_row_base,
                     causal=True):
    """Backward of :func:`attention_native.forward_chunked`.  ``dq`` is a destination view with ``q``'s
    geometry; ``dkv`` is ONE ``[rows, b, g, d]`` destination that receives dK and dV of the whole logical
    key range, logical chunk ``c`` of dK starting at row ``dk_row_base[c]`` and of dV at ``dv_row_base[c]``."""
    from .attention_native import _int_array, _ptr_array, check_chunked
    sq, b, g, rep, d, qs = check_chunked(q, sources, table, chunk_rows, q_positions)
    L = _lib()
    if not getattr(L, "_chunked_bwd_declared", False):
        P, I, LNG, F = c_void_p, c_int, c_long, c_float
        L.kb_flash_attn_bwd_chunked.argtypes = ([P, LNG, LNG, LNG, LNG, P, P, I, I, LNG, LNG, LNG, LNG, LNG, LNG, P, P,
                                                 I, I, I, P, P, P, P, P, LNG, LNG, LNG, LNG, P, LNG, LNG, LNG, P, P, P] +
                                                [I] * 5 + [F, I, P, P])
        L.kb_flash_attn_bwd_chunked.restype = c_int
        L._chunked_bwd_declared = True
    if not (_ok(dkv) and dkv.dim() == 4 and dkv.dtype == torch.bfloat16):
        raise KC.KernelError("dkv must be a bf16 [rows, b, g, d] view with 16-byte aligned strides")
    hq = g * rep
    o4, do4 = o.reshape(sq, b, hq, d), do.reshape(sq, b, hq, d)
    if not (o4.is_contiguous() and do4.is_contiguous()):
        KC._no_recording("making attention outputs contiguous")
        o4, do4 = o4.contiguous(), do4.contiguous()
    k0, v0 = sources[0]
    skv = len(table) * int(chunk_rows)
    _, _, _, _, _, dqs = _geom5(dq, k0.shape[2])
    work = torch.empty(L.kb_flash_attn_bwd_scratch_floats(sq, skv, b, g, rep, d), dtype=torch.float32, device=q.device)
    st = KC.status_word(q.device)
    rc = L.kb_flash_attn_bwd_chunked(
        q.data_ptr(), *qs, _ptr_array([k for k, _ in sources]), _ptr_array([v for _, v in sources]), len(sources),
        k0.shape[0], k0.stride(0), k0.stride(1), k0.stride(2), v0.stride(0), v0.stride(1), v0.stride(2),
        _int_array([t[0] for t in table]), _int_array([t[1] for t in table]), len(table), int(chunk_rows),
        sq // len(q_positions), _int_array(q_positions), o4.data_ptr(), do4.data_ptr(), lse.data_ptr(),
        dq.data_ptr(), *dqs, dkv.data_ptr(), dkv.stride(0), dkv.stride(1), dkv.stride(2), _int_array(dk_row_base),
        _int_array(dv_row_base), work.data_ptr(), sq, b, g, rep, d, float(scale), 1 if causal else 0, st.data_ptr(),
        KC._stream())
    KC._check(rc, "flash_attn_bwd_chunked")
    KC._count(6)
    return dq, dkv
