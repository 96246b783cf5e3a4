"""ctypes bindings of ``libkareus_b200.so`` (the sm_100a kernels) for torch CUDA tensors.

The library has a plain C ABI: pointers, sizes, strides and a ``cudaStream_t``.  Outputs are
allocated here with torch (caching allocator) and kernels are enqueued on torch's current
stream, so they compose with the engine's stream/event protocol.  Loading fails loudly when the
library is missing: there is no PyTorch fallback for bf16 CUDA tensors.  fp32/fp64 CUDA tensors
(numerics debugging) use the PyTorch statements of :mod:`.ref`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_uint, c_void_p
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch

from . import ref

_LIB: Optional[ctypes.CDLL] = None
_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libkareus_b200.so"

STATUS_NAMES = {0: "ok", 1: "timeout waiting for a TMA stage", 2: "timeout waiting for a free stage",
                3: "timeout waiting for an accumulator", 4: "timeout waiting for a free accumulator",
                5: "timeout waiting for a peer GPU", 6: "grid barrier timeout", 7: "bad argument"}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise KernelError(
                f"{LIB_PATH} is missing: build it with `python -m kareus_b200.kernels.build` "
                "(bf16 CUDA tensors have no PyTorch fallback)")
        _LIB = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        _declare(_LIB)
    return _LIB


def is_loaded() -> bool:
    return _LIB is not None


def _declare(L) -> None:
    P, I, LNG, F, U = c_void_p, c_int, c_long, c_float, c_uint
    sig = {
        "kb_gemm_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P],
        "kb_gemm_bias_act_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, I, P, P],
        "kb_rmsnorm_fwd": [P, P, P, P, I, I, F, P],
        "kb_rmsnorm_bwd": [P, P, P, P, P, P, P, I, I, P],
        "kb_rmsnorm_bwd_acc": [P, P, P, P, P, P, P, I, I, I, P],
        "kb_rope": [P, LNG, LNG, LNG, LNG, I, I, P, LNG, LNG, LNG, I, P, P, I, I, I, I, P],
        "kb_swiglu_fwd": [P, P, LNG, I, P],
        "kb_swiglu_bwd": [P, P, P, LNG, I, P],
        "kb_dropout_add_fwd": [P, P, P, LNG, F, U, P],
        "kb_dropout_bwd": [P, P, LNG, F, U, P],
        "kb_add": [P, P, P, LNG, P],
        "kb_embedding_fwd": [P, P, P, LNG, I, LNG, LNG, P],
        "kb_embedding_bwd": [P, P, P, LNG, I, LNG, LNG, P],
        "kb_ce_stats": [P, P, P, P, P, LNG, I, LNG, P],
        "kb_ce_grad": [P, P, P, P, P, LNG, I, LNG, P],
        "kb_adamw": [P, P, P, P, P, LNG, F, F, F, F, F, F, F, P, F, P],
        "kb_sumsq": [P, LNG, I, P, P],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = c_int
    L.kb_rmsnorm_bwd_scratch_elems.argtypes = [I, I]
    L.kb_rmsnorm_bwd_scratch_elems.restype = c_long
    for name, args in _OPTIONAL_SIGS.items():
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int


_OPTIONAL_SIGS: Dict[str, list] = {}


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Raw handle of torch's current stream on the current device."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc} ({STATUS_NAMES.get(rc, 'CUDA/driver error')})")


_LAUNCH_COUNTER = None


def _count(n: int = 1) -> None:
    global _LAUNCH_COUNTER
    if _LAUNCH_COUNTER is None:
        from . import _LAUNCHES
        _LAUNCH_COUNTER = _LAUNCHES
    _LAUNCH_COUNTER[0] += n


def _bf16(t: torch.Tensor) -> bool:
    return t.dtype == torch.bfloat16


def _no_recording(what: str) -> None:
    """Guard of wrapper paths that launch PyTorch kernels (invisible to a launch-list recording)."""
    from . import replay
    replay.require_recordable(what)


# per-device status word that kernels with bounded waits write to
_STATUS: Dict[int, torch.Tensor] = {}


def status_word(device) -> torch.Tensor:
    idx = device.index if isinstance(device, torch.device) else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _STATUS[idx] = t
    return t


def check_status(device=None, reset: bool = True) -> None:
    """Synchronising read of the status word; raises if a kernel recorded a bounded-wait expiry."""
    dev = device if device is not None else torch.cuda.current_device()
    w = status_word(dev)
    code = int(w.item())
    if code != 0:
        if reset:
            w.zero_()
        raise KernelError(f"a kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown')}")


def sm_count(device=None) -> int:
    return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count


# ----------------------------------------------------------------------------- norm
def rmsnorm_fwd(x, w, eps):
    if not _bf16(x):
        return ref.rmsnorm_fwd(x, w, eps)
    if not x.is_contiguous():
        _no_recording("making a norm input contiguous")
        x = x.contiguous()
    rows, H = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    wb = w if _bf16(w) else w.to(torch.bfloat16)
    _check(lib().kb_rmsnorm_fwd(x.data_ptr(), wb.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, H, float(eps),
                                _stream()), "rmsnorm_fwd")
    _count()
    return y, rstd


def rmsnorm_bwd(dy, x, rstd, w, dw_accum=None):
    """Returns ``(dx, dw)``.  With ``dw_accum`` (contiguous fp32 ``[H]``, the weight's main gradient) the
    weight gradient is added there by the kernel and ``dw`` is ``None``."""
    if not _bf16(x):
        dx, dw = ref.rmsnorm_bwd(dy, x, rstd, w)
        if dw_accum is not None:
            dw_accum.add_(dw.to(dw_accum.dtype))
            dw = None
        return dx, dw
    if not dy.is_contiguous():
        _no_recording("making a gradient contiguous")
        dy = dy.contiguous()
    rows, H = x.shape
    dx = torch.empty_like(x)
    acc = dw_accum is not None and dw_accum.dtype == torch.float32 and dw_accum.is_contiguous()
    dw = dw_accum if acc else torch.empty(H, dtype=torch.float32, device=x.device)
    L = lib()
    n = L.kb_rmsnorm_bwd_scratch_elems(rows, H)
    scratch = torch.empty(max(n, 1), dtype=torch.float32, device=x.device)
    wb = w if _bf16(w) else w.to(torch.bfloat16)
    _check(L.kb_rmsnorm_bwd_acc(dy.data_ptr(), x.data_ptr(), rstd.data_ptr(), wb.data_ptr(), dx.data_ptr(),
                                dw.data_ptr(), scratch.data_ptr(), rows, H, 1 if acc else 0, _stream()), "rmsnorm_bwd")
    _count(2)
    if acc:
        return dx, None
    if dw_accum is not None:
        dw_accum.add_(dw.to(dw_accum.dtype))
        return dx, None
    return dx, dw


# ----------------------------------------------------------------------------- rope
_ROPE_TABLES: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def _rope_tables(freqs: torch.Tensor):
    key = (freqs.data_ptr(), freqs.shape[0])
    hit = _ROPE_TABLES.get(key)
    if hit is not None and hit[0] is freqs:
        return hit[1], hit[2]
    half = freqs.shape[-1] // 2
    f = freqs[:, :half].to(torch.float64)
    cos, sin = f.cos().float().contiguous(), f.sin().float().contiguous()
    _ROPE_TABLES[key] = (freqs, cos, sin)
    return cos, sin


def rope_inplace(q, k, freqs, inverse=False):
    if not _bf16(q):
        q.copy_(ref.rope_apply(q, freqs, inverse))
        if k is not None:
            k.copy_(ref.rope_apply(k, freqs, inverse))
        return
    cos, sin = _rope_tables(freqs)
    if q.dim() == 4:
        S, B, Hq, D = q.shape
        G, R = 1, Hq
        qs = (q.stride(0), q.stride(1), 0, q.stride(2))
    else:
        S, B, G, R, D = q.shape
        qs = (q.stride(0), q.stride(1), q.stride(2), q.stride(3))
    if q.stride(-1) != 1 or (k is not None and k.stride(-1) != 1):
        raise KernelError("rope needs a contiguous head dimension")
    if k is not None:
        KG = k.shape[2]
        ks = (k.stride(0), k.stride(1), k.stride(2))
        kp = k.data_ptr()
    else:
        KG, ks, kp = 0, (0, 0, 0), 0
    _check(lib().kb_rope(q.data_ptr(), *qs, G, R, kp, *ks, KG, cos.data_ptr(), sin.data_ptr(), S, B, D,
                         1 if inverse else 0, _stream()), "rope")
    _count()


# ----------------------------------------------------------------------------- swiglu / dropout / add
def swiglu_fwd(x):
    if not _bf16(x):
        return ref.swiglu_fwd(x)
    if not x.is_contiguous():
        _no_recording("making a SwiGLU input contiguous")
        x = x.contiguous()
    rows, F2 = x.shape
    y = torch.empty(rows, F2 // 2, dtype=x.dtype, device=x.device)
    _check(lib().kb_swiglu_fwd(x.data_ptr(), y.data_ptr(), rows, F2 // 2, _stream()), "swiglu_fwd")
    _count()
    return y


def swiglu_bwd(dy, x):
    if not _bf16(x):
        return ref.swiglu_bwd(dy, x)
    if not dy.is_contiguous():
        _no_recording("making a SwiGLU gradient contiguous")
        dy = dy.contiguous()
    rows, F2 = x.shape
    dx = torch.empty_like(x)
    _check(lib().kb_swiglu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), rows, F2 // 2, _stream()), "swiglu_bwd")
    _count()
    return dx


def dropout_add_fwd(x, residual, p, seed):
    if not _bf16(x):
        return ref.dropout_add_fwd(x, residual, p, seed)
    if not (x.is_contiguous() and residual.is_contiguous()):
        _no_recording("making a dropout-add operand contiguous")
        x, residual = x.contiguous(), residual.contiguous()
    y = torch.empty_like(x)
    _check(lib().kb_dropout_add_fwd(x.data_ptr(), residual.data_ptr(), y.data_ptr(), x.numel(), float(p),
                                    int(seed) & 0xFFFFFFFF, _stream()), "dropout_add_fwd")
    _count()
    return y


def dropout_add_bwd(dy, p, seed):
    if not _bf16(dy):
        return ref.dropout_add_bwd(dy, p, seed)
    if p <= 0.0:
        return dy, dy
    dy = dy.contiguous()
    dx = torch.empty_like(dy)
    _check(lib().kb_dropout_bwd(dy.data_ptr(), dx.data_ptr(), dy.numel(), float(p), int(seed) & 0xFFFFFFFF,
                                _stream()), "dropout_bwd")
    _count()
    return dx, dy


def add(a, b):
    if not _bf16(a) or a.numel() % 8 or not (a.is_contiguous() and b.is_contiguous()):
        _no_recording("an elementwise add outside the library")
        return a + b
    y = torch.empty_like(a)
    _check(lib().kb_add(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), _stream()), "add")
    _count()
    return y


# ----------------------------------------------------------------------------- GEMM
def _rowmajor_ok(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 \
        and t.stride(0) >= t.shape[1]


ACTIVATIONS = {None: 0, "none": 0, "gelu": 1}


def gemm(a, b, trans_a=False, trans_b=True, out_dtype=None, accumulate=None, out=None, num_sms=None, bias=None,
         activation=None):
    """``op(a) @ op(b)`` on the tcgen05 kernel.  ``a``: [M,K] (or [K,M] if ``trans_a``); ``b``: [N,K]
    when ``trans_b`` (the nn.Linear weight layout) else [K,N].  ``bias`` ([N]) and ``activation``
    (``"gelu"``) are applied to the accumulator in the kernel's epilogue."""
    if not _bf16(a):
        if bias is not None or activation:
            r = ref.gemm(a, b, trans_a, trans_b, None, None)
            r = ref.bias_act(r, bias, activation)
            if out_dtype is not None:
                r = r.to(out_dtype)
            if out is not None:
                out.copy_(r)
                return out
            return r
        r = ref.gemm(a, b, trans_a, trans_b, out_dtype, accumulate)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if not _rowmajor_ok(a):
        _no_recording("making a GEMM operand contiguous")
        a = a.contiguous()
    if not _rowmajor_ok(b):
        _no_recording("making a GEMM operand contiguous")
        b = b.contiguous()
    if not (_rowmajor_ok(a) and _rowmajor_ok(b)):
        raise KernelError(f"gemm operands need 16-byte aligned rows: a{tuple(a.shape)} b{tuple(b.shape)}")
    M, K = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[0], b.shape[1]) if trans_b else (b.shape[1], b.shape[0])
    if K != Kb:
        raise ValueError(f"gemm shape mismatch: K={K} vs {Kb}")
    if accumulate is not None:
        if accumulate.dtype != torch.float32 or not accumulate.is_contiguous() or tuple(accumulate.shape) != (M, N):
            raise KernelError("accumulate must be a contiguous fp32 [M,N] tensor")
        c, f32, acc = accumulate, 1, 1
    else:
        dt = out_dtype or torch.bfloat16
        if out is None:
            out = torch.empty(M, N, dtype=dt, device=a.device)
        elif not (out.dim() == 2 and out.stride(1) == 1):
            raise KernelError("gemm out must have a contiguous last dim")
        c, f32, acc = out, 1 if out.dtype == torch.float32 else 0, 0
    st = status_word(a.device)
    if bias is not None or activation:
        if accumulate is not None:
            raise KernelError("a bias/activation epilogue cannot be combined with accumulation")
        if activation not in ACTIVATIONS:
            raise KernelError(f"unknown epilogue activation {activation!r}")
        bp = 0
        if bias is not None:
            if bias.numel() != N:
                raise KernelError(f"bias has {bias.numel()} elements for {N} output features")
            bias = bias if (_bf16(bias) and bias.is_contiguous()) else bias.to(torch.bfloat16).contiguous()
            bp = bias.data_ptr()
        rc = lib().kb_gemm_bias_act_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, 1 if trans_a else 0,
                                         a.stride(0), 0 if trans_b else 1, b.stride(0), c.stride(0), f32, 0,
                                         int(num_sms) if num_sms else 0, bp, ACTIVATIONS[activation], st.data_ptr(),
                                         _stream())
        if rc != 0:
            _check(rc, f"gemm+epilogue M={M} N={N} K={K}")
        _count()
        return c
    rc = lib().kb_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, 1 if trans_a else 0, a.stride(0),
                            0 if trans_b else 1, b.stride(0), c.stride(0), f32, acc,
                            int(num_sms) if num_sms else 0, st.data_ptr(), _stream())
    if rc != 0:
        _check(rc, f"gemm M={M} N={N} K={K}")
    _count()
    return c


def gemm_library(a, b, trans_a=False, trans_b=True, out_dtype=None, accumulate=None, out=None, bias=None,
                 activation=None):
    """cuBLAS through torch: the A/B baseline, never the default."""
    _no_recording("a cuBLAS GEMM")
    A = a.t() if trans_a else a
    B = b.t() if trans_b else b
    if bias is not None or activation:
        r = ref.bias_act(torch.matmul(A, B), bias, activation)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if accumulate is not None:
        accumulate.add_(torch.matmul(A, B).to(accumulate.dtype))
        return accumulate
    r = torch.matmul(A, B)
    if out_dtype is not None and r.dtype != out_dtype:
        r = r.to(out_dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


# ----------------------------------------------------------------------------- attention
def _heads4(t):
    if t.dim() == 5:
        s, b, g, r, d = t.shape
        if g == 1:
            return t.squeeze(2)
        if t.stride(2) == r * t.stride(3):
            return t.as_strided((s, b, g * r, d), (t.stride(0), t.stride(1), t.stride(3), t.stride(4)),
                                t.storage_offset())
        return t.reshape(s, b, g * r, d)
    return t


def attention_fwd_library(q, k, v, scale, causal=True, q_offset=0, kv_len=None):
    """flash-attention wheel (bshd views, no copies for the common strides)."""
    _no_recording("the flash-attention wheel")
    from flash_attn.flash_attn_interface import _flash_attn_forward
    q4 = _heads4(q)
    sk = k.shape[0] if kv_len is None else kv_len
    if q_offset != sk - q4.shape[0]:
        raise KernelError("library attention supports only bottom-right aligned causal masks")
    qb, kb, vb = q4.permute(1, 0, 2, 3), k[:sk].permute(1, 0, 2, 3), v[:sk].permute(1, 0, 2, 3)
    out, lse, _, _ = _flash_attn_forward(qb, kb, vb, 0.0, scale, causal=causal, window_size_left=-1,
                                         window_size_right=-1, softcap=0.0, alibi_slopes=None, return_softmax=False)
    return out.permute(1, 0, 2, 3), lse


def attention_bwd_library(do, q, k, v, o, lse, scale, causal=True, q_offset=0, kv_len=None, out=None):
    _no_recording("the flash-attention wheel")
    from flash_attn.flash_attn_interface import _flash_attn_backward
    q4 = _heads4(q)
    sk = k.shape[0] if kv_len is None else kv_len
    qb, kb, vb = q4.permute(1, 0, 2, 3), k[:sk].permute(1, 0, 2, 3), v[:sk].permute(1, 0, 2, 3)
    ob, dob = _heads4(o).permute(1, 0, 2, 3), _heads4(do).permute(1, 0, 2, 3)
    dq = torch.empty_like(qb)
    dk = torch.empty_like(kb)
    dv = torch.empty_like(vb)
    _flash_attn_backward(dob.contiguous(), qb, kb, vb, ob, lse, dq, dk, dv, 0.0, scale, causal, -1, -1, 0.0, None,
                         False)
    dq, dk, dv = dq.permute(1, 0, 2, 3), dk.permute(1, 0, 2, 3), dv.permute(1, 0, 2, 3)
    if sk != k.shape[0]:
        dkf, dvf = torch.zeros_like(k), torch.zeros_like(v)
        dkf[:sk], dvf[:sk] = dk, dv
        dk, dv = dkf, dvf
    if out is not None:
        out[0].copy_(dq.reshape(out[0].shape))
        out[1].copy_(dk)
        out[2].copy_(dv)
        return out
    return dq.reshape(q.shape), dk, dv


_FALLBACK_LOGGED = [False]


def attention_fallback_allowed(reason: str, strict: bool) -> None:
    """Gate of the only route from the native attention entry points to the flash-attention wheel.

    ``strict`` calls (operands may be peer memory) never pass.  Other calls pass only with
    ``KAREUS_B200_ATTENTION_FALLBACK=1`` and say so once on stderr."""
    if strict:
        raise KernelError(f"native attention kernel cannot take this call ({reason}) and the operands may be "
                          "another GPU's memory: no library or PyTorch route is allowed")
    if os.environ.get("KAREUS_B200_ATTENTION_FALLBACK", "0") != "1":
        raise KernelError(f"native attention kernel cannot take this call ({reason}); set "
                          "KAREUS_B200_ATTENTION_FALLBACK=1 to run such shapes on the flash-attention wheel")
    if not _FALLBACK_LOGGED[0]:
        import sys
        print(f"kareus_b200: attention falls back to the flash-attention wheel ({reason})", file=sys.stderr)
        _FALLBACK_LOGGED[0] = True


def attention_fwd(q, k, v, scale, causal=True, q_offset=0, kv_len=None, strict=False):
    if not _bf16(q):
        if strict:
            raise KernelError(f"attention on peer-memory operands needs bf16, got {q.dtype}")
        return ref.attention_fwd(q, k, v, scale, causal, q_offset, kv_len)
    from . import attention_cuda
    return attention_cuda.forward(q, k, v, scale, causal, q_offset, kv_len, strict=strict)


def attention_bwd(do, q, k, v, o, lse, scale, causal=True, q_offset=0, kv_len=None, out=None, strict=False):
    if not _bf16(q):
        if strict:
            raise KernelError(f"attention on peer-memory operands needs bf16, got {q.dtype}")
        dq, dk, dv = ref.attention_bwd(do, q, k, v, o, lse, scale, causal, q_offset, kv_len)
        if out is not None:
            out[0].copy_(dq.reshape(out[0].shape))
            out[1].copy_(dk)
            out[2].copy_(dv)
            return out
        return dq, dk, dv
    from . import attention_cuda
    return attention_cuda.backward(do, q, k, v, o, lse, scale, causal, q_offset, kv_len, out, strict=strict)


# ----------------------------------------------------------------------------- cross entropy
def cross_entropy_local_stats(logits, targets, vocab_start):
    if not _bf16(logits):
        return ref.cross_entropy_local_stats(logits, targets, vocab_start)
    rows, V = logits.shape
    st = torch.empty(3, rows, dtype=torch.float32, device=logits.device)
    targets = targets.contiguous()
    _check(lib().kb_ce_stats(logits.data_ptr(), targets.data_ptr(), st[0].data_ptr(), st[1].data_ptr(),
                             st[2].data_ptr(), rows, V, int(vocab_start), _stream()), "ce_stats")
    _count()
    return st[0], st[1], st[2]


def cross_entropy_finish(logits, targets, vocab_start, gmax, gsum, grad_scale):
    if not _bf16(logits):
        return ref.cross_entropy_finish(logits, targets, vocab_start, gmax, gsum, grad_scale)
    rows, V = logits.shape
    targets = targets.contiguous()
    gmax, gsum = gmax.contiguous().float(), gsum.contiguous().float()
    grad_scale = grad_scale.contiguous().float()
    _check(lib().kb_ce_grad(logits.data_ptr(), targets.data_ptr(), gmax.data_ptr(), gsum.data_ptr(),
                            grad_scale.data_ptr(), rows, V, int(vocab_start), _stream()), "ce_grad")
    _count()
    return logits


# ----------------------------------------------------------------------------- embedding
def embedding_fwd(tokens, weight, vocab_start):
    if not _bf16(weight):
        return ref.embedding_fwd(tokens, weight, vocab_start)
    tokens = tokens.contiguous()
    H = weight.shape[1]
    out = torch.empty(tuple(tokens.shape) + (H,), dtype=weight.dtype, device=weight.device)
    _check(lib().kb_embedding_fwd(tokens.data_ptr(), weight.data_ptr(), out.data_ptr(), tokens.numel(), H,
                                  int(vocab_start), weight.shape[0], _stream()), "embedding_fwd")
    _count()
    return out


def embedding_bwd(dout, tokens, grad_weight, vocab_start):
    if not _bf16(dout) or grad_weight.dtype != torch.float32:
        return ref.embedding_bwd(dout, tokens, grad_weight, vocab_start)
    dout, tokens = dout.contiguous(), tokens.contiguous()
    H = grad_weight.shape[1]
    _check(lib().kb_embedding_bwd(tokens.data_ptr(), dout.data_ptr(), grad_weight.data_ptr(), tokens.numel(), H,
                                  int(vocab_start), grad_weight.shape[0], _stream()), "embedding_bwd")
    _count()
    return grad_weight


# ----------------------------------------------------------------------------- optimizer
def adamw_step(p, g, m, v, master, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, grad_scale_tensor=None):
    """Flat-buffer AdamW.  ``p`` (bf16, may be None), ``g, m, v, master`` fp32, all the same length."""
    if master.dtype != torch.float32 or g.dtype != torch.float32 or (p is not None and p is not master and not _bf16(p)):
        return ref.adamw_step(p, g, m, v, master, lr, beta1, beta2, eps, wd, step, grad_scale)
    pp = 0 if (p is None or p is master) else p.data_ptr()
    gs = grad_scale_tensor.data_ptr() if grad_scale_tensor is not None else 0
    _check(lib().kb_adamw(pp, g.data_ptr(), m.data_ptr(), v.data_ptr(), master.data_ptr(), master.numel(), float(lr),
                          float(beta1), float(beta2), float(eps), float(wd), float(1 - beta1 ** step),
                          float(1 - beta2 ** step), gs, float(grad_scale), _stream()), "adamw")
    _count()


def sumsq(t):
    if t.dtype not in (torch.float32, torch.bfloat16):
        return ref.sumsq(t)
    t = t.contiguous()
    out = torch.zeros(1, dtype=torch.float32, device=t.device)
    _check(lib().kb_sumsq(t.data_ptr(), t.numel(), 1 if t.dtype == torch.float32 else 0, out.data_ptr(), _stream()),
           "sumsq")
    _count()
    return out[0]
