"""Launch lists: record the kernels a region of the step enqueues once, replay them from C++.

One training step of the 3B model enqueues about twenty thousand kernels per rank through Python and
ctypes; at eight GPUs the kernels are short enough that the interpreter, not the GPU, sets the
pace.  The arguments of those launches repeat from microbatch to microbatch, so the block engine
records them once (``csrc/launch_list.cpp``: every launch, copy, memset, event record and stream
wait issued by this library while a recording is open) and afterwards re-issues the list with one
call: same kernels, same streams, same event edges, no interpreter in the loop.  The reference has
no counterpart: it pays the per-operator Python cost on every step
(``kareus/megatron/core/partitions/partition_base.py:186-299``).

This module is the Python face of the recorder: opening and closing a recording, mirroring
``torch.cuda.Event`` records/waits into it, naming epoch counters, and keeping tensors alive that
another stream still uses.  Memory: a recording allocates from a private ``torch.cuda.MemPool``
and the pool keeps every block afterwards, so the addresses baked into the list stay valid; tensors
handed to another stream (``record_stream``) are additionally held until the recording ends, which
keeps the allocator from reusing them inside the list on the strength of events that a replay
does not have.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_size_t, c_uint64, c_void_p
from typing import Dict, List, Optional

import torch

from . import cuda as KC

_DECLARED = False
_ACTIVE: Optional["Recording"] = None


class ReplayError(RuntimeError):
    pass


def _lib():
    global _DECLARED
    L = KC.lib()
    if not _DECLARED:
        P, I = c_void_p, c_int
        L.kb_rec_begin.argtypes = [P]
        L.kb_rec_end.argtypes = []
        L.kb_rec_end.restype = c_long
        L.kb_rec_abort.argtypes = []
        L.kb_rec_new_event.argtypes = []
        L.kb_rec_event_record.argtypes = [I, P]
        L.kb_rec_stream_wait.argtypes = [P, I]
        L.kb_rec_next_epoch.argtypes = [ctypes.POINTER(c_uint64)]
        L.kb_replay.argtypes = [I, P]
        L.kb_rec_launches.argtypes = [I]
        L.kb_rec_launches.restype = c_long
        L.kb_rec_ops.argtypes = [I]
        L.kb_rec_ops.restype = c_long
        L.kb_rec_free.argtypes = [I]
        L.kb_memcpy_d2d.argtypes = [P, P, c_size_t, P]
        L.kb_memset.argtypes = [P, I, c_size_t, P]
        for n in ("kb_rec_begin", "kb_rec_abort", "kb_rec_new_event", "kb_rec_event_record", "kb_rec_stream_wait",
                  "kb_rec_next_epoch", "kb_replay", "kb_rec_free", "kb_memcpy_d2d", "kb_memset"):
            getattr(L, n).restype = c_int
        _DECLARED = True
    return L


def active() -> bool:
    """True while a recording is open (operators must then avoid every launch this library cannot see)."""
    return _ACTIVE is not None


def require_recordable(what: str) -> None:
    """Called on code paths that launch PyTorch or NCCL kernels: those cannot be part of a launch list."""
    if _ACTIVE is not None:
        raise ReplayError(f"{what} launches work outside this library and cannot be recorded into a launch list")


class LaunchList:
    """A finished recording."""

    def __init__(self, list_id: int, ops: int, launches: int):
        self.id, self.ops, self.launches = list_id, ops, launches

    def replay(self) -> None:
        rc = _lib().kb_replay(self.id, KC._stream())
        KC._check(rc, "launch-list replay")
        KC._count(self.launches)

    def free(self) -> None:
        if self.id:
            _lib().kb_rec_free(self.id)
            self.id = 0


class Recording:
    """Context manager around ``kb_rec_begin`` / ``kb_rec_end`` on the current stream."""

    def __init__(self):
        self.events: Dict[int, tuple] = {}       # id(torch event) -> (native event index, the event)
        self.keepalive: List[torch.Tensor] = []
        self.result: Optional[LaunchList] = None
        self._id = 0

    def __enter__(self) -> "Recording":
        global _ACTIVE
        if _ACTIVE is not None:
            raise ReplayError("a recording is already open")
        self._id = _lib().kb_rec_begin(KC._stream())
        if self._id <= 0:
            raise ReplayError("could not open a recording")
        _ACTIVE = self
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        global _ACTIVE
        _ACTIVE = None
        L = _lib()
        if exc_type is not None:
            L.kb_rec_abort()
        else:
            ops = L.kb_rec_end()
            if ops < 0:
                raise ReplayError("recording was not open")
            self.result = LaunchList(self._id, int(ops), int(L.kb_rec_launches(self._id)))
        self.events.clear()
        self.keepalive.clear()
        return False


# ----------------------------------------------------------------------------- hooks used by the engine
def _raw(stream) -> int:
    return stream.cuda_stream


def note_event_record(event, stream) -> None:
    """``event.record(stream)`` was issued: mirror it into the open recording."""
    r = _ACTIVE
    if r is None:
        return
    L = _lib()
    hit = r.events.get(id(event))
    if hit is None:
        idx = L.kb_rec_new_event()
        if idx < 0:
            raise ReplayError("could not create an event for the recording")
        r.events[id(event)] = (idx, event)
    else:
        idx = hit[0]
    KC._check(L.kb_rec_event_record(idx, _raw(stream)), "record event")


def note_stream_wait(stream, event) -> None:
    """``stream.wait_event(event)`` was issued."""
    r = _ACTIVE
    if r is None:
        return
    hit = r.events.get(id(event))
    if hit is None:
        raise ReplayError("a stream waits for an event that was recorded before the recording began")
    KC._check(_lib().kb_rec_stream_wait(_raw(stream), hit[0]), "stream wait")


def note_cross_stream_use(t) -> None:
    """``t`` is used on a stream other than the one it was allocated on: hold it to the end of the
    recording so its memory is not handed out again inside the list."""
    if _ACTIVE is not None and isinstance(t, torch.Tensor):
        _ACTIVE.keepalive.append(t)


def next_epoch(counter: c_uint64) -> None:
    """The next launch that carries a channel epoch takes it from ``counter`` on every replay."""
    if _ACTIVE is not None:
        _lib().kb_rec_next_epoch(ctypes.byref(counter))


# ----------------------------------------------------------------------------- recordable copies
def memcpy(dst: torch.Tensor, src: torch.Tensor) -> None:
    """Device-to-device copy of two contiguous tensors of the same byte size (recordable)."""
    n = src.numel() * src.element_size()
    if not (dst.is_contiguous() and src.is_contiguous()) or dst.numel() * dst.element_size() != n:
        raise ReplayError("memcpy needs two contiguous tensors of the same size")
    KC._check(_lib().kb_memcpy_d2d(dst.data_ptr(), src.data_ptr(), n, KC._stream()), "memcpy")


def copy_(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``dst.copy_(src)`` through the recordable copy when the layouts allow it."""
    if dst.is_cuda and src.is_cuda and dst.dtype == src.dtype and dst.is_contiguous() and src.is_contiguous() \
            and dst.numel() == src.numel():
        memcpy(dst, src)
        return dst
    require_recordable("a strided or converting tensor copy")
    return dst.copy_(src)


def clone(t: torch.Tensor) -> torch.Tensor:
    if t.is_cuda and t.is_contiguous():
        out = torch.empty_like(t)
        memcpy(out, t)
        return out
    require_recordable("a strided tensor clone")
    return t.clone()
