"""NVLink-switch (NVLS) buffer: every rank's memory bound to one multicast object, reduced in the switch.

``NvlsBuffer.create(heap, nbytes)`` is collective over the heap's group: rank 0 creates the multicast
object and hands its file descriptor to the other ranks over a Unix socket (``SCM_RIGHTS``), every
rank joins, binds freshly allocated device memory and maps two views of it — ``local`` (this rank's
copy, ordinary memory) and the multicast view that the kernels of ``csrc/nvls.cu`` address with
``multimem.ld_reduce`` / ``multimem.st``.  ``all_reduce`` and ``reduce_scatter`` then move every byte
through the switch once instead of pulling it from each peer.  Host sequence and device operations of
the reference: ``3rdparty/mscclpp/src/nvls.cc:59-214``, ``include/mscclpp/switch_channel_device.hpp:41-130``,
kernel ``python/mscclpp_benchmark/allreduce.cu:858-942`` (``allreduce6``).

Barriers use the symmetric heap's peer-mapped flags, so an ``NvlsBuffer`` lives next to a
:class:`~kareus_b200.parallel.symm_heap.SymmetricHeap`.

Off unless asked for (``KAREUS_NVLS=1`` in the collective operators, or explicit use).  A rank must
:meth:`close` the buffer (unmap, unbind, release) before it exits while others still run: tests that
end or lose a rank keep this path off and use plain peer loads.
"""
from __future__ import annotations

import array
import ctypes
import os
import socket
from ctypes import c_int, c_long, c_size_t, c_uint64, c_void_p
from typing import Optional

import torch
import torch.distributed as dist

from ..kernels import cuda as KC
from ..kernels import replay as _replay
from .symm_heap import Channel, SymmetricHeap, _Raw


def enabled() -> bool:
    return os.environ.get("KAREUS_NVLS", "0") == "1"


def _declare(L) -> None:
    if getattr(L, "_nvls_declared", False):
        return
    P, I, U64 = c_void_p, c_int, c_uint64
    L.kb_nvls_supported.argtypes = [I]
    L.kb_nvls_create.argtypes = [I, I, c_size_t, ctypes.POINTER(P), ctypes.POINTER(c_size_t), ctypes.POINTER(I)]
    L.kb_nvls_import.argtypes = [I, I, c_size_t, I, ctypes.POINTER(P)]
    L.kb_nvls_add_device.argtypes = [P]
    L.kb_nvls_bind.argtypes = [P, ctypes.POINTER(P), ctypes.POINTER(P)]
    L.kb_nvls_destroy.argtypes = [P]
    L.kb_nvls_allreduce.argtypes = [P, I, I, U64, P, U64, c_long, U64, I, I, P, P]
    L.kb_nvls_reducescatter.argtypes = [P, I, I, U64, P, U64, c_long, P, U64, I, I, P, P]
    for n in ("kb_nvls_supported", "kb_nvls_create", "kb_nvls_import", "kb_nvls_add_device", "kb_nvls_bind",
              "kb_nvls_destroy", "kb_nvls_allreduce", "kb_nvls_reducescatter"):
        getattr(L, n).restype = c_int
    L._nvls_declared = True


def _send_fd(sock: socket.socket, fd: int, payload: bytes) -> None:
    sock.sendmsg([payload], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))])


def _recv_fd(sock: socket.socket, nbytes: int):
    fds = array.array("i")
    msg, anc, _, _ = sock.recvmsg(nbytes, socket.CMSG_LEN(fds.itemsize))
    for level, kind, data in anc:
        if level == socket.SOL_SOCKET and kind == socket.SCM_RIGHTS:
            fds.frombytes(data[: len(data) - (len(data) % fds.itemsize)])
    if not fds:
        raise KC.KernelError("no file descriptor arrived with the multicast handle")
    return fds[0], msg


class NvlsBuffer:
    def __init__(self, heap: SymmetricHeap, state: int, size: int, uc_ptr: int, mc_ptr: int):
        self.heap, self._state, self.size = heap, state, size
        self.uc_ptr, self.mc_ptr = uc_ptr, mc_ptr
        self.local = torch.as_tensor(_Raw(uc_ptr, size), device=heap.device)      # this rank's copy, uint8
        self._top = 0
        self.closed = False

    # ------------------------------------------------------------------ set-up
    @classmethod
    def supported(cls, device) -> bool:
        L = KC.lib()
        _declare(L)
        idx = torch.device(device).index
        return L.kb_nvls_supported(idx if idx is not None else torch.cuda.current_device()) == 1

    @classmethod
    def create(cls, heap: SymmetricHeap, nbytes: int) -> "NvlsBuffer":
        """Collective over ``heap.group``."""
        L = KC.lib()
        _declare(L)
        rank, world, group = heap.rank, heap.world, heap.group
        dev = heap.device.index if heap.device.index is not None else torch.cuda.current_device()
        ok = torch.tensor([1 if cls.supported(heap.device) else 0], device=heap.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) != 1:
            raise KC.KernelError("switch multicast is not supported on every device of the group")
        state = c_void_p()
        size = c_size_t(0)
        name = [None]
        if rank == 0:
            fd = c_int(-1)
            KC._check(L.kb_nvls_create(dev, world, nbytes, ctypes.byref(state), ctypes.byref(size), ctypes.byref(fd)),
                      "multicast create")
            name[0] = f"\0kareus_nvls_{os.getpid()}_{id(heap) & 0xffffff}"
            srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            srv.bind(name[0])
            srv.listen(world)
        dist.broadcast_object_list(name, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        if rank == 0:
            srv.settimeout(60.0)
            try:
                for _ in range(world - 1):
                    conn, _ = srv.accept()
                    with conn:
                        _send_fd(conn, fd.value, str(size.value).encode())
            finally:
                srv.close()
                os.close(fd.value)
        else:
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                c.settimeout(60.0)
                c.connect(name[0])
                got, msg = _recv_fd(c, 64)
            size = c_size_t(int(msg.decode()))
            try:
                KC._check(L.kb_nvls_import(dev, world, size.value, got, ctypes.byref(state)), "multicast import")
            finally:
                os.close(got)
        KC._check(L.kb_nvls_add_device(state), "multicast add device")
        dist.barrier(group=group)                      # every device has joined before anyone binds
        uc, mc = c_void_p(), c_void_p()
        KC._check(L.kb_nvls_bind(state, ctypes.byref(uc), ctypes.byref(mc)), "multicast bind")
        torch.cuda.synchronize(heap.device)
        dist.barrier(group=group)
        return cls(heap, state.value, size.value, uc.value, mc.value)

    # ------------------------------------------------------------------ buffers
    def region(self, nbytes: int):
        """Bump-allocate ``nbytes`` (same offset on every rank); returns the byte offset."""
        off = (self._top + 1023) // 1024 * 1024
        if off + nbytes > self.size:
            raise MemoryError(f"NVLS buffer of {self.size >> 20} MiB is full")
        self._top = off + nbytes
        return off

    def view(self, off: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s_ in shape:
            n *= s_
        return self.local[off:off + n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(shape)

    # ------------------------------------------------------------------ collectives
    def _channel(self, tag: str) -> Channel:
        return self.heap.channel(f"nvls/{tag}")

    def _region_for(self, ch: Channel, nbytes: int) -> int:
        cur = ch.buffers.get("nvls")
        if cur is None or cur[1] < nbytes:
            cur = (self.region(nbytes), nbytes)
            ch.buffers["nvls"] = cur
        return cur[0]

    def staging(self, tag: str, shape, dtype) -> torch.Tensor:
        """This rank's input buffer of the collective ``tag`` (write the data here to save a copy)."""
        n = 1
        for s_ in shape:
            n *= s_
        ch = self._channel(tag)
        return self.view(self._region_for(ch, n * 2), shape, dtype)

    def all_reduce(self, x: torch.Tensor, tag: str = "ar", sm_num: int = 16, block_size: int = 1024) -> torch.Tensor:
        """Sum of ``x`` over the group; returns a view of the bound buffer (valid until the next call with
        this tag)."""
        SymmetricHeap._require_bf16(x, "NVLS all_reduce")
        if x.numel() % 8:
            raise KC.KernelError("NVLS all_reduce needs a multiple of 8 elements")
        ch = self._channel(tag)
        off = self._region_for(ch, x.numel() * 2)
        buf = self.view(off, x.shape, x.dtype)
        if buf.data_ptr() != x.data_ptr():
            _replay.copy_(buf, x if x.is_contiguous() else x.contiguous())
        ch.bump()
        st = KC.status_word(self.heap.device)
        KC._check(KC.lib().kb_nvls_allreduce(self.heap._bases_arr, self.heap.rank, self.heap.world, ch.flag_off,
                                             c_void_p(self.mc_ptr), off, x.numel(), ch.epoch, int(sm_num),
                                             int(block_size), st.data_ptr(), KC._stream()), "nvls allreduce")
        KC._count()
        return buf

    def reduce_scatter(self, x: torch.Tensor, tag: str = "rs", sm_num: int = 16, block_size: int = 1024) -> torch.Tensor:
        """Sum over the group of dim-0 shard ``rank`` of ``x``."""
        SymmetricHeap._require_bf16(x, "NVLS reduce_scatter")
        world = self.heap.world
        if x.shape[0] % world or (x.numel() // world) % 8:
            raise KC.KernelError("NVLS reduce_scatter needs dim 0 divisible by the group and shards of 8n elements")
        ch = self._channel(tag)
        off = self._region_for(ch, x.numel() * 2)
        buf = self.view(off, x.shape, x.dtype)
        if buf.data_ptr() != x.data_ptr():
            _replay.copy_(buf, x if x.is_contiguous() else x.contiguous())
        out = torch.empty((x.shape[0] // world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        ch.bump()
        st = KC.status_word(self.heap.device)
        KC._check(KC.lib().kb_nvls_reducescatter(self.heap._bases_arr, self.heap.rank, world, ch.flag_off,
                                                 c_void_p(self.mc_ptr), off, x.numel() // world, out.data_ptr(),
                                                 ch.epoch, int(sm_num), int(block_size), st.data_ptr(), KC._stream()),
                  "nvls reducescatter")
        KC._count()
        return out

    # ------------------------------------------------------------------ teardown
    def close(self, collective: bool = True) -> None:
        """Everyone stops using the object, then unmaps, unbinds and releases its part.  ``collective=False``
        skips the barriers: the way out for a rank that leaves on an error (its kernels have drained; the
        peers' waits on it are bounded)."""
        if self.closed:
            return
        self.closed = True
        torch.cuda.synchronize(self.heap.device)
        sync = collective and self.heap.world > 1 and dist.is_initialized()
        if sync:
            dist.barrier(group=self.heap.group)
        self.local = None
        KC._check(KC.lib().kb_nvls_destroy(c_void_p(self._state)), "multicast destroy")
        if sync:
            dist.barrier(group=self.heap.group)
