"""Symmetric heap: one device allocation per rank, mapped into every peer of the group.

Every buffer carved out of the heap has the same byte offset on every rank, so a kernel can reach
rank ``p``'s copy of a buffer as ``base[p] + offset`` with plain loads and stores over NVLink.
This replaces the reference's registered-memory exchange and memory channels
(``kareus/msccl/msccl_comm.py:44-206``; ``3rdparty/mscclpp/src/registered_memory.cc``): handles
are CUDA IPC handles exchanged with ``torch.distributed.all_gather_object``.

Layout: ``[flag region | data region]``.  Each *channel* (one per collective call site and
nanobatch) owns a block of 64-bit flag slots and its data buffers; buffers are allocated once
(bump allocator, identical call order on all ranks) and reused, which is what gives every
nanobatch its own staging memory.  Tokens written into flag slots grow monotonically with the
channel's call count, so nothing is ever reset.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_long, c_size_t, c_uint64, c_void_p
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..kernels import cuda as KC
from ..kernels import replay as _replay

MAX_PEERS = 8
MAX_SIGNAL_CTAS = 64
FLAG_BLOCK = MAX_PEERS * MAX_SIGNAL_CTAS * 8          # bytes of one channel's barrier flags
FLAG_REGION = 4 << 20


class _Raw:
    """Exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


GUARD_BYTES = 1024
GUARD_PATTERN = 0xA5


class GuardMap:
    """Canary words between heap buffers (race / overrun detection).

    Every buffer carved out of the heap is followed by ``GUARD_BYTES`` painted with a fixed pattern.
    No kernel has a reason to write there, so a guard that changed means some kernel, on this GPU or
    on a peer that maps this heap, wrote past the end of the buffer in front of it (or before the
    start of the one behind it).  ``check`` names the damaged guards.  The reference has no such
    check: its collective buffers are separate allocations and an overrun there is silent
    (``kareus/msccl/msccl_comm.py:44-206``)."""

    def __init__(self):
        self.guards: List[Tuple[int, int, str]] = []     # (offset, nbytes, name of the buffer in front)

    def add(self, off: int, nbytes: int, name: str) -> None:
        self.guards.append((off, nbytes, name))

    def paint(self, heap_bytes: torch.Tensor, off: int, nbytes: int) -> None:
        heap_bytes[off:off + nbytes].fill_(GUARD_PATTERN)

    def check(self, heap_bytes: torch.Tensor) -> List[str]:
        """Names of the buffers whose trailing guard no longer holds the pattern (one device sync)."""
        if not self.guards:
            return []
        bad = torch.stack([(heap_bytes[o:o + n] != GUARD_PATTERN).any() for o, n, _ in self.guards])
        return [self.guards[i][2] for i in torch.nonzero(bad.cpu()).flatten().tolist()]


class Channel:
    """One call site's flag block and buffers.  ``epoch`` counts the calls made on the channel; it lives
    in a ``c_uint64`` so that a launch-list replay (C++) can advance the same counter."""

    def __init__(self, index: int, flag_off: int):
        self.index, self.flag_off = index, flag_off
        self.counter = c_uint64(0)
        self.buffers: Dict[str, Tuple[int, int]] = {}     # name -> (offset, nbytes)

    @property
    def epoch(self) -> int:
        return self.counter.value

    @epoch.setter
    def epoch(self, v: int) -> None:
        self.counter.value = v

    def bump(self) -> int:
        """Advance the epoch for one more call and tell an open recording where it lives."""
        self.counter.value += 1
        _replay.next_epoch(self.counter)
        return self.counter.value


def node_identity() -> str:
    """Something that is equal for two processes exactly when they run on the same machine."""
    import socket
    boot = ""
    try:
        with open("/proc/sys/kernel/random/boot_id") as f:
            boot = f.read().strip()
    except OSError:
        pass
    return f"{socket.gethostname()}/{boot}"


def require_one_node(group, world: int) -> None:
    """Peer mappings (CUDA IPC) exist between GPUs of one machine only: the ranks of a heap — a tensor- or
    context-parallel group — must not span nodes (put pipeline and data parallelism across nodes instead, as
    the reference's launch scripts do).  Collective over ``group``."""
    if world <= 1 or not dist.is_initialized():
        return
    ids = [None] * world
    dist.all_gather_object(ids, node_identity(), group=group)
    if len(set(ids)) > 1:
        raise RuntimeError(f"the {world} ranks of this peer-memory group run on {len(set(ids))} different machines; "
                           "tensor/context-parallel groups that use the kernel backend must stay inside one node")


class SymmetricHeap:
    def __init__(self, group, rank: int, world: int, device, size_bytes: int):
        self.group, self.rank, self.world = group, rank, world
        self.device = torch.device(device)
        self.size = int(size_bytes)
        self.lib = KC.lib()
        self._declare()
        ptr = c_void_p()
        KC._check(self.lib.kb_heap_alloc(c_size_t(self.size), ctypes.byref(ptr)), "heap alloc")
        self.local_ptr = ptr.value
        handle = (ctypes.c_ubyte * 64)()
        KC._check(self.lib.kb_ipc_get_handle(c_void_p(self.local_ptr), handle), "ipc handle")
        handles: List[Optional[bytes]] = [None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        else:
            handles = [bytes(handle)]
        self.bases: List[int] = []
        for r, h in enumerate(handles):
            if r == rank:
                self.bases.append(self.local_ptr)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            p = c_void_p()
            KC._check(self.lib.kb_ipc_open(buf, ctypes.byref(p)), f"ipc open rank {r}")
            self.bases.append(p.value)
        self._bases_arr = (c_void_p * MAX_PEERS)(*(self.bases + [None] * (MAX_PEERS - world)))
        self.local = torch.as_tensor(_Raw(self.local_ptr, self.size), device=self.device)
        self._flag_top = 0
        self._data_top = FLAG_REGION
        self.guards = GuardMap()
        self.channels: Dict[str, Channel] = {}
        self._views: Dict[tuple, torch.Tensor] = {}
        self.nvls = None               # NvlsBuffer once enable_nvls() has run: all-reduce / reduce-scatter go
        self.closed = False            # through the NVLink switch (multimem) instead of peer loads
        if world > 1:
            dist.barrier(group=group)

    @classmethod
    def create(cls, group, device, size_bytes: int = 6 << 30) -> "SymmetricHeap":
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} ranks per heap")
        require_one_node(group, world)
        return cls(group, rank, world, device, size_bytes)

    def _declare(self) -> None:
        L = self.lib
        P, I, LNG, U64 = c_void_p, c_int, c_long, c_uint64
        L.kb_heap_alloc.argtypes = [c_size_t, ctypes.POINTER(c_void_p)]
        L.kb_ipc_get_handle.argtypes = [P, P]
        L.kb_ipc_open.argtypes = [P, ctypes.POINTER(c_void_p)]
        L.kb_ipc_close.argtypes = [P]
        L.kb_heap_free.argtypes = [P]
        L.kb_allreduce.argtypes = [P, I, I, U64, U64, LNG, U64, I, I, P, P]
        L.kb_allgather.argtypes = [P, I, I, U64, U64, LNG, U64, I, I, P, P]
        L.kb_reducescatter.argtypes = [P, I, I, U64, U64, LNG, P, U64, I, I, P, P]
        L.kb_wait_flag.argtypes = [P, U64, U64, P, P]
        L.kb_peer_barrier.argtypes = [P, I, I, U64, U64, P, P]
        L.kb_peer_barrier.restype = c_int
        for n in ("kb_heap_alloc", "kb_ipc_get_handle", "kb_ipc_open", "kb_ipc_close", "kb_heap_free", "kb_allreduce",
                  "kb_allgather", "kb_reducescatter", "kb_wait_flag"):
            getattr(L, n).restype = c_int

    def enable_nvls(self, nbytes: int = 1 << 30) -> bool:
        """Collective.  Bind ``nbytes`` per rank to an NVLink-switch multicast object and route all-reduce
        and reduce-scatter through it (see :mod:`kareus_b200.parallel.nvls`).  Returns False (and changes
        nothing) when a device of the group lacks multicast support."""
        from .nvls import NvlsBuffer
        if self.world < 2 or self.nvls is not None:
            return self.nvls is not None
        ok = torch.tensor([1 if NvlsBuffer.supported(self.device) else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) != 1:
            return False
        self.nvls = NvlsBuffer.create(self, nbytes)
        return True

    # ------------------------------------------------------------------ allocation
    def channel(self, name: str, flag_bytes: int = FLAG_BLOCK) -> Channel:
        ch = self.channels.get(name)
        if ch is None:
            need = (flag_bytes + 255) // 256 * 256
            if self._flag_top + need > FLAG_REGION:
                raise MemoryError("symmetric heap: flag region exhausted")
            ch = Channel(len(self.channels), self._flag_top)
            self._flag_top += need
            self.channels[name] = ch
        return ch

    def buffer(self, ch: Channel, name: str, nbytes: int) -> Tuple[int, torch.Tensor]:
        """Persistent buffer of a channel: ``(byte offset, uint8 view)``.  Grows by reallocation at the
        top of the heap if a later call needs more (all ranks make the same calls)."""
        cur = ch.buffers.get(name)
        if cur is None or cur[1] < nbytes:
            off = (self._data_top + 1023) // 1024 * 1024
            end = (off + nbytes + 15) // 16 * 16
            if end + GUARD_BYTES > self.size:
                raise MemoryError(f"symmetric heap of {self.size >> 20} MiB is full (asked {nbytes >> 20} MiB for {name})")
            # canary words behind the buffer (see GuardMap); painted once, checked on demand
            self.guards.paint(self.local, end, GUARD_BYTES)
            self.guards.add(end, GUARD_BYTES, f"channel {ch.index} buffer {name!r} at {off}")
            self._data_top = end + GUARD_BYTES
            ch.buffers[name] = (off, nbytes)
            cur = (off, nbytes)
        return cur[0], self.local[cur[0]:cur[0] + nbytes]

    def peer_view(self, rank: int, off: int, shape, dtype) -> torch.Tensor:
        """The same buffer in rank ``rank``'s heap, addressed through the peer mapping.  Only kernels of
        this package may read it (plain or TMA loads without multicast), through entry points called
        with ``peer=True``; those refuse every library or PyTorch route.  With the library baseline
        switched on no peer view is handed out at all."""
        from ..kernels import library_baseline
        if library_baseline():
            raise KC.KernelError("peer views are not available with KAREUS_B200_LIBRARY_BASELINE=1: a vendor-library "
                                 "kernel must never receive another GPU's memory as an operand")
        if rank == self.rank:
            return self.view(off, shape, dtype)
        n = 1
        for s_ in shape:
            n *= s_
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        raw = torch.as_tensor(_Raw(self.bases[rank] + off, nbytes), device=self.device)
        return raw.view(dtype).view(shape)

    def barrier(self, ch: Channel) -> None:
        """Stream-ordered barrier among the ranks (a one-CTA kernel on the current stream)."""
        ch.bump()
        st = KC.status_word(self.device)
        KC._check(self.lib.kb_peer_barrier(self._bases_arr, self.rank, self.world, ch.flag_off, ch.epoch,
                                           st.data_ptr(), KC._stream()), "peer barrier")
        KC._count()

    def view(self, off: int, shape, dtype) -> torch.Tensor:
        key = (off, tuple(shape), dtype)
        hit = self._views.get(key)
        if hit is not None:
            return hit
        t = self._make_view(off, shape, dtype)
        if len(self._views) < 4096:
            self._views[key] = t
        return t

    def _make_view(self, off: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[off:off + nbytes].view(dtype).view(shape)

    # ------------------------------------------------------------------ collectives
    def _launch_shape(self, sm_num, block_size):
        return int(sm_num or 16), int(block_size or 1024)

    @staticmethod
    def _require_bf16(x: torch.Tensor, what: str) -> None:
        """The all-pairs kernels add and move bf16 elements; any other dtype would be reinterpreted."""
        if x.dtype != torch.bfloat16:
            raise KC.KernelError(f"symmetric-heap {what} supports bf16 only, got {x.dtype}; use the "
                                 "torch.distributed backend for other dtypes")

    def all_reduce(self, x: torch.Tensor, nb: int = 0, sm_num=None, block_size=None, tag: str = "ar") -> torch.Tensor:
        self._require_bf16(x, "all_reduce")
        if self.nvls is not None and x.numel() % 8 == 0:
            sm, blk = self._launch_shape(sm_num, block_size)
            return self.nvls.all_reduce(x, tag=f"{tag}/{nb}", sm_num=sm, block_size=blk)
        ch = self.channel(f"{tag}/{nb}")
        n = x.numel()
        off, _ = self.buffer(ch, "x", n * x.element_size())
        buf = self.view(off, x.shape, x.dtype)
        if x.data_ptr() != buf.data_ptr():
            _replay.copy_(buf, x)
        ch.bump()
        sm, blk = self._launch_shape(sm_num, block_size)
        st = KC.status_word(self.device)
        KC._check(self.lib.kb_allreduce(self._bases_arr, self.rank, self.world, ch.flag_off, off, n, ch.epoch, sm, blk,
                                        st.data_ptr(), KC._stream()), "allreduce")
        KC._count()
        return buf

    def staging(self, kind: str, tag: str, nb: int, shape, dtype) -> torch.Tensor:
        """The heap buffer a collective would copy its input into; a producer that writes its result
        there (``gemm(..., out=...)``) saves the copy.  ``kind``: ``"ar"`` or ``"rs"``."""
        n = 1
        for s_ in shape:
            n *= s_
        if self.nvls is not None and dtype == torch.bfloat16 and n % (8 * self.world) == 0:
            return self.nvls.staging(f"{tag}/{nb}", shape, dtype)
        ch = self.channel(f"{tag}/{nb}")
        off, _ = self.buffer(ch, "x", n * torch.empty((), dtype=dtype).element_size())
        return self.view(off, shape, dtype)

    def all_gather(self, x: torch.Tensor, nb: int = 0, sm_num=None, block_size=None, tag: str = "ag",
                   keep: bool = False) -> torch.Tensor:
        self._require_bf16(x, "all_gather")
        ch = self.channel(f"{tag}/{nb}")
        shard = x.numel() * x.element_size()
        off, _ = self.buffer(ch, "x", shard * self.world)
        out = self.view(off, (x.shape[0] * self.world,) + tuple(x.shape[1:]), x.dtype)
        _replay.copy_(out[self.rank * x.shape[0]:(self.rank + 1) * x.shape[0]], x)
        ch.bump()
        sm, blk = self._launch_shape(sm_num, block_size)
        st = KC.status_word(self.device)
        KC._check(self.lib.kb_allgather(self._bases_arr, self.rank, self.world, ch.flag_off, off, shard, ch.epoch, sm,
                                        blk, st.data_ptr(), KC._stream()), "allgather")
        KC._count()
        # the buffer is reused by the next call of this site: callers that keep the result ask for a copy
        return _replay.clone(out) if keep else out

    def reduce_scatter(self, x: torch.Tensor, nb: int = 0, sm_num=None, block_size=None, tag: str = "rs") -> torch.Tensor:
        self._require_bf16(x, "reduce_scatter")
        if self.nvls is not None and (x.numel() // self.world) % 8 == 0 and x.shape[0] % self.world == 0:
            sm, blk = self._launch_shape(sm_num, block_size)
            return self.nvls.reduce_scatter(x, tag=f"{tag}/{nb}", sm_num=sm, block_size=blk)
        ch = self.channel(f"{tag}/{nb}")
        n = x.numel()
        off, _ = self.buffer(ch, "x", n * x.element_size())
        buf = self.view(off, x.shape, x.dtype)
        if x.data_ptr() != buf.data_ptr():
            _replay.copy_(buf, x)
        out = torch.empty((x.shape[0] // self.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        ch.bump()
        sm, blk = self._launch_shape(sm_num, block_size)
        st = KC.status_word(self.device)
        KC._check(self.lib.kb_reducescatter(self._bases_arr, self.rank, self.world, ch.flag_off, off, n // self.world,
                                            out.data_ptr(), ch.epoch, sm, blk, st.data_ptr(), KC._stream()),
                  "reducescatter")
        KC._count()
        return out

    def auto_tune(self, kind: str, shape, dtype=torch.bfloat16, sm_candidates=(4, 8, 12, 16, 24, 32),
                  block_candidates=(512, 1024), iters: int = 5):
        """Time a collective over a small grid of launch shapes and return ``(best (sm, block), table)``.
        Times are CUDA-event times, max over ranks (the reference's algorithm objects carry the same
        kind of ``auto_tune()`` candidate sweep: ``mscclpp_benchmark/mscclpp_op.py``)."""
        fn = {"all_reduce": self.all_reduce, "all_gather": self.all_gather, "reduce_scatter": self.reduce_scatter}[kind]
        x = torch.ones(shape, dtype=dtype, device=self.device)
        table = {}
        for sm in sm_candidates:
            for blk in block_candidates:
                fn(x, nb=0, sm_num=sm, block_size=blk, tag=f"__tune_{kind}")
                torch.cuda.synchronize(self.device)
                if self.world > 1:
                    dist.barrier(group=self.group)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(iters):
                    fn(x, nb=0, sm_num=sm, block_size=blk, tag=f"__tune_{kind}")
                b.record()
                torch.cuda.synchronize(self.device)
                t = torch.tensor([a.elapsed_time(b) / iters], device=self.device)
                if self.world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
                table[(sm, blk)] = float(t.item())
        best = min(table, key=table.get)
        return best, table

    def check_guards(self) -> None:
        """Raise if any kernel wrote into the canary words between heap buffers (synchronises)."""
        torch.cuda.synchronize(self.device)
        bad = self.guards.check(self.local)
        if bad:
            raise KC.KernelError("symmetric heap: canary words overwritten behind " + "; ".join(bad[:4]) +
                                 (f" (+{len(bad) - 4} more)" if len(bad) > 4 else ""))

    def wait_flag_probe(self, limit_ns: int = 200_000_000) -> None:
        """Launch a kernel that waits (bounded) on a flag nobody sets; the status word then holds the
        peer-timeout code.  Used to test the bounded-wait path without any peer."""
        ch = self.channel("__probe__")
        st = KC.status_word(self.device)
        slot = self.local_ptr + ch.flag_off
        KC._check(self.lib.kb_wait_flag(c_void_p(slot), 1 << 62, limit_ns, st.data_ptr(), KC._stream()), "wait_flag")

    def close(self, collective: bool = True) -> None:
        if self.closed:
            return
        self.closed = True
        if self.nvls is not None:
            self.nvls.close(collective)
            self.nvls = None
        torch.cuda.synchronize(self.device)
        for r, b in enumerate(self.bases):
            if r != self.rank:
                self.lib.kb_ipc_close(c_void_p(b))
        self.lib.kb_heap_free(c_void_p(self.local_ptr))
