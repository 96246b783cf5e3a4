"""Another GPU's memory never reaches a vendor-library or PyTorch kernel.

Peer views of the symmetric heap may only be read by this package's own kernels.  These tests run on
CPU: they drive the dispatch layers with stand-ins and check that every route from a peer-memory
call to a library refuses, and that collectives are bound to the heap of their own process group.
"""
import types

import pytest
import torch

import kareus_b200.kernels as K
from kareus_b200.kernels import attention_bwd_native, attention_native
from kareus_b200.kernels import cuda as KC
from kareus_b200.parallel.collectives import AllGatherKV, AllReduce, CommFactory, ReduceScatterKV
from kareus_b200.parallel.ring_attention import RingAttention
from kareus_b200.parallel.symm_heap import SymmetricHeap


class _Trap:
    """Stands in for ``kareus_b200.kernels.cuda``: any library or reference route is an error."""

    KernelError = KC.KernelError

    def __init__(self):
        self.native_calls = 0

    def attention_fwd_library(self, *a, **k):
        raise AssertionError("library attention reached with peer operands")

    attention_bwd_library = attention_fwd_library

    def attention_fwd(self, *a, strict=False, **k):
        assert strict, "peer call must be strict"
        self.native_calls += 1
        return "native"

    attention_bwd = attention_fwd


def _qkv(d=128, dtype=torch.bfloat16):
    q = torch.zeros(8, 1, 2, d, dtype=dtype)
    k = torch.zeros(8, 1, 2, d, dtype=dtype)
    return q, k, k.clone()


def test_peer_call_needs_cuda_tensors():
    q, k, v = _qkv()
    with pytest.raises(KC.KernelError):
        K.attention_fwd(q, k, v, 1.0, peer=True)
    with pytest.raises(KC.KernelError):
        K.attention_bwd(q, q, k, v, q, None, 1.0, peer=True)


def test_peer_call_refused_under_library_baseline(monkeypatch):
    trap = _Trap()
    monkeypatch.setattr(K, "is_cuda", lambda t: True)
    monkeypatch.setattr(K, "_cuda", lambda: trap)
    q, k, v = _qkv()
    assert K.attention_fwd(q, k, v, 1.0, peer=True) == "native"
    assert K.attention_bwd(q, q, k, v, q, None, 1.0, peer=True) == "native"
    monkeypatch.setenv("KAREUS_B200_LIBRARY_BASELINE", "1")
    with pytest.raises(KC.KernelError):
        K.attention_fwd(q, k, v, 1.0, peer=True)
    with pytest.raises(KC.KernelError):
        K.attention_bwd(q, q, k, v, q, None, 1.0, peer=True)
    assert trap.native_calls == 2


def test_strict_call_refuses_other_dtypes():
    q, k, v = _qkv(dtype=torch.float32)
    with pytest.raises(KC.KernelError):
        KC.attention_fwd(q, k, v, 1.0, strict=True)
    with pytest.raises(KC.KernelError):
        KC.attention_bwd(q, q, k, v, q, None, 1.0, strict=True)


@pytest.mark.parametrize("case", ["head_dim", "stride"])
def test_strict_call_refuses_shapes_the_native_kernels_do_not_cover(monkeypatch, case):
    def boom(*a, **k):
        raise AssertionError("library attention reached")

    monkeypatch.setattr(KC, "attention_fwd_library", boom)
    monkeypatch.setattr(KC, "attention_bwd_library", boom)
    monkeypatch.setenv("KAREUS_B200_ATTENTION_FALLBACK", "1")      # the opt-in must not open strict calls
    if case == "head_dim":
        q, k, v = _qkv(d=64)
    else:
        q, k, v = _qkv()
        k = torch.zeros(8, 1, 2, 132, dtype=torch.bfloat16)[..., 4:]   # rows start 8 bytes off alignment
    with pytest.raises(KC.KernelError):
        attention_native.forward(q, k, v, 1.0, strict=True)
    with pytest.raises(KC.KernelError):
        attention_bwd_native.backward(q, q, k, v, q, None, 1.0, strict=True)


def test_plain_call_needs_the_opt_in_to_leave_the_native_kernels(monkeypatch):
    monkeypatch.delenv("KAREUS_B200_ATTENTION_FALLBACK", raising=False)
    q, k, v = _qkv(d=64)
    with pytest.raises(KC.KernelError, match="KAREUS_B200_ATTENTION_FALLBACK"):
        attention_native.forward(q, k, v, 1.0)
    monkeypatch.setenv("KAREUS_B200_ATTENTION_FALLBACK", "1")
    monkeypatch.setattr(KC, "attention_fwd_library", lambda *a, **kw: "wheel")
    assert attention_native.forward(q, k, v, 1.0) == "wheel"


class _FakeHeap:
    def __init__(self, world, rank):
        self.world, self.rank = world, rank


class _FakeCuda:
    """Tensor stand-in that claims to be on a GPU."""
    is_cuda = True

    def __init__(self, dtype=torch.bfloat16):
        self.dtype = dtype


def test_ring_publication_refused_under_library_baseline_and_for_other_dtypes(monkeypatch):
    ring = RingAttention(None, 2, 0, heap=_FakeHeap(2, 0))
    monkeypatch.setenv("KAREUS_B200_LIBRARY_BASELINE", "1")
    with pytest.raises(KC.KernelError, match="LIBRARY_BASELINE"):
        ring._publish(_FakeCuda(), _FakeCuda(), 0, "fwd")
    monkeypatch.delenv("KAREUS_B200_LIBRARY_BASELINE")
    with pytest.raises(KC.KernelError, match="bf16"):
        ring._publish(_FakeCuda(torch.float32), _FakeCuda(torch.float32), 0, "fwd")
    assert ring._peer(_FakeCuda()) is True


def test_heap_hands_out_no_peer_view_under_library_baseline(monkeypatch):
    heap = SymmetricHeap.__new__(SymmetricHeap)
    heap.rank, heap.world = 0, 2
    monkeypatch.setenv("KAREUS_B200_LIBRARY_BASELINE", "1")
    with pytest.raises(KC.KernelError):
        heap.peer_view(1, 0, (4,), torch.bfloat16)


def test_heap_collectives_refuse_other_dtypes():
    heap = SymmetricHeap.__new__(SymmetricHeap)
    for fn in (heap.all_reduce, heap.all_gather, heap.reduce_scatter):
        with pytest.raises(KC.KernelError, match="bf16"):
            fn(torch.zeros(8, dtype=torch.float32))


def test_collectives_get_the_heap_of_their_own_group():
    mesh = types.SimpleNamespace(group=lambda a: None, size=lambda a: {"tp": 4, "cp": 2}[a],
                                 axis_rank=lambda a: {"tp": 3, "cp": 1}[a])
    tp_heap, cp_heap = _FakeHeap(4, 3), _FakeHeap(2, 1)
    f = CommFactory(mesh, "kernel", heap=tp_heap, heap_cp=cp_heap)
    assert f.make(AllReduce, "tp", "x").heap is tp_heap
    assert f.make(AllGatherKV, "cp", "kv").heap is cp_heap
    assert f.make(ReduceScatterKV, "cp", "dkv").heap is cp_heap
    # without a context-parallel heap the CP collectives use torch.distributed, never the TP heap
    g = CommFactory(mesh, "kernel", heap=tp_heap)
    op = g.make(AllGatherKV, "cp", "kv")
    assert op.heap is None and not op._use_kernel(torch.zeros(1), 8)
    with pytest.raises(ValueError, match="spans"):
        AllGatherKV(None, 2, 1, backend="kernel", heap=tp_heap, name="kv")


class _CudaClaim(torch.Tensor):
    """A CPU tensor that answers ``is_cuda`` with True, to drive predicates that look at it."""

    @property
    def is_cuda(self):
        return True


def test_kernel_backend_is_bf16_only():
    op = AllReduce(None, 2, 0, backend="kernel", heap=_FakeHeap(2, 0))
    bf = torch.zeros(1, dtype=torch.bfloat16).as_subclass(_CudaClaim)
    assert op._use_kernel(bf, 8)
    assert not op._use_kernel(bf, None)                 # no launch shape: library call
    for dt in (torch.float32, torch.float64, torch.float16):
        assert not op._use_kernel(torch.zeros(1, dtype=dt).as_subclass(_CudaClaim), 8)


def test_guard_words_between_heap_buffers_name_the_overrun():
    from kareus_b200.parallel.symm_heap import GUARD_BYTES, GuardMap
    heap = torch.zeros(16384, dtype=torch.uint8)
    g = GuardMap()
    for i, (off, n) in enumerate([(1024, 3000), (6144, 2048)]):
        end = (off + n + 15) // 16 * 16
        g.paint(heap, end, GUARD_BYTES)
        g.add(end, GUARD_BYTES, f"buffer {i}")
    heap[1024:1024 + 3000] = 7                      # writing inside a buffer is fine
    assert g.check(heap) == []
    heap[6144 + 2048 + 5] = 1                       # one byte past the end of buffer 1
    assert g.check(heap) == ["buffer 1"]


def _node_worker(rank, world):
    from kareus_b200.parallel import symm_heap
    import pytest as _pytest
    symm_heap.require_one_node(None, world)                       # both ranks on this machine: fine
    real = symm_heap.node_identity
    symm_heap.node_identity = lambda: f"node{rank}/boot"          # pretend the ranks sit on two machines
    try:
        with _pytest.raises(RuntimeError, match="different machines"):
            symm_heap.require_one_node(None, world)
    finally:
        symm_heap.node_identity = real


def test_peer_memory_groups_must_stay_inside_one_node():
    from dist_utils import run_distributed
    run_distributed(_node_worker, 2)
