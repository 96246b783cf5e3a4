"""Graph nodes that run a GEMM fused with its sequence-parallel collective.

Forward: ``FusedAGGemm`` (all-gather → column-parallel GEMM) and ``FusedGemmRS`` (row-parallel GEMM
→ reduce-scatter).  Backward mirrors: ``FusedDgradRS`` (column-parallel dgrad → reduce-scatter, plus
the local wgrad) and ``FusedAGDgrad`` (all-gather of dY → row-parallel dgrad, plus the wgrad on the
gathered dY).  All four wrap the kernels of ``csrc/fused_gemm_comm.cu``.

To the partition engine they are collective nodes: they run on the side stream, take the plan
entry's ``sm_num`` and overlap with the other nanobatch's compute.  ``sm_num`` means copy-driver CTAs
for the all-gather kernels; for the reduce-scatter kernels it is the number of SMs the kernel leaves
to the other nanobatch, honoured only when a plan names it (``planned=True``) — without a plan they
use their whole SM budget.  They also produce the GEMM results, so the graph has no separate compute node for the linear layer.
State kept between forward and backward (the gathered input, or the row-parallel input) lives in the
linear operator's own context: these nodes share its graph uid.
"""
from __future__ import annotations

import os
import re
from ctypes import c_int, c_uint32, c_uint64, c_void_p

import torch

from .. import kernels as K
from ..engine.graph import operator_uid
from ..kernels import cuda as KC
from ..kernels import replay as _replay
from .basic import ensure_main_grad

_DECLARED = False


def _lib():
    global _DECLARED
    L = KC.lib()
    if not _DECLARED:
        P, I, U32, U64 = c_void_p, c_int, c_uint32, c_uint64
        L.kb_ag_gemm_bf16.argtypes = [P, I, I, U64, U64, P, P, I, I, I, I, I, P, U32, I, I, P, P]
        L.kb_ag_gemm_local_bf16.argtypes = [P, I, I, U64, U64, P, P, P, I, I, I, I, I, P, U32, I, I, P, P]
        L.kb_gemm_rs_bf16.argtypes = [P, I, I, U64, U64, U64, P, I, P, I, I, P, I, I, I, P, U32, I, I, P, P]
        L.kb_fused_tiles_n.argtypes = [I]
        L.kb_ag_gemm_mc_bf16.argtypes = [P, I, I, U64, P, P, U64, U64, P, P, I, I, I, I, I, U32, I, I, P, P]
        L.kb_gemm_rs_mc_bf16.argtypes = [P, I, I, U64, P, P, U64, U64, P, I, P, I, I, P, I, I, I, P, U32, I, I, P, P]
        for n in ("kb_ag_gemm_bf16", "kb_ag_gemm_local_bf16", "kb_gemm_rs_bf16", "kb_fused_tiles_n", "kb_ag_gemm_mc_bf16", "kb_gemm_rs_mc_bf16"):
            getattr(L, n).restype = c_int
        _DECLARED = True
    return L


def _fused_sms() -> int:
    """SMs a fused kernel may occupy (copy drivers + GEMM CTAs); 0 = all.  When the kernel is link
    bound, fewer GEMM CTAs lose nothing and leave SMs to the other nanobatch's compute."""
    n = int(os.environ.get("KAREUS_FUSED_SMS", "0"))
    from ..engine.program import _per_nb_streams
    if n == 0 and _per_nb_streams():
        # two fused kernels (one per nanobatch stream) must be able to be resident together on every
        # rank: if each may fill the GPU, ranks can start them in different orders and wait for each
        # other forever (the bounded waits then report a peer timeout)
        n = KC.sm_count() // 2
    return n


def _wgrad(dy2, x, weight) -> None:
    """``main_grad += dy2ᵀ·x``.  With one side stream per nanobatch two nanobatches' wgrads of the same
    weight could overlap and lose updates, so they are funnelled through one ordered stream; the block
    engine makes the compute stream wait for it at the end of backward."""
    from ..engine.program import _per_nb_streams, _shared_comm_stream, record_stream, wait_stream
    acc = ensure_main_grad(weight)
    if not (_per_nb_streams() and dy2.is_cuda):
        K.gemm(dy2, x, trans_a=True, trans_b=False, accumulate=acc)
        return
    cur = torch.cuda.current_stream(dy2.device)
    ws = _shared_comm_stream(dy2.device, slot=0)
    wait_stream(ws, cur)
    with torch.cuda.stream(ws):
        K.gemm(dy2, x, trans_a=True, trans_b=False, accumulate=acc)
    record_stream(dy2, ws)
    record_stream(x, ws)


class _FusedBase:
    needs_ctx = True
    takes_planned = True      # run() wants to know whether sm_num comes from a plan entry
    group = "linear"

    def __init__(self, linear, heap, default_sm: int):
        self.linear, self.heap, self.default_sm = linear, heap, default_sm
        self.name = linear.name + "." + type(self).__name__
        # one set of heap buffers per call site, shared by all layers (layers run one after another on
        # the ordered side stream)
        self.tag = re.sub(r"layers\.\d+\.", "", linear.name) + "/" + type(self).__name__
        self._graph_uid = operator_uid(linear)
        self._local = {}

    def _nvls(self):
        """The heap's NVLink-switch buffer when the multicast variants of the kernels are to be used
        (``SymmetricHeap.enable_nvls`` has run and ``KAREUS_FUSED_NVLS`` is not 0)."""
        nv = getattr(self.heap, "nvls", None)
        if nv is not None and os.environ.get("KAREUS_FUSED_NVLS", "1") != "0":
            return nv
        return None

    def _nvls_region(self, ch, name: str, nbytes: int) -> int:
        """Persistent region of this call site inside the NVLS buffer (same offset on every rank)."""
        cur = ch.buffers.get("nvls:" + name)
        if cur is None or cur[1] < nbytes:
            if cur is None and ch.epoch != 0 and not any(k.startswith("nvls:") for k in ch.buffers):
                # the ready flags of the multicast kernels count calls: they must start with the channel
                raise KC.KernelError(f"{self.name}: this call site already ran without multicast; enable the "
                                     "NVLS buffer before the first call")
            if cur is not None and name == "ready":
                raise KC.KernelError(f"{self.name}: the number of row tiles of a call site must not grow")
            cur = (self._nvls().region(nbytes), nbytes)
            ch.buffers["nvls:" + name] = cur
        return cur[0]

    def _local_flags(self, key, n):
        t = self._local.get(key)
        if t is None or t.numel() < n:
            t = torch.zeros(n, dtype=torch.int32, device=self.heap.device)
            self._local[key] = t
        return t

    # ---- kernels ------------------------------------------------------------------------------
    @staticmethod
    def auto_drivers(sm_num: int, n_out: int, budget: int = 0) -> int:
        """Copy-driver CTAs when no plan names them.  Every driver keeps a fixed number of bytes in flight, so
        the pull rate grows with their number; a kernel with little math (narrow N) can give up GEMM CTAs for
        drivers until its GEMM takes as long as the gather: three times the base count up to N = 768, twice
        up to N = 1280, never more than a third of the SMs the kernel may use (``budget``, 0: the whole GPU)."""
        cap = max(sm_num, (budget or 148) // 3)
        if n_out <= 768:
            return min(3 * sm_num, cap)
        if n_out <= 1280:
            return min(2 * sm_num, cap)
        return sm_num

    def _ag_gemm(self, x2, w, n_out, b_mn: bool, sm_num, nb: int, planned: bool = True, keep: bool = False):
        """Gather ``x2`` ([Ms, K] shard) over the group and multiply: returns ``(y [M, n_out], xg [M, K])``.
        ``xg`` is the gathered input inside the heap (valid until this site's next call), or with ``keep`` a
        tensor of its own that the caller may hold on to: the copy drivers then write the peers' shards
        straight into it, and only this rank's shard goes through the heap."""
        heap = self.heap
        self._xg_owned = False          # set by the branch that returns a tensor of its own
        sm_num = int(sm_num or self.default_sm)
        if not planned and os.environ.get("KAREUS_AG_AUTO", "1") != "0":
            sm_num = self.auto_drivers(sm_num, n_out, _fused_sms())
        world, rank = heap.world, heap.rank
        ms, k = x2.shape
        m = ms * world
        if ms % 128 or x2.dtype != torch.bfloat16:
            raise KC.KernelError(f"fused all-gather GEMM needs bf16 and a multiple of 128 rows per rank, got {ms}")
        ch = heap.channel(f"{self.tag}/{nb}")
        nv = self._nvls()
        if nv is not None:
            # multicast variant: the drivers push this rank's shard through the switch into every rank's
            # gathered buffer; flags and data live in the NVLS buffer
            off = self._nvls_region(ch, "xg", m * k * 2)
            roff = self._nvls_region(ch, "ready", (m // 128) * 4)
            xg = nv.view(off, (m, k), torch.bfloat16)
            _replay.copy_(xg[rank * ms:(rank + 1) * ms], x2 if x2.is_contiguous() else x2.contiguous())
            ch.bump()
            y = torch.empty(m, n_out, dtype=torch.bfloat16, device=x2.device)
            st = KC.status_word(x2.device)
            rc = _lib().kb_ag_gemm_mc_bf16(heap._bases_arr, rank, world, ch.flag_off, c_void_p(nv.uc_ptr),
                                           c_void_p(nv.mc_ptr), off, roff, w.data_ptr(), y.data_ptr(), m, n_out, k,
                                           w.stride(0), 1 if b_mn else 0, ch.epoch, int(sm_num or self.default_sm),
                                           _fused_sms(), st.data_ptr(), KC._stream())
            KC._check(rc, f"ag_gemm (multicast) {self.name}")
            KC._count()
            return y, xg
        if keep and os.environ.get("KAREUS_AG_KEEP", "1") != "0":
            off, _ = heap.buffer(ch, "xs", ms * k * 2)
            x2c = x2 if x2.is_contiguous() else x2.contiguous()
            xg = torch.empty(m, k, dtype=torch.bfloat16, device=x2.device)
            _replay.copy_(heap.view(off, (ms, k), torch.bfloat16), x2c)      # what the peers pull
            _replay.copy_(xg[rank * ms:(rank + 1) * ms], x2c)
            ready = self._local_flags(("ready", nb), m // 128)
            ch.bump()
            y = torch.empty(m, n_out, dtype=torch.bfloat16, device=x2.device)
            st = KC.status_word(x2.device)
            rc = _lib().kb_ag_gemm_local_bf16(heap._bases_arr, rank, world, ch.flag_off, off, xg.data_ptr(),
                                              w.data_ptr(), y.data_ptr(), m, n_out, k, w.stride(0), 1 if b_mn else 0,
                                              ready.data_ptr(), ch.epoch, int(sm_num or self.default_sm),
                                              _fused_sms(), st.data_ptr(), KC._stream())
            KC._check(rc, f"ag_gemm {self.name}")
            KC._count()
            self._xg_owned = True
            return y, xg
        off, _ = heap.buffer(ch, "xg", m * k * 2)
        xg = heap.view(off, (m, k), torch.bfloat16)
        _replay.copy_(xg[rank * ms:(rank + 1) * ms], x2 if x2.is_contiguous() else x2.contiguous())
        ready = self._local_flags(("ready", nb), m // 128)
        ch.bump()
        y = torch.empty(m, n_out, dtype=torch.bfloat16, device=x2.device)
        st = KC.status_word(x2.device)
        rc = _lib().kb_ag_gemm_bf16(heap._bases_arr, rank, world, ch.flag_off, off, w.data_ptr(), y.data_ptr(), m,
                                    n_out, k, w.stride(0), 1 if b_mn else 0, ready.data_ptr(), ch.epoch,
                                    int(sm_num or self.default_sm), _fused_sms(), st.data_ptr(), KC._stream())
        KC._check(rc, f"ag_gemm {self.name}")
        KC._count()
        return y, xg

    def _gemm_rs(self, a2, w, n_out, b_mn: bool, sm_num, nb: int):
        """``reduce_scatter_rows(a2 · op(w))`` → ``[M/world, n_out]``.  ``sm_num``: SMs left free."""
        heap = self.heap
        world, rank = heap.world, heap.rank
        if not KC._rowmajor_ok(a2):
            _replay.require_recordable("making a GEMM operand contiguous")
            a2 = a2.contiguous()
        m, k = a2.shape
        ms = m // world
        if m % (world * 128) or a2.dtype != torch.bfloat16:
            raise KC.KernelError(f"fused GEMM reduce-scatter needs bf16 and rows divisible by {world * 128}, got {m}")
        L = _lib()
        tiles_n = L.kb_fused_tiles_n(n_out)
        ch = heap.channel(f"{self.tag}/{nb}")
        nv = self._nvls()
        if nv is not None:
            # multicast variant: partial tiles stay in local staging; each rank fetches its own rows summed
            # over all ranks by the switch
            stage_off = self._nvls_region(ch, "stage", m * n_out * 2)
            cnt_off, _ = heap.buffer(ch, "cnt", world * (ms // 128) * tiles_n * 4)
            go = self._local_flags(("go", nb), 1)
            ch.bump()
            out = torch.empty(ms, n_out, dtype=torch.bfloat16, device=a2.device)
            st = KC.status_word(a2.device)
            rc = L.kb_gemm_rs_mc_bf16(heap._bases_arr, rank, world, ch.flag_off, c_void_p(nv.uc_ptr), c_void_p(nv.mc_ptr),
                                      stage_off, cnt_off, a2.data_ptr(), a2.stride(0), w.data_ptr(), w.stride(0),
                                      1 if b_mn else 0, out.data_ptr(), m, n_out, k, go.data_ptr(), ch.epoch,
                                      int(sm_num or 0), _fused_sms(), st.data_ptr(), KC._stream())
            KC._check(rc, f"gemm_rs (multicast) {self.name}")
            KC._count()
            return out, a2
        stage_off, _ = heap.buffer(ch, "stage", m * n_out * 2)
        cnt_off, _ = heap.buffer(ch, "cnt", world * (ms // 128) * tiles_n * 4)
        go = self._local_flags(("go", nb), 1)
        ch.bump()
        out = torch.empty(ms, n_out, dtype=torch.bfloat16, device=a2.device)
        st = KC.status_word(a2.device)
        rc = L.kb_gemm_rs_bf16(heap._bases_arr, rank, world, ch.flag_off, stage_off, cnt_off, a2.data_ptr(),
                               a2.stride(0), w.data_ptr(), w.stride(0), 1 if b_mn else 0, out.data_ptr(), m, n_out, k,
                               go.data_ptr(), ch.epoch, int(sm_num or 0), _fused_sms(), st.data_ptr(),
                               KC._stream())
        KC._check(rc, f"gemm_rs {self.name}")
        KC._count()
        return out, a2


class FusedAGGemm(_FusedBase):
    """forward of a column-parallel layer: ``Y = AllGather(x)·Wᵀ``."""

    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None, planned=False):
        (x,) = tensors
        lin = self.linear
        lead = x.shape[:-1]
        keep = ctx is not None and ctx.requires_grad       # the wgrad GEMM of the backward pass reads xg
        y, xg = self._ag_gemm(x.reshape(-1, x.shape[-1]), lin.weight, lin.out_features, False, sm_num, nb, planned,
                              keep=keep)
        if keep:
            # a buffer of the call site (heap or NVLS buffer) is overwritten by the next layer: copy it out
            ctx.save_for_backward(xg if self._xg_owned else _replay.clone(xg))
        return (y.reshape((lead[0] * self.heap.world,) + tuple(lead[1:]) + (lin.out_features,)),)


class FusedGemmRS(_FusedBase):
    """forward of a row-parallel layer: ``Y_shard = ReduceScatter(a·Wᵀ)``."""

    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None, planned=False):
        (a,) = tensors
        lin = self.linear
        lead = a.shape[:-1]
        out, a2 = self._gemm_rs(a.reshape(-1, a.shape[-1]), lin.weight, lin.out_features, False,
                                sm_num if planned else 0, nb)
        if ctx is not None and ctx.requires_grad:
            ctx.save_for_backward(a2)
        return (out.reshape((lead[0] // self.heap.world,) + tuple(lead[1:]) + (lin.out_features,)),)


class FusedDgradRS(_FusedBase):
    """backward of a column-parallel layer: ``dX_shard = ReduceScatter(dY·W)`` and ``dW += dYᵀ·X``."""

    releases_ctx = True       # last user of the layer's saved input: the engine drops it afterwards

    def run(self, tensors, sm_num=None, block_size=None, backward=True, nb=0, ctx=None, planned=False):
        (dy,) = tensors
        lin = self.linear
        (x_full,) = ctx.saved_tensors
        lead = dy.shape[:-1]
        dx, dy2 = self._gemm_rs(dy.reshape(-1, dy.shape[-1]), lin.weight, lin.in_features, True,
                                sm_num if planned else 0, nb)
        _wgrad(dy2, x_full, lin.weight)
        return (dx.reshape((lead[0] // self.heap.world,) + tuple(lead[1:]) + (lin.in_features,)),)


class FusedAGDgrad(_FusedBase):
    """backward of a row-parallel layer: ``dX = AllGather(dY)·W`` and ``dW += AllGather(dY)ᵀ·A``."""

    releases_ctx = True

    def run(self, tensors, sm_num=None, block_size=None, backward=True, nb=0, ctx=None, planned=False):
        (dy,) = tensors
        lin = self.linear
        (a2,) = ctx.saved_tensors
        lead = dy.shape[:-1]
        dx, dyg = self._ag_gemm(dy.reshape(-1, dy.shape[-1]), lin.weight, lin.in_features, True, sm_num, nb, planned)
        _wgrad(dyg, a2, lin.weight)
        if dyg.is_cuda:
            # `dyg` lives in this call site's heap buffer, which the site's next call overwrites: when
            # the weight-gradient GEMM was moved to the ordered stream, this stream must not run ahead
            from ..engine.program import _per_nb_streams, _shared_comm_stream, wait_stream
            if _per_nb_streams():
                wait_stream(torch.cuda.current_stream(dyg.device), _shared_comm_stream(dyg.device, slot=0))
        return (dx.reshape((lead[0] * self.heap.world,) + tuple(lead[1:]) + (lin.in_features,)),)


def attach_fused(layer, heap, default_sm: int = 16) -> None:
    """Give the four linear layers of a transformer layer their fused forward and backward nodes."""
    for lin in (layer.qkv, layer.fc1):
        lin.fused_ag_gemm = FusedAGGemm(lin, heap, default_sm)
        lin.fused_dgrad_rs = FusedDgradRS(lin, heap, default_sm)
    for lin in (layer.proj, layer.fc2):
        lin.fused_gemm_rs = FusedGemmRS(lin, heap, default_sm)
        lin.fused_ag_dgrad = FusedAGDgrad(lin, heap, default_sm)
