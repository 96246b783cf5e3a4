"""Non-interleaved 1F1B pipeline schedule over point-to-point sends/receives.

Instruction order per stage (reference ``3rdparty/Megatron-LM/megatron/core/pipeline_parallel/
schedules.py:1775-2085``): ``min(pp - rank - 1, M)`` warm-up forwards, ``M - warmup`` steady
forward/backward pairs, then the cool-down backwards.  That order is also the order of the
entries of a stage in ``freqs_pipeline_*.py`` / ``scheds_pipeline_*.py``.

Transfers are batched like Megatron's (a send and the matching receive of the opposite direction go
into one ``batch_isend_irecv``, which keeps neighbouring stages' pairs matched and the schedule
deadlock free) but never block the host: waiting on a receive only orders the compute stream after
the NCCL stream, sends are completed at the end of the step, so the transfers run under the compute
that is already enqueued (the reference only removes a ``cuda.synchronize`` after its blocking p2p
calls: ``p2p_communication.py:401-412``).  The message is the list of nanobatch tensors of one
microbatch, ``[s/cp(/tp), mbs/N, h]`` each.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def one_f_one_b_order(pp: int, pp_rank: int, num_microbatches: int) -> List[Tuple[str, int]]:
    """``[('forward', mb), ('backward', mb), ...]`` in this stage's execution order."""
    warm = min(pp - pp_rank - 1, num_microbatches)
    out: List[Tuple[str, int]] = [("forward", i) for i in range(warm)]
    f, b = warm, 0
    for _ in range(num_microbatches - warm):
        out.append(("forward", f))
        f += 1
        out.append(("backward", b))
        b += 1
    while b < num_microbatches:
        out.append(("backward", b))
        b += 1
    return out


class P2PStats:
    """How long the compute stream stood still for pipeline receives.

    A pair of CUDA events brackets every receive wait on the compute stream; their distance is the
    time the stream could not run because the data (or the neighbour stage that produces it) was not
    there yet — transfer time that compute did not hide plus pipeline bubble.  ``summary()``
    synchronises and returns totals; the engine never reads it on its own."""

    def __init__(self):
        self.pairs = []
        self.bytes = 0

    def bracket(self, reqs, tensors):
        if not reqs or not tensors or not tensors[0].is_cuda:
            for r in reqs:
                r.wait()
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for r in reqs:
            r.wait()
        b.record()
        self.pairs.append((a, b))
        self.bytes += sum(t.numel() * t.element_size() for t in tensors)

    def summary(self, reset: bool = True) -> dict:
        if self.pairs:
            torch.cuda.synchronize()
        out = {"receives": len(self.pairs), "stall_ms": sum(a.elapsed_time(b) for a, b in self.pairs),
               "received_bytes": self.bytes}
        if reset:
            self.pairs, self.bytes = [], 0
        return out


class _Pending:
    def __init__(self, tensors, reqs, stats: Optional[P2PStats] = None):
        self.tensors, self.reqs, self.stats = tensors, reqs, stats

    def wait(self):
        if self.stats is not None and self.tensors is not None:
            self.stats.bracket(self.reqs, self.tensors)
        else:
            for r in self.reqs:
                r.wait()
        self.reqs = []
        return self.tensors


class P2P:
    """Asynchronous neighbour exchange of lists of tensors with known shapes."""

    def __init__(self, mesh, shapes: Sequence[Tuple[int, ...]], dtype, device):
        self.mesh = mesh
        self.shapes, self.dtype, self.device = [tuple(s) for s in shapes], dtype, device
        self.prev = mesh.pp_neighbor(-1) if not mesh.is_first_stage else None
        self.next = mesh.pp_neighbor(+1) if not mesh.is_last_stage else None
        self.group = mesh.group("pp")
        self._sends: List[_Pending] = []
        self.stats: Optional[P2PStats] = None          # set to a P2PStats() to measure receive stalls

    def _bufs(self):
        return [torch.empty(s, dtype=self.dtype, device=self.device) for s in self.shapes]

    def _post(self, ops):
        if not ops:
            return []
        return dist.batch_isend_irecv(ops)

    def exchange(self, send: Optional[Sequence[torch.Tensor]] = None, send_to: Optional[int] = None,
                 recv_from: Optional[int] = None) -> Optional[_Pending]:
        """Post one batch with an optional send and an optional receive (a combined batch keeps
        neighbouring stages' send/recv pairs matched, which is what makes 1F1B deadlock free).
        Returns the pending receive, whose ``wait()`` orders the compute stream after the data."""
        ops, keep, bufs = [], None, None
        if send is not None and send_to is not None:
            keep = [t.detach().contiguous() for t in send]
            ops += [dist.P2POp(dist.isend, t, send_to, self.group) for t in keep]
        if recv_from is not None:
            bufs = self._bufs()
            ops += [dist.P2POp(dist.irecv, b, recv_from, self.group) for b in bufs]
        reqs = self._post(ops)
        if keep is not None:
            self._sends.append(_Pending(keep, reqs if bufs is None else []))
        return _Pending(bufs, reqs, self.stats) if bufs is not None else None

    def finish_sends(self) -> None:
        for p in self._sends:
            p.wait()
        self._sends.clear()


class PipelineSchedule:
    """Runs one training step of ``num_microbatches`` through this stage.

    ``forward_fn(mb, inputs) -> outputs`` gets the received hidden-state list (``None`` on the
    first stage) and returns the list to send on (or the scalar loss on the last stage).
    ``hooks`` receive ``on_instruction_begin/end(name)`` (frequency controller, comm scheduler).
    """

    def __init__(self, mesh, p2p: Optional[P2P], forward_fn: Callable, hooks: Sequence[object] = ()):
        self.mesh, self.p2p, self.forward_fn, self.hooks = mesh, p2p, forward_fn, list(hooks)

    def _begin(self, name):
        for h in self.hooks:
            h.on_instruction_begin(name)

    def _end(self, name):
        for h in self.hooks:
            h.on_instruction_end(name)

    def run_forward_only(self, num_microbatches: int) -> List[torch.Tensor]:
        """Evaluation: every microbatch goes forward through the stages, nothing comes back.  Returns the
        per-microbatch losses on the last stage (empty elsewhere).  The caller disables autograd."""
        mesh, p2p = self.mesh, self.p2p
        first, last = mesh.is_first_stage, mesh.is_last_stage
        losses: List[torch.Tensor] = []
        for mb in range(num_microbatches):
            inputs = None if first else list(p2p.exchange(recv_from=p2p.prev).wait())
            self._begin("forward")
            out = self.forward_fn(mb, inputs)
            self._end("forward")
            if last:
                losses.append(out.detach())
            else:
                p2p.exchange(send=list(out), send_to=p2p.next)
        if p2p is not None:
            p2p.finish_sends()
        return losses

    def run(self, num_microbatches: int) -> List[torch.Tensor]:
        mesh, p2p = self.mesh, self.p2p
        first, last = mesh.is_first_stage, mesh.is_last_stage
        M = num_microbatches
        warm = min(mesh.pp - mesh.pp_rank - 1, M)
        steady = M - warm
        losses: List[torch.Tensor] = []
        saved = {}                                   # mb -> (inputs, outputs)
        fwd_mb, bwd_mb = 0, 0

        def recv_forward():
            if first:
                return None
            return [t.requires_grad_(True) for t in p2p.exchange(recv_from=p2p.prev).wait()]

        def forward(inputs):
            nonlocal fwd_mb
            mb = fwd_mb
            fwd_mb += 1
            self._begin("forward")
            out = self.forward_fn(mb, inputs)
            if last:
                losses.append(out.detach())
                saved[mb] = (inputs, [out])
            else:
                saved[mb] = (inputs, list(out))
            self._end("forward")
            return out

        def backward(grads):
            nonlocal bwd_mb
            mb = bwd_mb
            bwd_mb += 1
            self._begin("backward")
            inputs, outputs = saved.pop(mb)
            if last:
                torch.autograd.backward(outputs)
            else:
                torch.autograd.backward(outputs, grads)
            self._end("backward")
            return None if first else [t.grad for t in inputs]

        for _ in range(warm):
            out = forward(recv_forward())
            p2p.exchange(send=out, send_to=p2p.next)
        inputs = recv_forward() if steady > 0 else None
        for i in range(steady):
            out = forward(inputs)
            grads = None
            if not last:
                grads = p2p.exchange(send=out, send_to=p2p.next, recv_from=p2p.next).wait()
            in_grads = backward(grads)
            if i == steady - 1:
                inputs = None
                if not first:
                    p2p.exchange(send=in_grads, send_to=p2p.prev)
            elif not first:
                inputs = [t.requires_grad_(True) for t in
                          p2p.exchange(send=in_grads, send_to=p2p.prev, recv_from=p2p.prev).wait()]
            else:
                inputs = None
        for _ in range(warm):
            grads = p2p.exchange(recv_from=p2p.next).wait()
            in_grads = backward(grads)
            if not first:
                p2p.exchange(send=in_grads, send_to=p2p.prev)
        if p2p is not None:
            p2p.finish_sends()
        return losses
