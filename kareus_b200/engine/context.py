"""Per-nanobatch execution state: tensor store, operator contexts and stream events.

Role of the reference's ``kareus/megatron/core/partitions/context_manager.py:29-206`` and of
TransformerEngine's ``OperationContext`` (``transformer_engine/pytorch/ops/op.py:29-57``).  Each
tensor in the store can carry the CUDA event of the side-stream work that produced it, so the
consumer waits for exactly that work (and the engine can assert stream order) instead of relying
on one global synchronisation point.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch


class OpContext:
    """State an operator keeps between its forward and backward."""

    __slots__ = ("saved_tensors", "requires_grad", "needs_input_grad", "extra", "nb_index")

    def __init__(self, nb_index: int = 0):
        self.saved_tensors: Tuple[Optional[torch.Tensor], ...] = ()
        self.requires_grad: bool = True
        self.needs_input_grad: Tuple[bool, ...] = ()
        self.extra: Dict[str, Any] = {}
        self.nb_index = nb_index

    def save_for_backward(self, *tensors: Optional[torch.Tensor]) -> None:
        self.saved_tensors = tuple(tensors)

    def clear(self) -> None:
        self.saved_tensors = ()
        self.extra.clear()


class TensorStore:
    """``tensor_id -> tensor`` with optional producing events."""

    def __init__(self):
        self._t: Dict[str, torch.Tensor] = {}
        self._ev: Dict[str, Any] = {}

    def put(self, tid: str, tensor, event=None) -> None:
        self._t[tid] = tensor
        if event is not None:
            self._ev[tid] = event
        else:
            self._ev.pop(tid, None)

    def get(self, tid: str):
        if tid not in self._t:
            raise KeyError(f"tensor {tid} is not in the store (live: {sorted(self._t)[:8]}...)")
        return self._t[tid]

    def has(self, tid: str) -> bool:
        return tid in self._t

    def event(self, tid: str):
        return self._ev.get(tid)

    def clear_event(self, tid: str) -> None:
        self._ev.pop(tid, None)

    def pending_events(self) -> List[str]:
        return list(self._ev)

    def pop(self, tid: str):
        self._ev.pop(tid, None)
        return self._t.pop(tid, None)

    def clear(self) -> None:
        self._t.clear()
        self._ev.clear()

    def __len__(self) -> int:
        return len(self._t)

    def ids(self) -> List[str]:
        return list(self._t)


class NanoBatchContext:
    """Everything one nanobatch owns while a block executes."""

    def __init__(self, index: int):
        self.index = index
        self.store = TensorStore()
        self.op_ctx: Dict[int, OpContext] = {}
        self.ready_event: Dict[int, Any] = {}   # segment index -> event on the compute stream

    def ctx_for(self, op_id: int, create: bool = True) -> OpContext:
        c = self.op_ctx.get(op_id)
        if c is None:
            if not create:
                raise KeyError(f"no forward context saved for op {op_id} (nanobatch {self.index})")
            c = OpContext(self.index)
            self.op_ctx[op_id] = c
        return c

    def release_op(self, op_id: int) -> None:
        c = self.op_ctx.pop(op_id, None)
        if c is not None:
            c.clear()

    def saved_bytes(self) -> int:
        seen, total = set(), 0
        for c in self.op_ctx.values():
            for t in c.saved_tensors:
                if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    def reset(self) -> None:
        self.store.clear()
        for c in self.op_ctx.values():
            c.clear()
        self.op_ctx.clear()
        self.ready_event.clear()
