"""Host-side failure detection between training steps.

Every rank publishes the last step it *finished* in the rendezvous store; before launching the next
step a rank checks that all peers finished the previous one within ``timeout_s``.  A rank that died
or stalled is therefore noticed on the host, before any kernel or collective that would wait for it
is launched (device-side waits are bounded as a second line of defence and report a status code).
The reference has no such mechanism: its device-side spins assert (trap the GPU) when their limit
is hit (``3rdparty/mscclpp/include/mscclpp/poll_device.hpp:12-18``).
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    def __init__(self, missing: List[int], step: int):
        super().__init__(f"ranks {missing} did not finish step {step}")
        self.missing, self.step = missing, step


class Heartbeat:
    def __init__(self, store=None, rank: Optional[int] = None, world: Optional[int] = None, prefix: str = "kareus/hb",
                 timeout_s: float = 30.0, poll_s: float = 0.05):
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix, self.timeout_s, self.poll_s = prefix, timeout_s, poll_s

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def finished(self, step: int) -> None:
        self.store.set(self._key(self.rank), str(step))

    def _read(self, r: int) -> int:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return -1
            return int(self.store.get(self._key(r)))
        except Exception:
            return -1

    def check(self, step: int) -> None:
        """Raise :class:`RankFailure` unless every peer has finished ``step`` within the timeout."""
        deadline = time.monotonic() + self.timeout_s
        missing = list(range(self.world))
        while True:
            missing = [r for r in missing if r != self.rank and self._read(r) < step]
            if not missing:
                return
            if time.monotonic() > deadline:
                raise RankFailure(missing, step)
            time.sleep(self.poll_s)
