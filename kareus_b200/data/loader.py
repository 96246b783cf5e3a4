"""Per-step batches of one data-parallel rank, read ahead of the training loop by a host thread.

Sample order follows Megatron's pretraining sampler (``megatron/legacy/data/data_samplers.py``,
``MegatronPretrainingSampler``): the global stream of samples is consumed in blocks of
``micro_batch x dp`` and rank ``r`` takes rows ``[r*micro_batch, (r+1)*micro_batch)`` of every block, so
a run resumes from ``consumed_samples`` alone and any data-parallel size sees the same global batches.
"""
from __future__ import annotations

import queue
import threading
from typing import Dict, Iterator, Optional

import torch


class PretrainingBatches:
    """``next()`` → ``{"tokens", "labels", "loss_mask"}`` with ``num_microbatches * micro_batch`` rows (host
    tensors, pinned when CUDA is there), the layout ``Trainer.train_step`` takes."""

    def __init__(self, dataset, micro_batch_size: int, num_microbatches: int, dp_rank: int = 0, dp_size: int = 1,
                 consumed_samples: int = 0, cp: int = 1, cp_rank: int = 0, pin: Optional[bool] = None,
                 prefetch: int = 2):
        if not (0 <= dp_rank < dp_size):
            raise ValueError(f"dp_rank {dp_rank} outside 0..{dp_size}")
        self.dataset = dataset
        self.mbs, self.num_mb, self.dp_rank, self.dp_size = micro_batch_size, num_microbatches, dp_rank, dp_size
        self.global_batch = micro_batch_size * num_microbatches * dp_size
        if consumed_samples % self.global_batch:
            raise ValueError(f"consumed_samples {consumed_samples} is not a multiple of the global batch "
                             f"{self.global_batch}")
        self.consumed_samples = consumed_samples
        self.cp, self.cp_rank = cp, cp_rank
        self.pin = torch.cuda.is_available() if pin is None else pin
        self._q: "queue.Queue" = queue.Queue(maxsize=max(1, prefetch))
        self._stop = threading.Event()
        self._next_to_read = consumed_samples
        self._thread = threading.Thread(target=self._worker, name="kareus-data", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ index arithmetic
    def sample_ids(self, consumed: int):
        """Global sample ids of this rank's rows of the step that starts at ``consumed``."""
        block = self.mbs * self.dp_size
        return [consumed + m * block + self.dp_rank * self.mbs + j for m in range(self.num_mb) for j in range(self.mbs)]

    def steps_left(self) -> int:
        return (len(self.dataset) - self.consumed_samples) // self.global_batch

    # ------------------------------------------------------------------ reading
    def _assemble(self, consumed: int) -> Dict[str, torch.Tensor]:
        rows = [self.dataset[i] for i in self.sample_ids(consumed)]
        out = {k: torch.stack([r[k] for r in rows]) for k in ("tokens", "labels", "loss_mask")}
        if self.cp > 1:
            from ..parallel.collectives import dual_chunk_ids
            s = out["tokens"].shape[1]
            c = s // (2 * self.cp)
            a, b = dual_chunk_ids(self.cp, self.cp_rank)
            idx = torch.cat([torch.arange(a * c, (a + 1) * c), torch.arange(b * c, (b + 1) * c)])
            out = {k: v[:, idx].contiguous() for k, v in out.items()}
        if self.pin:
            out = {k: v.pin_memory() for k, v in out.items()}
        return out

    def _worker(self) -> None:
        try:
            while not self._stop.is_set():
                if self._next_to_read + self.global_batch > len(self.dataset):
                    self._put(StopIteration())
                    return
                item = self._assemble(self._next_to_read)
                self._next_to_read += self.global_batch
                if not self._put(item):
                    return
        except BaseException as e:           # handed to the consumer, which re-raises it
            self._put(e)

    def _put(self, item) -> bool:
        while not self._stop.is_set():
            try:
                self._q.put(item, timeout=0.2)
                return True
            except queue.Full:
                continue
        return False

    # ------------------------------------------------------------------ iteration
    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        item = self._q.get()
        if isinstance(item, StopIteration):
            self._q.put(item)                 # stay exhausted
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        self.consumed_samples += self.global_batch
        return item

    def close(self) -> None:
        self._stop.set()
        try:
            while True:
                self._q.get_nowait()
        except queue.Empty:
            pass
        self._thread.join(timeout=5.0)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
