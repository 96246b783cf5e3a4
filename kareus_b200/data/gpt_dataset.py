"""Fixed-length language-model samples over an indexed token file.

What the reference gets from Megatron's ``GPTDataset``
(``3rdparty/Megatron-LM/megatron/core/datasets/gpt_dataset.py``): documents are shuffled per epoch and laid
end to end, the stream is cut every ``seq_len`` tokens, a sample is ``seq_len + 1`` consecutive tokens
(``tokens = sample[:-1]``, ``labels = sample[1:]``, so neighbouring samples share one token), and the
samples are visited in a shuffled order.  Everything is a pure function of ``(files, seq_len, num_samples,
seed, document range)``, so every rank builds the same index and a resumed run continues where it stopped.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import torch

from .indexed import IndexedDataset


def split_documents(num_documents: int, weights: Sequence[float]) -> Tuple[Tuple[int, int], ...]:
    """Contiguous document ranges for e.g. ``(949, 50, 1)`` → train / validation / test."""
    w = np.asarray(weights, dtype=np.float64)
    if (w < 0).any() or w.sum() <= 0:
        raise ValueError(f"bad split weights {weights}")
    bounds = np.concatenate([[0], np.round(np.cumsum(w) / w.sum() * num_documents).astype(np.int64)])
    bounds[-1] = num_documents
    return tuple((int(bounds[i]), int(bounds[i + 1])) for i in range(len(w)))


def _sample_index_numpy(doc_len: np.ndarray, doc_order: np.ndarray, seq_len: int, num_samples: int) -> np.ndarray:
    lens = doc_len[doc_order]
    ends = np.cumsum(lens, dtype=np.int64)                 # stream position where each entry of doc_order ends
    pos = np.arange(num_samples + 1, dtype=np.int64) * seq_len
    if len(ends) == 0 or pos[-1] >= ends[-1]:
        raise ValueError("the document stream is too short for this many samples")
    d = np.searchsorted(ends, pos, side="right")           # first entry whose end lies beyond pos
    starts = ends - lens
    return np.stack([d, pos - starts[d]], axis=1).astype(np.int64)


def build_sample_index(doc_len: np.ndarray, doc_order: np.ndarray, seq_len: int, num_samples: int,
                       native: Optional[bool] = None) -> np.ndarray:
    """``[num_samples + 1, 2]`` int64: (position in ``doc_order``, offset in that document) of every sample
    start.  Uses the native walker of the kernel library when it is built (``native=None``: if available)."""
    doc_len = np.ascontiguousarray(doc_len, dtype=np.int64)
    doc_order = np.ascontiguousarray(doc_order, dtype=np.int64)
    lib = None
    if native is not False:
        try:
            from ..kernels import build as _build
            if _build.LIB.exists():
                lib = ctypes.CDLL(str(_build.LIB))
                lib.kb_build_sample_index.restype = ctypes.c_int
        except (OSError, AttributeError):
            lib = None
        if lib is None and native:
            raise RuntimeError("the native library is not built (python -m kareus_b200.kernels.build)")
    if lib is None:
        return _sample_index_numpy(doc_len, doc_order, seq_len, num_samples)
    out = np.empty((num_samples + 1, 2), dtype=np.int64)
    P = ctypes.c_void_p
    rc = lib.kb_build_sample_index(P(doc_len.ctypes.data), P(doc_order.ctypes.data), ctypes.c_int64(len(doc_order)),
                                   ctypes.c_int64(seq_len), ctypes.c_int64(num_samples), P(out.ctypes.data))
    if rc == 8:
        raise ValueError("the document stream is too short for this many samples")
    if rc:
        raise ValueError(f"bad arguments to the sample index builder (code {rc})")
    return out


@dataclass
class GPTDatasetConfig:
    seq_len: int
    num_samples: int                       # samples the run will consume (steps x global batch)
    seed: int = 1234
    documents: Optional[Tuple[int, int]] = None   # [first, last) document of the split; None: all
    eod_token: Optional[int] = None        # with it, loss is masked on end-of-document positions
    shuffle_samples: bool = True
    vocab_size: Optional[int] = None       # with it, a token id outside [0, vocab_size) is an error, not an
                                           # out-of-range embedding row on the device


class GPTDataset(torch.utils.data.Dataset):
    def __init__(self, data: IndexedDataset, cfg: GPTDatasetConfig, native: Optional[bool] = None):
        self.data, self.cfg = data, cfg
        lo, hi = cfg.documents if cfg.documents is not None else (0, data.num_documents)
        if not (0 <= lo < hi <= data.num_documents):
            raise ValueError(f"document range [{lo}, {hi}) outside 0..{data.num_documents}")
        self._doc_ids = np.arange(lo, hi, dtype=np.int64)
        all_len = data.document_lengths()
        self._doc_len = all_len                      # indexed by global document id
        tokens_per_epoch = int(all_len[lo:hi].sum())
        if tokens_per_epoch < 2:
            raise ValueError("the split holds fewer than two tokens")
        need = cfg.num_samples * cfg.seq_len + 1
        self.num_epochs = max(1, -(-need // tokens_per_epoch))
        rng = np.random.RandomState(cfg.seed)
        # one independent permutation of the documents per epoch
        self.doc_order = np.concatenate([rng.permutation(self._doc_ids) for _ in range(self.num_epochs)])
        self.sample_index = build_sample_index(self._doc_len, self.doc_order, cfg.seq_len, cfg.num_samples, native)
        self.shuffle = (np.random.RandomState(cfg.seed + 1).permutation(cfg.num_samples).astype(np.int64)
                        if cfg.shuffle_samples else np.arange(cfg.num_samples, dtype=np.int64))
        # every document is one sequence or a run of sequences: map a document to its first sequence
        self._doc_first_seq = data.document_indices

    def __len__(self) -> int:
        return self.cfg.num_samples

    def _read(self, d: int, off: int, n: int) -> np.ndarray:
        """``n`` tokens of the stream starting at (position ``d`` of doc_order, offset ``off``)."""
        out = np.empty(n, dtype=np.int64)
        got = 0
        while got < n:
            doc = int(self.doc_order[d])
            first, last = int(self._doc_first_seq[doc]), int(self._doc_first_seq[doc + 1])
            # walk the sequences of the document (usually one)
            skip = off
            for s in range(first, last):
                ln = int(self.data.sequence_lengths[s])
                if skip >= ln:
                    skip -= ln
                    continue
                take = min(ln - skip, n - got)
                out[got:got + take] = self.data.get(s, skip, take)
                got += take
                skip = 0
                if got == n:
                    break
            d += 1
            off = 0
        return out

    def sample_tokens(self, i: int) -> np.ndarray:
        """The ``seq_len + 1`` tokens of the i-th sample in visiting order."""
        j = int(self.shuffle[i])
        d, off = self.sample_index[j]
        return self._read(int(d), int(off), self.cfg.seq_len + 1)

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        t = torch.from_numpy(self.sample_tokens(i))
        if self.cfg.vocab_size is not None and t.numel() and (int(t.min()) < 0 or int(t.max()) >= self.cfg.vocab_size):
            raise ValueError(f"sample {i} holds token id {int(t.max())} (or a negative one): the file was tokenised "
                             f"for a larger vocabulary than the model's {self.cfg.vocab_size}")
        tokens, labels = t[:-1].contiguous(), t[1:].contiguous()
        mask = torch.ones(self.cfg.seq_len, dtype=torch.float32)
        if self.cfg.eod_token is not None:
            mask[tokens == self.cfg.eod_token] = 0.0
        return {"tokens": tokens, "labels": labels, "loss_mask": mask}


def build_blend_index(weights: Sequence[float], num_samples: int, native: Optional[bool] = None):
    """``(dataset of sample i, index of that sample inside its dataset)`` for a weighted blend: every sample goes
    to the dataset that is furthest behind its share.  Native when the kernel library is built."""
    w = np.asarray(weights, dtype=np.float64)
    if w.ndim != 1 or len(w) == 0 or (w < 0).any() or w.sum() <= 0:
        raise ValueError(f"bad blend weights {weights}")
    w = np.ascontiguousarray(w / w.sum())
    ds = np.empty(num_samples, dtype=np.int16)
    pos = np.empty(num_samples, dtype=np.int64)
    lib = None
    if native is not False:
        try:
            from ..kernels import build as _build
            if _build.LIB.exists():
                lib = ctypes.CDLL(str(_build.LIB))
                lib.kb_build_blend_index.restype = ctypes.c_int
        except (OSError, AttributeError):
            lib = None
        if lib is None and native:
            raise RuntimeError("the native library is not built (python -m kareus_b200.kernels.build)")
    if lib is not None:
        P = ctypes.c_void_p
        rc = lib.kb_build_blend_index(P(w.ctypes.data), ctypes.c_int(len(w)), ctypes.c_int64(num_samples),
                                      P(ds.ctypes.data), P(pos.ctypes.data))
        if rc:
            raise ValueError(f"bad arguments to the blend index builder (code {rc})")
        return ds, pos
    taken = np.zeros(len(w), dtype=np.int64)
    for i in range(num_samples):
        d = int(np.argmax(w * (i + 1) - taken))
        ds[i], pos[i] = d, taken[d]
        taken[d] += 1
    return ds, pos


class BlendedDataset(torch.utils.data.Dataset):
    """Weighted mix of GPT datasets (``model.data.data_prefix: [w0, prefix0, w1, prefix1, ...]`` of the
    reference's run configs; Megatron's ``BlendedDataset``).  ``make(d, n)`` builds dataset ``d`` with room for
    ``n`` samples; each one is asked for as many samples as the blend takes from it."""

    def __init__(self, weights: Sequence[float], make, num_samples: int, native: Optional[bool] = None):
        self.ds_index, self.pos_index = build_blend_index(weights, num_samples, native)
        counts = np.bincount(self.ds_index, minlength=len(weights))
        self.datasets = [make(d, int(c)) if c > 0 else None for d, c in enumerate(counts)]
        self.num_samples = num_samples

    def __len__(self) -> int:
        return self.num_samples

    def __getitem__(self, i: int):
        return self.datasets[int(self.ds_index[i])][int(self.pos_index[i])]
