"""Token files in Megatron's memory-mapped indexed format (``<prefix>.bin`` + ``<prefix>.idx``).

The reference trains on WikiText-103 tokenised into this format by Megatron's ``preprocess_data.py``
(``tests/data/prepare_data_llama.sh``, ``tests/data/prepare_data.sh``) and reads it through
``megatron.core.datasets.indexed_dataset`` (``3rdparty/Megatron-LM/megatron/core/datasets/indexed_dataset.py``).
A run of this package can therefore be pointed at the same files.

``.bin`` holds the tokens of all sequences back to back.  ``.idx`` is::

    9 bytes   b"MMIDIDX\\x00\\x00"
    <Q        version (1)
    <B        dtype code (table below)
    <Q        number of sequences
    <Q        number of document boundaries (= documents + 1)
    int32[]   length of every sequence, in tokens
    int64[]   byte offset of every sequence inside .bin
    int64[]   document boundaries: indices into the sequence arrays, first 0, last = number of sequences

A document is a run of sequences (one sequence per document unless sentences were split).
"""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Iterable, Optional, Sequence, Union

import numpy as np

HEADER = b"MMIDIDX\x00\x00"
VERSION = 1
DTYPE_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32,
               8: np.uint16}
_CODE_OF = {np.dtype(v): k for k, v in DTYPE_CODES.items()}


def best_dtype(vocab_size: int):
    """uint16 up to 65 500 entries (as Megatron's preprocessing chooses), int32 above."""
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


class IndexedDataset:
    """Read-only view of ``<prefix>.bin/.idx``; both files are memory mapped, nothing is loaded eagerly."""

    def __init__(self, prefix: Union[str, Path]):
        self.prefix = str(prefix)
        idx_path, bin_path = Path(self.prefix + ".idx"), Path(self.prefix + ".bin")
        if not idx_path.exists() or not bin_path.exists():
            raise FileNotFoundError(f"{self.prefix}.idx / .bin not found")
        with open(idx_path, "rb") as f:
            if f.read(len(HEADER)) != HEADER:
                raise ValueError(f"{idx_path} is not an indexed-dataset index (bad magic)")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != VERSION:
                raise ValueError(f"{idx_path}: index version {version}, this reader knows {VERSION}")
            (code,) = struct.unpack("<B", f.read(1))
            if code not in DTYPE_CODES:
                raise ValueError(f"{idx_path}: unknown dtype code {code}")
            self.dtype = np.dtype(DTYPE_CODES[code])
            (n_seq,) = struct.unpack("<Q", f.read(8))
            (n_doc,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._idx = np.memmap(idx_path, mode="r", order="C")
        self.sequence_lengths = np.frombuffer(self._idx, dtype=np.int32, count=n_seq, offset=offset)
        offset += self.sequence_lengths.nbytes
        self.sequence_pointers = np.frombuffer(self._idx, dtype=np.int64, count=n_seq, offset=offset)
        offset += self.sequence_pointers.nbytes
        self.document_indices = np.frombuffer(self._idx, dtype=np.int64, count=n_doc, offset=offset)
        self._bin = np.memmap(bin_path, mode="r", order="C")
        if n_seq:
            end = int(self.sequence_pointers[-1]) + int(self.sequence_lengths[-1]) * self.dtype.itemsize
            if end > self._bin.size:
                raise ValueError(f"{bin_path} is shorter ({self._bin.size} B) than its index says ({end} B)")

    def __len__(self) -> int:
        return len(self.sequence_lengths)

    @property
    def num_documents(self) -> int:
        return max(len(self.document_indices) - 1, 0)

    @property
    def num_tokens(self) -> int:
        return int(self.sequence_lengths.sum(dtype=np.int64))

    def get(self, i: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        """Tokens ``[offset, offset + length)`` of sequence ``i`` (a view of the mapped file)."""
        n = int(self.sequence_lengths[i])
        if length is None:
            length = n - offset
        if offset < 0 or length < 0 or offset + length > n:
            raise IndexError(f"sequence {i} has {n} tokens, asked [{offset}, {offset + length})")
        start = int(self.sequence_pointers[i]) + offset * self.dtype.itemsize
        return np.frombuffer(self._bin, dtype=self.dtype, count=length, offset=start)

    def __getitem__(self, i: int) -> np.ndarray:
        return self.get(i)

    def document_lengths(self) -> np.ndarray:
        """Tokens per document (int64)."""
        csum = np.concatenate([[0], np.cumsum(self.sequence_lengths, dtype=np.int64)])
        return csum[self.document_indices[1:]] - csum[self.document_indices[:-1]]


class IndexedDatasetWriter:
    """Writes ``<prefix>.bin/.idx``: ``add_document`` per document (or ``add_sequence`` + ``end_document``
    when a document has several sequences), then ``finalize``.  Usable as a context manager."""

    def __init__(self, prefix: Union[str, Path], dtype=np.int32):
        self.prefix = str(prefix)
        self.dtype = np.dtype(dtype)
        if self.dtype not in _CODE_OF:
            raise ValueError(f"dtype {self.dtype} has no code in the index format")
        Path(self.prefix).parent.mkdir(parents=True, exist_ok=True)
        self._bin = open(self.prefix + ".bin", "wb")
        self._lengths: list = []
        self._docs: list = [0]
        self._done = False

    def add_sequence(self, tokens: Union[Sequence[int], np.ndarray]) -> None:
        arr = np.asarray(tokens)
        if arr.ndim != 1:
            raise ValueError("a sequence is a 1-D array of token ids")
        if arr.size and (arr.min() < np.iinfo(self.dtype).min or arr.max() > np.iinfo(self.dtype).max):
            raise OverflowError(f"token ids do not fit {self.dtype}")
        self._bin.write(arr.astype(self.dtype, copy=False).tobytes(order="C"))
        self._lengths.append(int(arr.size))

    def end_document(self) -> None:
        self._docs.append(len(self._lengths))

    def add_document(self, tokens) -> None:
        self.add_sequence(tokens)
        self.end_document()

    def add_documents(self, docs: Iterable) -> None:
        for d in docs:
            self.add_document(d)

    def finalize(self) -> None:
        if self._done:
            return
        self._done = True
        self._bin.close()
        if self._docs[-1] != len(self._lengths):      # sequences added after the last end_document
            self._docs.append(len(self._lengths))
        lengths = np.asarray(self._lengths, dtype=np.int32)
        pointers = np.zeros(len(lengths), dtype=np.int64)
        if len(lengths) > 1:
            np.cumsum(lengths[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
        docs = np.asarray(self._docs, dtype=np.int64)
        with open(self.prefix + ".idx", "wb") as f:
            f.write(HEADER)
            f.write(struct.pack("<Q", VERSION))
            f.write(struct.pack("<B", _CODE_OF[self.dtype]))
            f.write(struct.pack("<Q", len(lengths)))
            f.write(struct.pack("<Q", len(docs)))
            f.write(lengths.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(docs.tobytes(order="C"))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.finalize()
