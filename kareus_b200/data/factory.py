"""From a ``--data-path`` argument to datasets: one token file or a weighted blend, split by document share."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

from .gpt_dataset import BlendedDataset, GPTDataset, GPTDatasetConfig, split_documents
from .indexed import IndexedDataset

TRAIN, VALIDATION, TEST = 0, 1, 2


def parse_data_path(tokens: Sequence[str]) -> Tuple[List[float], List[str]]:
    """``[prefix]`` or ``[w0, prefix0, w1, prefix1, ...]`` → (weights, prefixes)."""
    tokens = list(tokens)
    if len(tokens) == 1:
        return [1.0], tokens
    if len(tokens) % 2 == 0 and tokens:
        try:
            return [float(w) for w in tokens[0::2]], list(tokens[1::2])
        except ValueError as e:
            raise ValueError(f"--data-path pairs are `weight prefix`: {e}") from None
    raise ValueError("--data-path takes one prefix or pairs `weight prefix`")


class TokenData:
    """The token files of a run and how their documents are shared out."""

    def __init__(self, data_path: Sequence[str], split: str, seq_len: int, seed: int = 1234,
                 eod_token: Optional[int] = None, vocab_size: Optional[int] = None):
        self.weights, self.prefixes = parse_data_path(data_path)
        self.files = [IndexedDataset(p) for p in self.prefixes]
        self.split = [float(w) for w in split.split(",")]
        self.seq_len, self.seed, self.eod_token, self.vocab_size = seq_len, seed, eod_token, vocab_size

    def has_share(self, part: int) -> bool:
        """Does every file have at least one document in this share of the split?"""
        for f in self.files:
            ranges = split_documents(f.num_documents, self.split)
            if part >= len(ranges) or ranges[part][1] <= ranges[part][0]:
                return False
        return True

    def _one(self, d: int, part: int, num_samples: int, shuffle: bool) -> GPTDataset:
        docs = split_documents(self.files[d].num_documents, self.split)[part]
        return GPTDataset(self.files[d], GPTDatasetConfig(seq_len=self.seq_len, num_samples=num_samples,
                                                          seed=self.seed + d, documents=docs, eod_token=self.eod_token,
                                                          vocab_size=self.vocab_size, shuffle_samples=shuffle))

    def dataset(self, part: int, num_samples: int, shuffle: bool = True):
        """``num_samples`` samples from the given share (TRAIN, VALIDATION, TEST) of every file, blended by weight."""
        if len(self.files) == 1:
            return self._one(0, part, num_samples, shuffle)
        return BlendedDataset(self.weights, lambda d, n: self._one(d, part, n, shuffle), num_samples)

    def describe(self) -> List[str]:
        return [f"{p}: {f.num_documents} documents, {f.num_tokens} tokens" for p, f in zip(self.prefixes, self.files)]
