"""Tokenise a text corpus into ``<output-prefix>_<key>_document.bin/.idx``.

    python -m kareus_b200.data.preprocess --input corpus.jsonl --json-keys text \\
        --tokenizer hf:/path/to/tokenizer --append-eod --output-prefix data/wikitext

Same outputs as the step the reference runs with Megatron's ``tools/preprocess_data.py``
(``tests/data/prepare_data.sh``: WikiText-103 → ``*_text_document``).  Inputs: JSON lines (one document per
line, text under ``--json-keys``), plain text (one document per line, or per blank-line separated block with
``--split-on-blank``), or ``.npy`` / whitespace-separated integer files that are already token ids.
Tokenizers: ``byte`` (UTF-8 bytes, end-of-document id 256 — needs no files), ``hf:<dir>`` (a Hugging Face
tokenizer directory on disk), ``sentencepiece:<model file>``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Callable, Iterator, List, Optional, Tuple

import numpy as np

from .indexed import IndexedDatasetWriter, best_dtype


def make_tokenizer(spec: str) -> Tuple[Callable[[str], List[int]], int, Optional[int]]:
    """→ (encode, vocabulary size, end-of-document id or None)."""
    if spec == "byte":
        return (lambda s: list(s.encode("utf-8"))), 257, 256
    kind, _, path = spec.partition(":")
    if kind == "hf":
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(path, local_files_only=True)
        eod = tok.eos_token_id
        return (lambda s: tok.encode(s, add_special_tokens=False)), len(tok), eod
    if kind == "sentencepiece":
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor(model_file=path)
        eod = sp.eos_id() if sp.eos_id() >= 0 else None
        return (lambda s: sp.encode(s)), sp.get_piece_size(), eod
    raise ValueError(f"unknown tokenizer {spec!r} (byte, hf:<dir>, sentencepiece:<file>)")


def read_documents(path: Path, json_key: Optional[str], split_on_blank: bool) -> Iterator[str]:
    with open(path, "r", encoding="utf-8") as f:
        if json_key is not None:
            for line in f:
                line = line.strip()
                if line:
                    text = json.loads(line).get(json_key, "")
                    if text:
                        yield text
        elif split_on_blank:
            block: List[str] = []
            for line in f:
                if line.strip():
                    block.append(line)
                elif block:
                    yield "".join(block)
                    block = []
            if block:
                yield "".join(block)
        else:
            for line in f:
                if line.strip():
                    yield line.rstrip("\n")


def read_token_documents(path: Path) -> Iterator[np.ndarray]:
    if path.suffix == ".npy":
        arr = np.load(path, allow_pickle=False)
        if arr.ndim == 1:
            yield arr
        else:
            for row in arr:
                yield row
    else:
        with open(path, "r") as f:
            for line in f:
                if line.strip():
                    yield np.asarray(line.split(), dtype=np.int64)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--json-keys", nargs="*", default=None, help="text fields of a JSON-lines input (one output per key)")
    ap.add_argument("--token-ids", action="store_true", help="the input already holds token ids (.npy or integers per line)")
    ap.add_argument("--split-on-blank", action="store_true", help="plain text: documents are separated by blank lines")
    ap.add_argument("--tokenizer", default="byte")
    ap.add_argument("--append-eod", action="store_true")
    ap.add_argument("--vocab-size", type=int, default=None, help="with --token-ids: picks the on-disk integer width")
    a = ap.parse_args(argv)
    src = Path(a.input)
    if a.token_ids:
        prefix = f"{a.output_prefix}_text_document"
        n_docs = n_tok = 0
        with IndexedDatasetWriter(prefix, dtype=best_dtype(a.vocab_size)) as w:
            for doc in read_token_documents(src):
                w.add_document(doc)
                n_docs += 1
                n_tok += len(doc)
        print(f"{prefix}: {n_docs} documents, {n_tok} tokens")
        return 0
    encode, vocab, eod = make_tokenizer(a.tokenizer)
    if a.append_eod and eod is None:
        print("the tokenizer has no end-of-document id; --append-eod needs one", file=sys.stderr)
        return 2
    keys = a.json_keys if a.json_keys else [None]
    for key in keys:
        prefix = f"{a.output_prefix}_{key or 'text'}_document"
        n_docs = n_tok = 0
        with IndexedDatasetWriter(prefix, dtype=best_dtype(vocab)) as w:
            for text in read_documents(src, key, a.split_on_blank):
                ids = encode(text)
                if a.append_eod:
                    ids = list(ids) + [eod]
                if not ids:
                    continue
                w.add_document(ids)
                n_docs += 1
                n_tok += len(ids)
        print(f"{prefix}: {n_docs} documents, {n_tok} tokens, vocabulary {vocab}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
