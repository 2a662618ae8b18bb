"""Corpus -> Megatron indexed dataset (``.bin`` + ``.idx``).

    python -m cppmega_b200.tools.data_prep --input corpus.jsonl --text-key text --tokenizer sp.model --out data/corpus
    python -m cppmega_b200.tools.data_prep --input shard-*.parquet --text-key content --tokenizer bytes --out data/code

Inputs: ``.jsonl`` (one JSON object per line), ``.txt`` (one document per line) or ``.parquet`` (a text column).
Tokenizers: a SentencePiece model file, a Hugging Face tokenizer directory / name that is available offline, or
``bytes`` (UTF-8 bytes + 256 as end-of-document).  Documents are filtered by a minimum length, get an end-of-document
token appended, are optionally packed FIM-style, and are written as one indexed dataset that
:class:`cppmega_b200.data.indexed.TokenStream` and the native loader read.  This covers the last stages of the
reference's corpus pipeline (tokenise, filter, write Megatron ``.bin/.idx``; scripts/data_prep_parquet_to_megatron.py,
docs/data_preparation.md:10-18).
"""
from __future__ import annotations

import argparse
import glob
import json
import random
import sys
from typing import Callable, Iterator, List, Optional, Sequence

import numpy as np

from ..data.indexed import write_indexed_dataset


def iter_documents(paths: Sequence[str], text_key: str) -> Iterator[str]:
    for path in paths:
        if path.endswith(".parquet"):
            import pyarrow.parquet as pq
            for batch in pq.ParquetFile(path).iter_batches(columns=[text_key]):
                for v in batch.column(0).to_pylist():
                    if v:
                        yield v
        elif path.endswith(".jsonl") or path.endswith(".json"):
            with open(path, encoding="utf-8") as f:
                for line in f:
                    line = line.strip()
                    if line:
                        v = json.loads(line).get(text_key)
                        if v:
                            yield v
        else:
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        yield line.rstrip("\n")


def load_tokenizer(spec: str):
    """Returns (encode(text) -> List[int], eod id, vocab size)."""
    if spec == "bytes":
        return (lambda t: list(t.encode("utf-8"))), 256, 257
    if spec.endswith(".model"):
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor(model_file=spec)
        eod = sp.eos_id() if sp.eos_id() >= 0 else sp.vocab_size()
        return (lambda t: sp.encode(t)), eod, max(sp.vocab_size(), eod + 1)
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(spec, local_files_only=True)
    eod = tok.eos_token_id if tok.eos_token_id is not None else len(tok)
    return (lambda t: tok.encode(t, add_special_tokens=False)), eod, max(len(tok), eod + 1)


def fim_transform(ids: List[int], rng: random.Random, rate: float, prefix_id: int, middle_id: int, suffix_id: int) -> List[int]:
    """Fill-in-the-middle permutation (PSM order) applied to a fraction ``rate`` of the documents."""
    if rate <= 0 or rng.random() >= rate or len(ids) < 3:
        return ids
    a, b = sorted(rng.sample(range(1, len(ids)), 2))
    return [prefix_id] + ids[:a] + [suffix_id] + ids[b:] + [middle_id] + ids[a:b]


def prepare(paths: Sequence[str], text_key: str, encode: Callable[[str], List[int]], eod: int, out_prefix: str,
            vocab_size: int, min_tokens: int = 8, fim_rate: float = 0.0, seed: int = 0,
            max_docs: Optional[int] = None) -> dict:
    rng = random.Random(seed)
    docs: List[np.ndarray] = []
    dropped = total = 0
    dtype = np.uint16 if vocab_size + 3 <= 65536 else np.int32
    for text in iter_documents(paths, text_key):
        ids = encode(text)
        if len(ids) < min_tokens:
            dropped += 1
            continue
        ids = fim_transform(ids, rng, fim_rate, vocab_size, vocab_size + 1, vocab_size + 2) + [eod]
        docs.append(np.asarray(ids, dtype=dtype))
        total += len(ids)
        if max_docs and len(docs) >= max_docs:
            break
    if not docs:
        raise SystemExit("no document survived the filters")
    write_indexed_dataset(out_prefix, docs, dtype=dtype)
    return {"documents": len(docs), "dropped": dropped, "tokens": total, "dtype": str(np.dtype(dtype)), "prefix": out_prefix}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input", nargs="+", required=True, help="files or glob patterns (.jsonl / .txt / .parquet)")
    ap.add_argument("--text-key", default="text")
    ap.add_argument("--tokenizer", default="bytes")
    ap.add_argument("--out", required=True, help="output prefix (<out>.bin / <out>.idx)")
    ap.add_argument("--min-tokens", type=int, default=8)
    ap.add_argument("--fim-rate", type=float, default=0.0)
    ap.add_argument("--max-docs", type=int, default=None)
    ap.add_argument("--seed", type=int, default=0)
    ns = ap.parse_args(argv)
    paths: List[str] = []
    for pat in ns.input:
        hits = sorted(glob.glob(pat))
        paths += hits if hits else [pat]
    encode, eod, vocab = load_tokenizer(ns.tokenizer)
    info = prepare(paths, ns.text_key, encode, eod, ns.out, vocab, ns.min_tokens, ns.fim_rate, ns.seed, ns.max_docs)
    print(json.dumps(info))
    return 0


if __name__ == "__main__":
    sys.exit(main())
