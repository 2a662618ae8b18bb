"""Check an indexed dataset (``<prefix>.bin`` + ``<prefix>.idx``) before a run.

    python -m cppmega_b200.tools.verify_dataset <prefix> [--vocab-size 131072] [--eod 0] [--sample 1000]

Checks: the index parses; the document sizes add up to the length of the ``.bin`` file; no empty documents; every
sampled token id is inside the vocabulary; (optionally) every sampled document ends with the end-of-document id.  Prints
one JSON line and exits 1 on any violation - the counterpart of the reference's dataset verifier
(scripts/data/verify_dataset_megacpp.py).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional, Sequence

import numpy as np

from ..data.indexed import read_index


def verify(prefix: str, vocab_size: Optional[int] = None, eod: Optional[int] = None, sample: int = 1000, seed: int = 0) -> dict:
    problems: List[str] = []
    idx = read_index(prefix)
    sizes = np.asarray(idx["sizes"], dtype=np.int64)
    dtype = np.dtype(idx["dtype"])
    nbytes = os.path.getsize(prefix + ".bin")
    total = int(sizes.sum())
    if total * dtype.itemsize != nbytes:
        problems.append(f"sizes sum to {total} tokens = {total * dtype.itemsize} bytes but the .bin file has {nbytes}")
    if (sizes <= 0).any():
        problems.append(f"{int((sizes <= 0).sum())} empty documents")
    data = np.memmap(prefix + ".bin", dtype=dtype, mode="r")
    offsets = np.concatenate([[0], np.cumsum(sizes)])
    rng = np.random.default_rng(seed)
    picks = np.arange(len(sizes)) if len(sizes) <= sample else rng.choice(len(sizes), size=sample, replace=False)
    max_id, bad_eod = -1, 0
    for d in picks:
        lo, hi = int(offsets[d]), int(offsets[d + 1])
        if hi > len(data) or hi <= lo:
            continue
        doc = np.asarray(data[lo:hi])
        max_id = max(max_id, int(doc.max()))
        if doc.min() < 0:
            problems.append(f"negative token id in document {int(d)}")
        if eod is not None and int(doc[-1]) != eod:
            bad_eod += 1
    if vocab_size is not None and max_id >= vocab_size:
        problems.append(f"token id {max_id} outside the vocabulary of {vocab_size}")
    if bad_eod:
        problems.append(f"{bad_eod} of {len(picks)} sampled documents do not end with eod={eod}")
    return {"prefix": prefix, "documents": int(len(sizes)), "tokens": total, "dtype": str(dtype), "max_token_id_sampled": max_id,
            "sampled_documents": int(len(picks)), "problems": problems}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="verify an indexed dataset")
    ap.add_argument("prefix")
    ap.add_argument("--vocab-size", type=int, default=None)
    ap.add_argument("--eod", type=int, default=None)
    ap.add_argument("--sample", type=int, default=1000)
    ns = ap.parse_args(argv)
    rep = verify(ns.prefix, ns.vocab_size, ns.eod, ns.sample)
    print(json.dumps(rep))
    return 1 if rep["problems"] else 0


if __name__ == "__main__":
    sys.exit(main())
