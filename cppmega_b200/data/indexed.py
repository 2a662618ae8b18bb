"""Token datasets: the Megatron indexed format (``.bin`` + ``.idx``) through the native prefetching loader,
a pure-Python fallback reader, and a writer used by tests and by the data-preparation tool.

The reference trains from Megatron ``GPTDataset`` files produced by its 5-stage corpus pipeline
(docs/data_preparation.md:10-18, scripts/data_prep_parquet_to_megatron.py); the ``.idx`` header layout
written and parsed here is Megatron's ``MMIDIDX`` version 1.
"""
from __future__ import annotations

import ctypes
import os
import struct
from typing import Dict, Iterator, List, Optional, Sequence

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


def write_indexed_dataset(prefix: str, documents: Sequence[Sequence[int]], dtype=np.int32) -> None:
    """Write ``<prefix>.bin`` / ``<prefix>.idx`` from token-id documents."""
    dtype = np.dtype(dtype)
    sizes = np.array([len(d) for d in documents], dtype=np.int32)
    with open(prefix + ".bin", "wb") as f:
        for d in documents:
            f.write(np.asarray(d, dtype=dtype).tobytes())
    pointers = np.zeros(len(documents), dtype=np.int64)
    if len(documents) > 1:
        pointers[1:] = np.cumsum(sizes[:-1].astype(np.int64)) * dtype.itemsize
    doc_idx = np.arange(len(documents) + 1, dtype=np.int64)
    with open(prefix + ".idx", "wb") as f:
        f.write(_MAGIC)
        f.write(struct.pack("<Q", 1))
        f.write(struct.pack("<B", _CODES[dtype]))
        f.write(struct.pack("<Q", len(sizes)))
        f.write(struct.pack("<Q", len(doc_idx)))
        f.write(sizes.tobytes())
        f.write(pointers.tobytes())
        f.write(doc_idx.tobytes())


def read_index(prefix: str) -> Dict:
    with open(prefix + ".idx", "rb") as f:
        if f.read(9) != _MAGIC:
            raise ValueError(f"{prefix}.idx is not a Megatron indexed dataset")
        (version,) = struct.unpack("<Q", f.read(8))
        (code,) = struct.unpack("<B", f.read(1))
        (n_seq,) = struct.unpack("<Q", f.read(8))
        (n_doc,) = struct.unpack("<Q", f.read(8))
        sizes = np.frombuffer(f.read(4 * n_seq), dtype=np.int32)
        pointers = np.frombuffer(f.read(8 * n_seq), dtype=np.int64)
    return {"version": version, "dtype": np.dtype(_DTYPES[code]), "sizes": sizes, "pointers": pointers, "num_docs": n_doc}


class TokenStream:
    """Batches of ``{"input_ids", "labels"}`` from one indexed dataset, sharded over data-parallel ranks."""

    def __init__(self, prefix: str, seq_len: int, micro_batch: int, rank: int = 0, world: int = 1, seed: int = 1234,
                 depth: int = 4, pin: bool = True, native: Optional[bool] = None):
        idx = read_index(prefix)
        self.dtype = idx["dtype"]
        self.seq_len, self.micro_batch = seq_len, micro_batch
        self.rank, self.world, self.seed = rank, world, seed
        self.path = prefix + ".bin"
        self.width = seq_len + 1
        pin = pin and torch.cuda.is_available()
        self._lib = None
        if native is not False:
            self._lib = _load_runtime()
        if self._lib is None and native:
            raise RuntimeError("native data loader requested but libcppmega_b200_runtime.so is not built")
        if self._lib is not None:
            L = self._lib
            self._h = L.cm_loader_open(self.path.encode(), self.dtype.itemsize, 0, seq_len, micro_batch, rank, world,
                                       seed, depth)
            if not self._h:
                raise ValueError(f"cannot open {self.path} (too short for seq_len={seq_len}?)")
            self._bufs = [torch.empty(micro_batch, self.width, dtype=torch.int64) for _ in range(depth)]
            if pin:
                self._bufs = [b.pin_memory() for b in self._bufs]
            arr = (ctypes.c_void_p * depth)(*[b.data_ptr() for b in self._bufs])
            if L.cm_loader_start(self._h, arr, depth) != 0:
                raise RuntimeError("cm_loader_start failed")
            self.num_samples = L.cm_loader_num_samples(self._h)
        else:
            self._tokens = np.memmap(self.path, dtype=self.dtype, mode="r")
            self.num_samples = (len(self._tokens) - 1) // seq_len
            self._epoch, self._cursor = 0, 0
            self._order = self._perm()

    def _perm(self) -> np.ndarray:
        rng = np.random.default_rng(self.seed + 7919 * (self._epoch + 1))
        return rng.permutation(self.num_samples)

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        if self._lib is not None:
            s = self._lib.cm_loader_next(self._h)
            batch = self._bufs[s].clone()
            self._lib.cm_loader_release(self._h)
        else:
            rows = []
            for _ in range(self.micro_batch):
                g = self._cursor * self.world + self.rank
                if g >= self.num_samples:
                    self._epoch += 1
                    self._order = self._perm()
                    self._cursor, g = 0, self.rank
                st = int(self._order[g % self.num_samples]) * self.seq_len
                rows.append(torch.from_numpy(np.asarray(self._tokens[st:st + self.width]).astype(np.int64)))
                self._cursor += 1
            batch = torch.stack(rows)
        return {"input_ids": batch[:, :-1].contiguous(), "labels": batch[:, 1:].contiguous()}

    def skip(self, n_batches: int) -> None:
        """Advance the stream by ``n_batches`` micro-batches without returning them (resume from a checkpoint: the
        number of batches a run has consumed is stored with it).  The pure-Python reader replays only the cursor
        arithmetic; the native loader has its samples in flight already and consumes them."""
        if n_batches <= 0:
            return
        if self._lib is not None:
            for _ in range(n_batches):
                next(self)
            return
        for _ in range(n_batches * self.micro_batch):
            g = self._cursor * self.world + self.rank
            if g >= self.num_samples:
                self._epoch += 1
                self._order = self._perm()
                self._cursor = 0
            self._cursor += 1

    def close(self) -> None:
        if self._lib is not None and getattr(self, "_h", None):
            self._lib.cm_loader_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_RT = None


def _load_runtime():
    global _RT
    if _RT is not None:
        return _RT or None
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "runtime", "libcppmega_b200_runtime.so")
    if not os.path.exists(path):
        _RT = False
        return None
    L = ctypes.CDLL(path)
    vp, i32, i64, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong
    L.cm_loader_open.argtypes = [ctypes.c_char_p, i32, i64, i32, i32, i32, i32, u64, i32]
    L.cm_loader_open.restype = vp
    L.cm_loader_num_samples.argtypes = [vp]
    L.cm_loader_num_samples.restype = i64
    L.cm_loader_num_tokens.argtypes = [vp]
    L.cm_loader_num_tokens.restype = i64
    L.cm_loader_start.argtypes = [vp, vp, i32]
    L.cm_loader_start.restype = i32
    L.cm_loader_next.argtypes = [vp]
    L.cm_loader_next.restype = i32
    L.cm_loader_release.argtypes = [vp]
    L.cm_loader_release.restype = None
    L.cm_loader_close.argtypes = [vp]
    L.cm_loader_close.restype = None
    _RT = L
    return L


def blend_streams(streams: List[TokenStream], weights: Sequence[float], seed: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Weighted mixture of several datasets (Megatron ``--data-path w1 p1 w2 p2``)."""
    gen = torch.Generator().manual_seed(seed)
    w = torch.tensor(list(weights), dtype=torch.float64)
    w = w / w.sum()
    while True:
        i = int(torch.multinomial(w, 1, generator=gen))
        yield next(streams[i])
