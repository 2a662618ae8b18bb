"""Wrappers for the sequence-mixer, attention and embedding kernels (filled in per kernel)."""
from __future__ import annotations

import ctypes

from .. import functional as F_

_REGISTRY = []


def declare(L: ctypes.CDLL) -> None:
    for fn in _REGISTRY:
        fn(L)


def register() -> None:
    pass


_ = F_
