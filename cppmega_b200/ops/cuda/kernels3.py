"""Wrappers for the Mamba3 scan / sparse attention / indexer / embedding kernels."""
from __future__ import annotations

import ctypes

from .. import functional as F_


def declare(L: ctypes.CDLL) -> None:
    pass


def register() -> None:
    pass


_ = F_
