"""Hybrid layer-pattern language.

Two alphabets describe the same stack:

* the *NAM* alphabet used by recipes: ``A`` attention, ``M`` Mamba3 mixer,
  ``R`` M2RNN mixer, ``E`` MoE MLP, ``D`` dense MLP, ``G`` gated-delta (reserved),
  and the pipe character as a pipeline-stage separator;
* the *hybrid* alphabet used on the command line (``--hybrid-layer-pattern``):
  ``*`` attention, ``M`` mixer (Mamba3 or M2RNN, selected per layer), ``E`` MoE,
  ``-`` dense MLP, with ``/``-separated multi-token-prediction suffixes.

A short NAM pattern tiles cyclically to the requested depth; a pattern that
contains pipes must already have the exact depth.  Unknown symbols are rejected
(the reference behaves the same way: cppmega/recipes/nam56r_megatron.py:57-78 for
tiling, :88-165 for translation and the custom-mixer flags).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

NAM_SYMBOLS = frozenset("AMREDG|")
HYBRID_SYMBOLS = frozenset("*MEG-|")

_NAM_TO_HYBRID = {"A": "*", "M": "M", "R": "M", "E": "E", "D": "-", "G": "G"}

MTP_DEPTH_SUFFIX = "*-"


class PatternError(ValueError):
    """Raised for a malformed or unsupported layer pattern."""


def expand_nam_pattern(pattern: str, depth: int) -> List[str]:
    """Return one NAM symbol per layer for ``depth`` layers."""
    if not pattern:
        raise PatternError("pattern must be non-empty")
    if depth <= 0:
        raise PatternError(f"depth must be positive, got {depth}")
    up = pattern.upper()
    bad = sorted(set(up) - NAM_SYMBOLS)
    if bad:
        raise PatternError(
            f"invalid pattern symbols {bad!r}; allowed: {sorted(NAM_SYMBOLS)!r}"
        )
    if "|" in up:
        flat = up.replace("|", "")
        if len(flat) != depth:
            raise PatternError(
                f"pipe-delimited pattern has {len(flat)} layers, expected depth={depth}"
            )
        return list(flat)
    return [up[i % len(up)] for i in range(depth)]


def count_symbols(pattern: str, depth: int) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for s in expand_nam_pattern(pattern, depth):
        out[s] = out.get(s, 0) + 1
    return out


@dataclass(frozen=True)
class PatternIssue:
    symbol: str
    message: str


@dataclass(frozen=True)
class HybridPlan:
    """Result of translating a NAM pattern into the hybrid alphabet."""

    source_pattern: str
    depth: int
    layer_symbols: Tuple[str, ...]          # NAM symbols, one per layer
    hybrid_pattern: str                     # main stack, hybrid alphabet
    mtp_depths: int
    r_layer_numbers: Tuple[int, ...]        # 1-indexed layers running M2RNN
    attention_layer_numbers: Tuple[int, ...]  # 1-indexed layers running attention
    issues: Tuple[PatternIssue, ...] = field(default_factory=tuple)

    @property
    def full_pattern(self) -> str:
        """Main pattern plus one ``/*-`` suffix per MTP depth."""
        if self.mtp_depths <= 0:
            return self.hybrid_pattern
        return self.hybrid_pattern + "".join("/" + MTP_DEPTH_SUFFIX for _ in range(self.mtp_depths))

    @property
    def needs_mamba3(self) -> bool:
        return "M" in self.layer_symbols

    @property
    def needs_m2rnn(self) -> bool:
        return "R" in self.layer_symbols

    def split_for_pipeline(self, pp: int, vpp: int = 1) -> str:
        """Hybrid pattern with a pipe between each of the ``pp*vpp`` chunks."""
        return split_pattern_for_pipeline(self.hybrid_pattern, pp, vpp)


def translate_pattern(pattern: str, depth: int, mtp_depths: int = 0) -> HybridPlan:
    symbols = expand_nam_pattern(pattern, depth)
    issues: List[PatternIssue] = []
    out: List[str] = []
    for s in symbols:
        if s == "G":
            issues.append(PatternIssue("G", "gated-delta layers are reserved and have no runtime"))
        out.append(_NAM_TO_HYBRID[s])
    return HybridPlan(
        source_pattern=pattern,
        depth=depth,
        layer_symbols=tuple(symbols),
        hybrid_pattern="".join(out),
        mtp_depths=int(mtp_depths),
        r_layer_numbers=tuple(i + 1 for i, s in enumerate(symbols) if s == "R"),
        attention_layer_numbers=tuple(i + 1 for i, s in enumerate(symbols) if s == "A"),
        issues=tuple(issues),
    )


def split_pattern_for_pipeline(hybrid_pattern: str, pp: int, vpp: int = 1) -> str:
    """Insert pipes so that the pattern has ``pp*vpp`` near-equal chunks.

    Earlier chunks receive the remainder layers, so 52 layers over 4 chunks is
    13+13+13+13 and 10 over 4 is 3+3+2+2.
    """
    flat = hybrid_pattern.replace("|", "")
    chunks = pp * vpp
    if chunks <= 0:
        raise PatternError("pp*vpp must be positive")
    if chunks > len(flat):
        raise PatternError(f"cannot split {len(flat)} layers into {chunks} chunks")
    base, rem = divmod(len(flat), chunks)
    parts, pos = [], 0
    for c in range(chunks):
        n = base + (1 if c < rem else 0)
        parts.append(flat[pos:pos + n])
        pos += n
    return "|".join(parts)


def parse_hybrid_pattern(full_pattern: str) -> Tuple[List[str], int, List[int]]:
    """Parse a command-line hybrid pattern.

    Returns ``(main_symbols, mtp_depths, chunk_sizes)`` where ``chunk_sizes`` are
    the pipe-delimited chunk lengths of the main stack.
    """
    if not full_pattern:
        raise PatternError("hybrid pattern must be non-empty")
    main, *mtp = full_pattern.split("/")
    bad = sorted(set(main) - HYBRID_SYMBOLS)
    if bad:
        raise PatternError(f"invalid hybrid symbols {bad!r}")
    for suffix in mtp:
        if suffix != MTP_DEPTH_SUFFIX:
            raise PatternError(
                f"MTP suffix must be {MTP_DEPTH_SUFFIX!r} (attention + dense MLP), got {suffix!r}"
            )
    chunks = [len(c) for c in main.split("|")]
    if any(c == 0 for c in chunks):
        raise PatternError("empty pipeline chunk in hybrid pattern")
    return list(main.replace("|", "")), len(mtp), chunks


def attention_ranks(layer_symbols: Sequence[str]) -> Dict[int, int]:
    """Map 1-indexed layer number -> rank among attention layers (0-based)."""
    ranks, r = {}, 0
    for i, s in enumerate(layer_symbols):
        if s in ("A", "*"):
            ranks[i + 1] = r
            r += 1
    return ranks


def parse_int_list(spec: str | Sequence[int] | None) -> Tuple[int, ...]:
    """Parse ``"1,2,5-7"`` (or a sequence) into a sorted tuple of unique ints."""
    if spec is None:
        return ()
    if not isinstance(spec, str):
        return tuple(sorted({int(x) for x in spec}))
    vals = set()
    for item in spec.split(","):
        item = item.strip()
        if not item:
            continue
        if "-" in item[1:]:
            lo, hi = item.split("-", 1)
            lo_i, hi_i = int(lo), int(hi)
            if hi_i < lo_i:
                raise PatternError(f"descending range {item!r}")
            vals.update(range(lo_i, hi_i + 1))
        else:
            vals.add(int(item))
    if any(v < 0 for v in vals):
        raise PatternError("indices must be non-negative")
    return tuple(sorted(vals))
