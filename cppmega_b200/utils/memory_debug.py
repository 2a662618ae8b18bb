"""CUDA memory statistics, per-phase peaks and allocator snapshots with filtered stack frames
(the reference's NANOCHAT_MEMORY_DEBUG tooling, cppmega/megatron/memory_debug.py:1-70, and its at-exit
per-rank peak reporter, scripts/remote_smoke_h200_dsa_9_4_m.sh:446-464)."""
from __future__ import annotations

import contextlib
import os
import pickle
from typing import Dict, List, Optional

import torch


def memory_stats(device=None) -> Dict[str, float]:
    if not torch.cuda.is_available():
        return {}
    gib = 2 ** 30
    free, total = torch.cuda.mem_get_info(device)
    return {"allocated_gib": torch.cuda.memory_allocated(device) / gib,
            "reserved_gib": torch.cuda.memory_reserved(device) / gib,
            "peak_allocated_gib": torch.cuda.max_memory_allocated(device) / gib,
            "peak_reserved_gib": torch.cuda.max_memory_reserved(device) / gib,
            "free_gib": free / gib, "total_gib": total / gib}


def peak_memory_report(device=None) -> str:
    s = memory_stats(device)
    if not s:
        return "[mem] no CUDA device"
    return (f"[mem] peak allocated {s['peak_allocated_gib']:.2f} GiB, peak reserved {s['peak_reserved_gib']:.2f} GiB, "
            f"free {s['free_gib']:.2f} / {s['total_gib']:.2f} GiB")


@contextlib.contextmanager
def phase_peak(name: str, sink: Optional[Dict[str, float]] = None, device=None):
    """Record the peak allocation reached inside the block under ``sink[name]`` (GiB)."""
    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.reset_peak_memory_stats(device)
    base = torch.cuda.memory_allocated(device)
    try:
        yield
    finally:
        peak = torch.cuda.max_memory_allocated(device)
        if sink is not None:
            sink[name] = (peak - base) / 2 ** 30


def dtype_audit(module: torch.nn.Module) -> Dict[str, Dict[str, float]]:
    """Parameter bytes per dtype, and per top-level sub-module (what holds the memory)."""
    by_dtype: Dict[str, float] = {}
    by_child: Dict[str, float] = {}
    for name, p in module.named_parameters():
        b = p.numel() * p.element_size()
        by_dtype[str(p.dtype)] = by_dtype.get(str(p.dtype), 0.0) + b
        top = name.split(".")[0]
        by_child[top] = by_child.get(top, 0.0) + b
    return {"by_dtype_gib": {k: v / 2 ** 30 for k, v in by_dtype.items()},
            "by_module_gib": {k: v / 2 ** 30 for k, v in by_child.items()}}


def start_history(max_entries: int = 100000) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=max_entries)


def dump_snapshot(path: str, keep_frames: Optional[List[str]] = None) -> Optional[str]:
    """Write the allocator snapshot; stack frames are reduced to those whose filename contains one of
    ``keep_frames`` (default: this package) so the dump stays readable."""
    if not torch.cuda.is_available():
        return None
    snap = torch.cuda.memory._snapshot()
    keep = keep_frames or ["cppmega_b200"]
    for seg in snap.get("segments", []):
        for blk in seg.get("blocks", []):
            frames = blk.get("frames")
            if frames:
                blk["frames"] = [f for f in frames if any(k in f.get("filename", "") for k in keep)][:8]
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        pickle.dump(snap, f)
    return path
