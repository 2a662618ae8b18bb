"""Group a profiler kernel table into the step's cost centres.

    python -m cppmega_b200.tools.profile_report <profile dir or kernel_table.txt> [--top 25] [--json out.json]

``utils/profiling.profile_steps`` (``bench.py --profile-dir``, ``pretrain --profile``) writes ``kernel_table.txt``: one row
per kernel / operator with its device time and launch count.  This tool keeps the device kernels (rows whose self device
time is a kernel's own), attributes each to a group (dense GEMM, grouped GEMM, MIMO scan, M2RNN, cross-entropy, MoE
transport, optimizer, norms, sparse attention, library attention, collectives, PyTorch elementwise / copies) and prints
the groups with shares plus the top kernels - the report the reference builds from its nsys exports
(tools/profiling/profile_report.py:1-60, docs/fp8_optimization_session_2026_04_13.md:477-494).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from typing import Dict, List, Optional, Sequence, Tuple

GROUPS: List[Tuple[str, str]] = [
    ("dense GEMM (tcgen05 bf16)", r"gemm_bf16_kernel<.*, [034]>\(|gemm_bf16_kernel<.*, [56]>\("),
    ("grouped GEMM (experts)", r"gemm_bf16_kernel<.*, [12]>\("),
    ("MXFP8 GEMM + quantise", r"mxfp8_gemm_kernel|quantize_(rowwise|colwise|both)_kernel|dequantize_kernel|swizzle_scales"),
    ("Mamba3 MIMO scan", r"mimo_|angle_|head_reduce_kernel|state_scan"),
    ("M2RNN", r"m2rnn_"),
    ("cross-entropy (non-GEMM part)", r"ce_fwd_bwd|cross_entropy|(?<![a-z])ce_"),
    ("MoE transport / permute", r"moe_|router_topk|zero_pad"),
    ("optimizer", r"adamw|reduce_shard|sumsq|muon|qmuon"),
    ("norms / SwiGLU / RoPE / small ops", r"rmsnorm|swiglu|rope_|ngram"),
    ("sparse attention + indexer", r"sparse_mla|indexer_"),
    ("library attention (cuDNN)", r"cudnn|sdpa|flash_(fprop|bprop)|fmha"),
    ("NCCL", r"nccl"),
    ("peer flag waits / signals", r"wait_flags_kernel|signal_peers_kernel"),
    ("strided copies (own kernel)", r"strided_copy_kernel|sum_slots"),
    ("PyTorch elementwise / copy / cat", r"at::native|at_cuda_detail|at::cuda|elementwise_kernel|CatArray|Memcpy|Memset|fill"),
]
_TIME = re.compile(r"^([0-9.]+)(us|ms|s)$")


def _ms(tok: str) -> Optional[float]:
    m = _TIME.match(tok)
    if not m:
        return None
    return float(m.group(1)) * {"us": 1e-3, "ms": 1.0, "s": 1e3}[m.group(2)]


def parse_table(text: str) -> List[Tuple[str, float, int]]:
    """(name, self device ms, calls) for every row that is a device kernel."""
    rows = []
    lines = text.splitlines()
    header = next((l for l in lines if "Self CUDA" in l and "# of Calls" in l), None)
    if header is None:
        return rows
    name_w = header.index("Self CPU %") - 2 if "Self CPU %" in header else 90
    cols = header[name_w:].split("  ")
    cols = [c.strip() for c in cols if c.strip()]
    i_self, i_calls = cols.index("Self CUDA"), cols.index("# of Calls")
    for l in lines:
        if l.startswith("-") or l is header or not l.strip() or l.startswith("Self "):
            continue
        name, rest = l[:name_w].strip(), l[name_w:].split()
        if len(rest) <= max(i_self, i_calls):
            continue
        ms = _ms(rest[i_self])
        if ms is None or ms <= 0 or not rest[i_calls].isdigit():
            continue
        is_kernel = (name.startswith("void ") or "::" in name and "(" in name or "kernel" in name.lower() or "Memcpy" in name
                     or "Memset" in name or name.startswith("nccl") or re.search(r"cudnn_generated|_sdpa_|flash_[fb]prop|cutlass", name))
        if not is_kernel or name.startswith("aten::") or name.startswith("autograd::"):
            continue          # autograd / operator rows repeat their kernels' time
        rows.append((name, ms, int(rest[i_calls])))
    return rows


def group_rows(rows: Sequence[Tuple[str, float, int]]) -> Dict[str, Dict[str, float]]:
    out: Dict[str, Dict[str, float]] = {}
    for name, ms, calls in rows:
        g = next((gname for gname, pat in GROUPS if re.search(pat, name)), "other")
        d = out.setdefault(g, {"ms": 0.0, "launches": 0})
        d["ms"] += ms
        d["launches"] += calls
    return out


def report(text: str, top: int = 25) -> Dict:
    rows = parse_table(text)
    total = sum(r[1] for r in rows) or 1.0
    groups = group_rows(rows)
    return {"total_ms": total,
            "groups": [{"group": g, "ms": round(d["ms"], 3), "share": round(d["ms"] / total, 4), "launches": int(d["launches"])}
                       for g, d in sorted(groups.items(), key=lambda kv: -kv[1]["ms"])],
            "top": [{"kernel": n[:110], "ms": round(ms, 3), "launches": c} for n, ms, c in sorted(rows, key=lambda r: -r[1])[:top]]}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="group a profiler kernel table into cost centres")
    ap.add_argument("path")
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--json", default=None)
    ns = ap.parse_args(argv)
    path = os.path.join(ns.path, "kernel_table.txt") if os.path.isdir(ns.path) else ns.path
    rep = report(open(path, encoding="utf-8", errors="replace").read(), ns.top)
    print(f"device kernel time in the table: {rep['total_ms']:.1f} ms")
    for g in rep["groups"]:
        print(f"  {g['ms']:9.2f} ms  {100 * g['share']:5.1f} %  {g['launches']:6d} launches  {g['group']}")
    print("top kernels:")
    for k in rep["top"]:
        print(f"  {k['ms']:9.2f} ms  {k['launches']:6d}  {k['kernel']}")
    if ns.json:
        with open(ns.json, "w") as f:
            json.dump(rep, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
