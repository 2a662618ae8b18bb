"""Training-log contract checker and run comparison.

    python -m cppmega_b200.tools.log_check run.log [--min-steps 20] [--max-final-loss 4.0] [--require-fused moe,optimizer]
    python -m cppmega_b200.tools.log_check --compare a.log b.log

The ``pretrain`` entry point prints one JSON object per logged iteration and a header line.  This tool parses such a
log and fails (exit 1) when the run does not meet its contract: enough iterations, finite and non-increasing loss
(first-quarter mean vs last-quarter mean), no operator fallbacks, the expected fused paths active, no kernel error.
It is the counterpart of the reference's log-contract validator and report builders
(tools/probes/gb10_accepted_path_validation.py, tools/profiling/profile_report.py:1-60, compare_bf16_mxfp8.py:1-70).
"""
from __future__ import annotations

import argparse
import json
import math
import re
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


@dataclass
class RunLog:
    records: List[Dict] = field(default_factory=list)
    header: str = ""
    fused: Dict[str, bool] = field(default_factory=dict)
    errors: List[str] = field(default_factory=list)

    @property
    def losses(self) -> List[float]:
        return [r["loss"] for r in self.records if "loss" in r]

    def mean(self, key: str, skip: int = 2) -> Optional[float]:
        vals = [r[key] for r in self.records[skip:] if key in r]
        return sum(vals) / len(vals) if vals else None


def parse_log(text: str) -> RunLog:
    run = RunLog()
    for line in text.splitlines():
        line = line.strip()
        if line.startswith("[cppmega_b200]"):
            run.header = line
            m = re.search(r"fused paths (\{.*\})", line)
            if m:
                try:
                    run.fused = json.loads(m.group(1).replace("'", '"').replace("True", "true").replace("False", "false"))
                except json.JSONDecodeError:
                    pass
        elif line.startswith("{") and line.endswith("}"):
            try:
                rec = json.loads(line)
            except json.JSONDecodeError:
                continue
            if "iteration" in rec or "step" in rec:
                run.records.append(rec)
        elif "KernelError" in line or "NonFiniteLossError" in line or "Traceback" in line:
            run.errors.append(line)
    return run


def check(run: RunLog, min_steps: int = 1, max_final_loss: Optional[float] = None,
          require_fused: Sequence[str] = (), allow_fallbacks: Sequence[str] = ()) -> List[str]:
    problems: List[str] = list(run.errors)
    losses = run.losses
    if len(losses) < min_steps:
        problems.append(f"only {len(losses)} logged iterations, need {min_steps}")
    if any(not math.isfinite(l) for l in losses):
        problems.append("non-finite loss in the log")
    if len(losses) >= 8:
        q = max(len(losses) // 4, 1)
        first, last = sum(losses[:q]) / q, sum(losses[-q:]) / q
        if last > first * 1.02:
            problems.append(f"loss went up: first-quarter mean {first:.4f}, last-quarter mean {last:.4f}")
    if max_final_loss is not None and losses and losses[-1] > max_final_loss:
        problems.append(f"final loss {losses[-1]:.4f} above {max_final_loss}")
    for name in require_fused:
        if not run.fused.get(name, False):
            problems.append(f"fused path {name!r} is not active")
    for rec in run.records:
        fb = {k: v for k, v in rec.get("fallback_ops", {}).items() if k not in allow_fallbacks and v}
        if fb:
            problems.append(f"operator fallbacks at iteration {rec.get('iteration', rec.get('step'))}: {fb}")
            break
    return problems


def compare(a: RunLog, b: RunLog) -> Dict[str, Dict[str, Optional[float]]]:
    out: Dict[str, Dict[str, Optional[float]]] = {}
    for key in ("tokens_per_s", "tflops_per_gpu", "elapsed_ms", "loss"):
        va, vb = a.mean(key), b.mean(key)
        out[key] = {"a": va, "b": vb, "b_over_a": (vb / va) if va and vb else None}
    n = min(len(a.losses), len(b.losses))
    if n:
        out["loss_curve"] = {"max_abs_diff": max(abs(x - y) for x, y in zip(a.losses[:n], b.losses[:n])), "steps": float(n)}
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="check or compare cppmega_b200 training logs")
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--min-steps", type=int, default=1)
    ap.add_argument("--max-final-loss", type=float, default=None)
    ap.add_argument("--require-fused", default="")
    ap.add_argument("--allow-fallbacks", default="causal_attention")
    ns = ap.parse_args(argv)
    runs = [parse_log(open(p, encoding="utf-8", errors="replace").read()) for p in ns.logs]
    if ns.compare:
        if len(runs) != 2:
            ap.error("--compare needs two logs")
        print(json.dumps(compare(runs[0], runs[1]), indent=1))
        return 0
    rc = 0
    for path, run in zip(ns.logs, runs):
        problems = check(run, ns.min_steps, ns.max_final_loss, [s for s in ns.require_fused.split(",") if s],
                         [s for s in ns.allow_fallbacks.split(",") if s])
        print(f"{path}: {len(run.records)} iterations, " + ("OK" if not problems else "FAILED"))
        for p in problems:
            print("  - " + p)
        rc |= bool(problems)
    return rc


if __name__ == "__main__":
    sys.exit(main())
