"""Named launch lanes.

    python -m cppmega_b200.tools.launch list
    python -m cppmega_b200.tools.launch b200_nam56r_bf16_ep8 [--dry-run] [--set training.train_iters=50 ...] [--data <prefix>]
    python -m cppmega_b200.tools.launch recipe:native_pretrain --data /data/corpus

A lane is a run profile (``config/run_profiles.py``) or a recipe (``config/recipes.py``, prefix ``recipe:``); the tool
renders its environment and argv and execs ``torch.distributed.run`` (or plain ``python`` for one process).  This is
the counterpart of the reference's ``scripts/launch.sh {bench3-fp8,europe-bf16,bench3-smoke,gb10}`` lanes
(scripts/launch.sh:16-25), with overrides as typed ``--set section.field=value`` assignments instead of raw env vars.
"""
from __future__ import annotations

import argparse
import os
import shlex
import sys
from typing import List, Optional, Sequence, Tuple


def resolve(lane: str, overrides: Sequence[str], data: Optional[str]) -> Tuple[dict, List[str], int]:
    """(environment additions, argv for the pretrain entry point, number of processes)."""
    import dataclasses
    from ..config import recipes, run_profiles
    if lane.startswith("recipe:"):
        r = recipes.get_recipe(lane[len("recipe:"):])
        prof = run_profiles.apply_overrides(r.profile, overrides) if overrides else r.profile
        r = dataclasses.replace(r, profile=prof)
        return r.to_env_dict(), r.to_args(data_path=data), r.profile.nproc
    prof = run_profiles.get_profile(lane)
    if data is not None:
        overrides = list(overrides) + [f"training.data_path={data}", "training.mock_data=false"]
    if overrides:
        prof = run_profiles.apply_overrides(prof, overrides)
    env = {"NCCL_NVLS_ENABLE": "0", "PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True"}
    return env, prof.argv(), prof.nproc


def command(argv: List[str], nproc: int, master_port: int) -> List[str]:
    if nproc > 1:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                "--master-addr", "127.0.0.1", "--master-port", str(master_port), "-m", "cppmega_b200.training.pretrain"] + argv
    return [sys.executable, "-m", "cppmega_b200.training.pretrain"] + argv


def main(args: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="launch a named training lane")
    ap.add_argument("lane")
    ap.add_argument("--set", action="append", default=[], dest="overrides")
    ap.add_argument("--data", default=None)
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--dry-run", action="store_true")
    ns = ap.parse_args(args)
    if ns.lane == "list":
        from ..config import recipes, run_profiles
        for name, p in sorted(run_profiles.PROFILES.items()):
            print(f"{name:32s} {p.description}")
        for name in sorted(recipes.RECIPES):
            print(f"recipe:{name}")
        return 0
    env, argv, nproc = resolve(ns.lane, ns.overrides, ns.data)
    cmd = command(argv, nproc, ns.master_port)
    if ns.dry_run:
        print(" ".join(f"{k}={shlex.quote(v)}" for k, v in sorted(env.items())) + " " + " ".join(shlex.quote(c) for c in cmd))
        return 0
    os.environ.update(env)
    os.execv(cmd[0], cmd)
    return 0      # pragma: no cover


if __name__ == "__main__":
    sys.exit(main())
