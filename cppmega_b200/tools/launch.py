"""Named launch lanes.

    python -m cppmega_b200.tools.launch list
    python -m cppmega_b200.tools.launch b200_nam56r_bf16_ep8 [--dry-run] [--set training.train_iters=50 ...] [--data <prefix>]
    python -m cppmega_b200.tools.launch recipe:native_pretrain --data /data/corpus

    python -m cppmega_b200.tools.launch <lane> --max-restarts 3      # supervise: resume from the last checkpoint on failure

A lane is a run profile (``config/run_profiles.py``) or a recipe (``config/recipes.py``, prefix ``recipe:``); the tool
renders its environment and argv and execs ``torch.distributed.run`` (or plain ``python`` for one process).  This is
the counterpart of the reference's ``scripts/launch.sh {bench3-fp8,europe-bf16,bench3-smoke,gb10}`` lanes
(scripts/launch.sh:16-25), with overrides as typed ``--set section.field=value`` assignments instead of raw env vars.

With ``--max-restarts N`` the tool stays as the parent of the job: when the job ends with a non-zero status (a rank
raised or was killed, the step watchdog aborted a stalled step, a collective timed out) it starts it again, on another
rendezvous port, with ``--load`` pointing at the lane's ``--save`` directory, so the run continues from its last
complete checkpoint (iteration, data position, RNG and optimizer state are part of it).  The reference has no such
driver; its failures are diagnosed after the fact (scripts/bisect_nan_golden.sh:1-40).
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
    ap.add_argument("--max-restarts", type=int, default=0,
                    help="stay as the job's parent and, after a failure, resume it from the last checkpoint up to this many times")
    ap.add_argument("--extra", nargs=argparse.REMAINDER, default=[],
                    help="everything after this flag is appended to the training argv as it is")
    ns = ap.parse_args(args)
    if ns.lane == "list":
        from ..config import recipes, run_profiles
        for name, p in sorted(run_profiles.PROFILES.items()):
            print(f"{name:32s} {p.description}")
        for name in sorted(recipes.RECIPES):
            print(f"recipe:{name}")
        return 0
    env, argv, nproc = resolve(ns.lane, ns.overrides, ns.data)
    argv = argv + list(ns.extra)
    cmd = command(argv, nproc, ns.master_port)
    if ns.dry_run:
        print(" ".join(f"{k}={shlex.quote(v)}" for k, v in sorted(env.items())) + " " + " ".join(shlex.quote(c) for c in cmd))
        return 0
    os.environ.update(env)
    if ns.max_restarts <= 0:
        os.execv(cmd[0], cmd)
        return 0      # pragma: no cover
    return supervise(argv, nproc, ns.master_port, ns.max_restarts)


def _arg_value(argv: Sequence[str], flag: str) -> Optional[str]:
    for i, a in enumerate(argv):
        if a == flag and i + 1 < len(argv):
            return argv[i + 1]
    return None


def supervise(argv: List[str], nproc: int, master_port: int, max_restarts: int, run=None) -> int:
    """Run the job; after a failure run it again from the last checkpoint, at most ``max_restarts`` times.  Returns the
    exit status of the last attempt.  ``run(cmd) -> int`` defaults to ``subprocess.call`` (tests pass their own)."""
    import subprocess
    from ..checkpoint import sharded
    run = run or (lambda c: subprocess.call(c))
    save_dir = _arg_value(argv, "--save")
    attempt = 0
    while True:
        args = list(argv)
        if attempt > 0 and save_dir and sharded.latest_iteration(save_dir) is not None and _arg_value(args, "--load") is None:
            args += ["--load", save_dir]
        rc = run(command(args, nproc, master_port + attempt))
        if rc == 0:
            return 0
        if attempt >= max_restarts:
            print(f"[launch] attempt {attempt + 1} ended with status {rc}; no restarts left", flush=True)
            return rc
        it = sharded.latest_iteration(save_dir) if save_dir else None
        where = f"iteration {it} of {save_dir}" if it is not None else "the beginning (no checkpoint yet)"
        print(f"[launch] attempt {attempt + 1} ended with status {rc}; restarting from {where}", flush=True)
        attempt += 1


if __name__ == "__main__":
    sys.exit(main())
