"""Typed run profiles: the single source of truth for a launch.

A :class:`RunProfile` bundles the model, parallel, training and profiling configuration of one named lane and
renders it as an argument vector for :mod:`cppmega_b200.training.pretrain` (and as a ``torchrun`` shell line).
Overrides are explicit ``--set section.field=value`` flags on the renderer, never environment variables - the
contract of the reference's ``RunProfile`` layer (cppmega/recipes/run_profiles.py:1-9,266-279,697) with its
~90 rendered ``CPPMEGA_*`` exports replaced by the typed tree itself.

    python -m cppmega_b200.config.run_profiles list
    python -m cppmega_b200.config.run_profiles describe b200_nam56r_bf16_ep8
    python -m cppmega_b200.config.run_profiles argv b200_nam56r_bf16_ep8 --set training.micro_batch_size=2
    python -m cppmega_b200.config.run_profiles shell b200_nam56r_mxfp8_tp2_ep4 --nproc 8
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import shlex
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..parallel.dist_optimizer import OptimizerConfig
from ..parallel.state import ParallelConfig
from ..training.lr import LRSchedule
from .model import ModelConfig, nam56r_full, nam56r_quarter, nam56r_tiny


@dataclass(frozen=True)
class ProfilingProfile:
    """Capture window of an external profiler (cppmega/recipes/run_profiles.py:235-262)."""

    enabled: bool = False
    tool: str = "torch"                  # torch | nsys | ncu
    capture_mode: str = "cudaProfilerApi"  # full | delay | cudaProfilerApi
    step_start: int = 3
    step_end: int = 4
    trace: str = "cuda,nvtx,osrt"
    output_dir: str = "profiles_out"
    ncu_case: str = ""                   # tool == "ncu": single-kernel workload of tools/ncu_cases.py to capture
    ncu_kernel: str = ""                 # kernel-name regex (default: the case name)

    def __post_init__(self):
        if self.tool not in ("torch", "nsys", "ncu"):
            raise ValueError(f"unknown profiling tool {self.tool!r}")
        if self.capture_mode not in ("full", "delay", "cudaProfilerApi"):
            raise ValueError(f"unknown capture mode {self.capture_mode!r}")
        if self.step_end <= self.step_start:
            raise ValueError("profiling window must be non-empty")


@dataclass(frozen=True)
class TrainingProfile:
    micro_batch_size: int = 4
    global_batch_size: Optional[int] = None
    train_iters: int = 100
    dtype: str = "bf16"
    precision_recipe: str = "bf16"       # bf16 | mxfp8 | tensorwise
    recompute: str = "none"
    seed: int = 1234
    log_interval: int = 1
    save: Optional[str] = None
    load: Optional[str] = None
    save_interval: int = 0
    data_path: Optional[str] = None
    mock_data: bool = False
    pipeline_schedule: str = "1f1b"
    step_timeout_s: float = 0.0
    monitor_port: int = 0


@dataclass(frozen=True)
class RunProfile:
    name: str
    description: str
    model: ModelConfig
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    training: TrainingProfile = field(default_factory=TrainingProfile)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    lr: LRSchedule = field(default_factory=lambda: LRSchedule(lr=1e-5, style="constant"))
    profiling: ProfilingProfile = field(default_factory=ProfilingProfile)
    nproc: int = 8

    def validate(self) -> "RunProfile":
        t, p, m = self.training, self.parallel, self.model
        if t.precision_recipe in ("mxfp8", "tensorwise") and t.dtype != "bf16":
            raise ValueError("fp8 recipes keep bf16 master activations: dtype must be bf16")
        if m.moe.dispatcher == "flex" and (p.ep <= 1 or m.moe.router_dtype != "fp32"):
            raise ValueError("flex dispatcher needs expert parallelism and an fp32 router")
        if self.nproc % (p.tp * p.pp):
            raise ValueError(f"nproc={self.nproc} not divisible by tp*pp={p.tp * p.pp}")
        dp = self.nproc // (p.tp * p.pp)
        if dp % p.ep:
            raise ValueError(f"data-parallel size {dp} not divisible by ep={p.ep}")
        if m.moe.num_experts % p.ep:
            raise ValueError(f"{m.moe.num_experts} experts not divisible by ep={p.ep}")
        if t.pipeline_schedule == "dualpipev" and p.ep > 1:
            raise ValueError("DualPipeV is incompatible with expert parallelism > 1")
        if t.pipeline_schedule == "dualpipev" and p.pp != 2:
            raise ValueError("DualPipeV runs on pipeline groups of 2 ranks")
        if t.global_batch_size and t.global_batch_size % (t.micro_batch_size * dp):
            raise ValueError("global batch must be a multiple of micro_batch * dp")
        if not t.mock_data and not t.data_path and t.train_iters > 0:
            raise ValueError("a profile needs training.data_path or training.mock_data=true")
        return self

    # ---- rendering ---------------------------------------------------------------------------
    def argv(self) -> List[str]:
        from ..training.arguments import render_args
        from ..training.trainer import TrainConfig
        self.validate()
        t = self.training
        tcfg = TrainConfig(micro_batch_size=t.micro_batch_size, global_batch_size=t.global_batch_size,
                           seq_length=self.model.seq_length, dtype=t.dtype, recompute=t.recompute, seed=t.seed,
                           log_interval=t.log_interval, precision_recipe=t.precision_recipe,
                           optimizer=dataclasses.replace(self.optimizer, lr=self.lr.lr, min_lr=self.lr.min_lr),
                           lr_schedule=self.lr, pipeline_schedule=t.pipeline_schedule)
        a = render_args(self.model, self.parallel, tcfg, train_iters=t.train_iters, data_path=t.data_path, save=t.save,
                        load=t.load, save_interval=t.save_interval, mock_data=t.mock_data)
        if t.step_timeout_s:
            a += ["--step-timeout-s", str(t.step_timeout_s)]
        if t.monitor_port:
            a += ["--monitor-port", str(t.monitor_port)]
        if self.profiling.enabled:
            a += ["--profile", "--profile-step-start", str(self.profiling.step_start), "--profile-step-end",
                  str(self.profiling.step_end)]
        return a

    def shell(self, nproc: Optional[int] = None, master_port: int = 29500) -> str:
        n = nproc or self.nproc
        head = ["python", "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
                "127.0.0.1", "--master-port", str(master_port), "-m", "cppmega_b200.training.pretrain"]
        prof = self.profiling
        if prof.enabled and prof.tool == "nsys":
            head = ["nsys", "profile", "-t", prof.trace, "-c", prof.capture_mode, "-o", f"{prof.output_dir}/{self.name}"] + head
        elif prof.enabled and prof.tool == "ncu":
            # Nsight Compute replays every captured launch dozens of times and serialises the process: it is only ever
            # wrapped around ONE process running ONE small single-kernel workload (tools/ncu_cases.py), never around a
            # training run and never around several ranks.
            case = prof.ncu_case
            if not case:
                raise ValueError("profiling.tool='ncu' needs profiling.ncu_case (a workload name of "
                                 "cppmega_b200.tools.ncu_cases); a whole training run is not captured under ncu")
            cmd = ["ncu", "--set", "full", "--clock-control", "none", "-k", f"regex:{prof.ncu_kernel or case}", "-c", "3",
                   "-o", f"{prof.output_dir}/{case}", "python", "-m", "cppmega_b200.tools.ncu_cases", case]
            return " ".join(shlex.quote(x) for x in cmd)
        return " ".join(shlex.quote(x) for x in head + self.argv())

    def describe(self) -> Dict:
        pc = self.model.param_count()
        dp = self.nproc // (self.parallel.tp * self.parallel.pp)
        t = self.training
        return {
            "name": self.name, "description": self.description,
            "model": {"name": self.model.name, "pattern": self.model.plan().full_pattern, "depth": self.model.depth,
                      "hidden": self.model.hidden_size, "vocab": self.model.vocab_size, "seq": self.model.seq_length,
                      "params_total": pc["total"], "params_active": pc["active"]},
            "parallel": {"nproc": self.nproc, "tp": self.parallel.tp, "pp": self.parallel.pp, "vpp": self.parallel.vpp,
                         "ep": self.parallel.ep, "dp": dp, "sequence_parallel": self.parallel.sequence_parallel,
                         "distributed_optimizer": self.parallel.distributed_optimizer,
                         "fused_collectives": self.parallel.fused_collectives},
            "training": dataclasses.asdict(t),
            "tokens_per_step": (t.global_batch_size or t.micro_batch_size * dp) * self.model.seq_length,
        }


def apply_overrides(profile: RunProfile, assignments: Sequence[str]) -> RunProfile:
    """``section.field=value`` (sections: model, model.<sub>, parallel, training, optimizer, lr, profiling) or
    ``nproc=N``.  Values are parsed as JSON when possible, else kept as strings."""
    for item in assignments:
        if "=" not in item:
            raise ValueError(f"override {item!r} is not key=value")
        key, raw = item.split("=", 1)
        try:
            val = json.loads(raw)
        except json.JSONDecodeError:
            val = raw
        if isinstance(val, list):
            val = tuple(val)
        path = key.split(".")
        if path == ["nproc"]:
            profile = dataclasses.replace(profile, nproc=int(val))
            continue
        profile = _set_path(profile, path, val)
    return profile.validate()


def _set_path(obj, path: List[str], val):
    name = path[0]
    if not dataclasses.is_dataclass(obj) or name not in {f.name for f in dataclasses.fields(obj)}:
        raise KeyError(f"unknown override field {name!r} on {type(obj).__name__}")
    if len(path) == 1:
        return dataclasses.replace(obj, **{name: val})
    return dataclasses.replace(obj, **{name: _set_path(getattr(obj, name), path[1:], val)})


def _profiles() -> Dict[str, RunProfile]:
    full = nam56r_full()
    mock = TrainingProfile(mock_data=True)
    out = [
        RunProfile("b200_nam56r_bf16_ep8", "headline: 8xB200, EP=8 DP=8, ZeRO-1, bf16, micro-batch 4, fused collectives",
                   full, ParallelConfig(ep=8, distributed_optimizer=True),
                   dataclasses.replace(mock, recompute="selective")),
        RunProfile("b200_nam56r_bf16_ep8_nccl", "same lane on the plain NCCL collectives (the measured baseline)",
                   full, ParallelConfig(ep=8, distributed_optimizer=True, fused_collectives=False),
                   dataclasses.replace(mock, recompute="selective")),
        RunProfile("b200_nam56r_mxfp8_tp2_ep4", "8xB200, TP=2 (+SP) EP=4 DP=4, MXFP8 block-scaled linears",
                   full, ParallelConfig(tp=2, ep=4, sequence_parallel=True, distributed_optimizer=True),
                   dataclasses.replace(mock, precision_recipe="mxfp8", recompute="selective")),
        RunProfile("b200_nam56r_single", "1xB200, all 16 experts local, per-layer recomputation",
                   full, ParallelConfig(distributed_optimizer=True),
                   dataclasses.replace(mock, recompute="full"), nproc=1,
                   optimizer=OptimizerConfig(grad_dtype="bf16")),
        RunProfile("europe_bf16_ep4", "the reference's bf16 record topology: PP1 EP4 DP2 (here on B200), MBS 8",
                   full, ParallelConfig(ep=4, distributed_optimizer=True),
                   dataclasses.replace(mock, micro_batch_size=8, global_batch_size=64, recompute="selective")),
        RunProfile("pp2_vpp2_ep4", "the reference launcher's default topology: PP2 VPP2 EP4, MBS 4",
                   full, ParallelConfig(pp=2, vpp=2, ep=4, distributed_optimizer=True),
                   dataclasses.replace(mock, pipeline_schedule="interleaved", global_batch_size=32)),
        RunProfile("local_quarter", "13-layer quarter model on one GPU (correctness lane)",
                   nam56r_quarter(), ParallelConfig(), dataclasses.replace(mock, micro_batch_size=2), nproc=1),
        RunProfile("smoke_tiny", "CPU / gloo plumbing: tiny NAM56R-pattern model, fp32, EP=2",
                   nam56r_tiny(), ParallelConfig(ep=2), dataclasses.replace(mock, micro_batch_size=2, dtype="fp32", train_iters=10),
                   optimizer=OptimizerConfig(lr=1e-3, weight_decay=0.0), lr=LRSchedule(lr=1e-3, style="constant"), nproc=2),
    ]
    return {p.name: p for p in out}


PROFILES = _profiles()


def get_profile(name: str) -> RunProfile:
    if name not in PROFILES:
        raise KeyError(f"unknown run profile {name!r}; known: {sorted(PROFILES)}")
    return PROFILES[name]


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="cppmega_b200.config.run_profiles")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list")
    for cmd in ("describe", "argv", "shell"):
        sp = sub.add_parser(cmd)
        sp.add_argument("profile")
        sp.add_argument("--set", action="append", default=[], metavar="section.field=value")
        if cmd == "shell":
            sp.add_argument("--nproc", type=int, default=None)
            sp.add_argument("--master-port", type=int, default=29500)
    ns = ap.parse_args(argv)
    if ns.cmd == "list":
        for n, p in PROFILES.items():
            print(f"{n:32s} {p.description}")
        return 0
    prof = apply_overrides(get_profile(ns.profile), ns.set)
    if ns.cmd == "describe":
        print(json.dumps(prof.describe(), indent=1, default=str))
    elif ns.cmd == "argv":
        print(" ".join(shlex.quote(a) for a in prof.argv()))
    else:
        print(prof.shell(ns.nproc, ns.master_port))
    return 0


if __name__ == "__main__":
    sys.exit(main())
