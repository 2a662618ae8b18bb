"""Named launch recipes: complete (model, parallel, training, optimizer) bundles with an argv and an environment.

Counterpart of the reference's recipe layer (cppmega/recipes/nam56r_nemo_recipe.py:110-458 ``to_args`` /
``to_env_dict`` and the nine pre-built recipes at :465-684; flag bundles of cppmega/recipes/megatron_args.py:34-173).
A recipe here is a :class:`RunProfile` plus the process environment a launch wants; ``to_args()`` gives the argv for
``python -m cppmega_b200.training.pretrain`` and ``to_env_dict()`` the exports.  Real recipes refuse mock data, as
the reference's do; only ``smoke_test`` trains on synthetic tokens.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from ..parallel.dist_optimizer import OptimizerConfig
from ..parallel.state import ParallelConfig
from ..training.lr import LRSchedule
from ..utils.deprecated import require_deprecated_ack
from .model import ModelConfig, nam56r_full, nam56r_tiny
from .run_profiles import RunProfile, TrainingProfile

MOE_DISPATCHERS = ("alltoall", "allgather", "flex")
FLEX_BACKENDS = ("fused_p2p",)


@dataclass(frozen=True)
class Recipe:
    name: str
    profile: RunProfile
    env: Dict[str, str] = field(default_factory=dict)
    notes: str = ""

    def to_args(self, data_path: Optional[str] = None, **training_overrides) -> List[str]:
        t = self.profile.training
        if data_path is not None:
            t = dataclasses.replace(t, data_path=data_path, mock_data=False)
        if training_overrides:
            t = dataclasses.replace(t, **training_overrides)
        if t.mock_data and self.name != "smoke_test":
            raise ValueError(f"recipe {self.name!r} refuses mock data: pass data_path=<indexed dataset prefix>")
        return dataclasses.replace(self.profile, training=t).argv()

    def to_env_dict(self) -> Dict[str, str]:
        env = {
            "CUDA_DEVICE_MAX_CONNECTIONS": "1" if self.profile.parallel.tp > 1 else "8",
            "NCCL_NVLS_ENABLE": "0",                      # peer mappings must survive a rank that leaves between steps
            "PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True",
            "TORCH_NCCL_AVOID_RECORD_STREAMS": "1",
            "OMP_NUM_THREADS": "4",
        }
        env.update(self.env)
        return env

    def shell(self, data_path: Optional[str] = None, master_port: int = 29500) -> str:
        exports = " ".join(f"{k}={v}" for k, v in sorted(self.to_env_dict().items()))
        argv = " ".join(self.to_args(data_path))
        n = self.profile.nproc
        launcher = (f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {n} --master-addr 127.0.0.1 "
                    f"--master-port {master_port} -m cppmega_b200.training.pretrain" if n > 1
                    else "python -m cppmega_b200.training.pretrain")
        return f"{exports} {launcher} {argv}"


def validate_moe_flags(model: ModelConfig, parallel: ParallelConfig) -> None:
    """Cross-field checks of the MoE / DSA flag bundle (cppmega/recipes/megatron_args.py:99-158)."""
    moe, dsa = model.moe, model.dsa
    if moe.dispatcher not in MOE_DISPATCHERS:
        raise ValueError(f"moe dispatcher must be one of {MOE_DISPATCHERS}, got {moe.dispatcher!r}")
    if moe.dispatcher == "flex" and moe.flex_backend not in FLEX_BACKENDS:
        raise ValueError(f"flex dispatcher backend must be one of {FLEX_BACKENDS}, got {moe.flex_backend!r}")
    if moe.dispatcher == "flex" and parallel.ep <= 1:
        raise ValueError("the flex dispatcher needs expert parallelism > 1")
    if dsa.attention_ranks and dsa.indexer_dtype != "bf16":
        raise ValueError("the DSA indexer runs in bf16 only")


def _full(**kw) -> ModelConfig:
    return dataclasses.replace(nam56r_full(), **kw)


def _train(**kw) -> TrainingProfile:
    base = dict(micro_batch_size=4, train_iters=1000, recompute="selective", mock_data=False, data_path="<data>")
    base.update(kw)
    return TrainingProfile(**base)


def _lr() -> LRSchedule:
    return LRSchedule(lr=1e-4, min_lr=1e-5, style="cosine", warmup_steps=50, decay_steps=1000)


def _recipes() -> Dict[str, Callable[[], Recipe]]:
    opt = OptimizerConfig(lr=1e-4, min_lr=1e-5, weight_decay=0.1, clip_grad=1.0)

    def native_pretrain():
        return Recipe("native_pretrain", RunProfile(
            "native_pretrain", "NAM56R, 8 GPUs, EP=8, ZeRO-1 with overlapped reduce / gather, bf16",
            _full(), ParallelConfig(ep=8, distributed_optimizer=True), _train(), opt, _lr()))

    def native_max_throughput():
        return Recipe("native_max_throughput", RunProfile(
            "native_max_throughput", "throughput lane: MBS 8, no recomputation, fused collectives",
            _full(), ParallelConfig(ep=8, distributed_optimizer=True),
            _train(micro_batch_size=8, recompute="none"), opt, _lr()),
            env={"CPPMEGA_B200_FUSED_COLLECTIVES": "1"})

    def dp_only():
        return Recipe("dp_only", RunProfile(
            "dp_only", "pure data parallel (every rank holds all experts): the reference's 'author DP' lane",
            _full(), ParallelConfig(distributed_optimizer=True), _train(recompute="full"), opt, _lr()))

    def mamba3_native():
        return Recipe("mamba3_native", RunProfile(
            "mamba3_native", "MIMO mixer on the in-tree scan kernels, TP=2 with sequence parallel",
            _full(), ParallelConfig(tp=2, ep=4, sequence_parallel=True, distributed_optimizer=True), _train(), opt, _lr()))

    def mamba3_native_max():
        return Recipe("mamba3_native_max", RunProfile(
            "mamba3_native_max", "as mamba3_native with MXFP8 block-scaled linears",
            _full(), ParallelConfig(tp=2, ep=4, sequence_parallel=True, distributed_optimizer=True),
            _train(precision_recipe="mxfp8"), opt, _lr()))

    def noconv():
        return Recipe("noconv", RunProfile(
            "noconv", "'branch B' stack: no-convolution SSD mixer with B/C norm, bias, data-dependent A, trapezoid",
            _full(mamba_variant="noconv_ssd"), ParallelConfig(ep=8, distributed_optimizer=True), _train(), opt, _lr()))

    def noconv_max():
        return Recipe("noconv_max", RunProfile(
            "noconv_max", "noconv stack, MBS 8, no recomputation",
            _full(mamba_variant="noconv_ssd"), ParallelConfig(ep=8, distributed_optimizer=True),
            _train(micro_batch_size=8, recompute="none"), opt, _lr()))

    def mamba3_te(ack: bool = False):
        require_deprecated_ack("mamba3_te recipe", ack, replacement="mamba3_native",
                               reason="the library-fused mixer path was retired; the in-tree kernels cover it")
        return Recipe("mamba3_te", RunProfile(
            "mamba3_te", "retired lane kept for launch-script compatibility", _full(mamba_variant="ssd"),
            ParallelConfig(ep=8, distributed_optimizer=True), _train(), opt, _lr()))

    def smoke_test():
        return Recipe("smoke_test", RunProfile(
            "smoke_test", "tiny model, synthetic tokens, 2 ranks", nam56r_tiny(), ParallelConfig(ep=2),
            TrainingProfile(micro_batch_size=2, dtype="fp32", train_iters=10, mock_data=True),
            OptimizerConfig(lr=1e-3, weight_decay=0.0), LRSchedule(lr=1e-3, style="constant"), nproc=2))

    return {f.__name__: f for f in (native_pretrain, native_max_throughput, dp_only, mamba3_native, mamba3_native_max,
                                    noconv, noconv_max, mamba3_te, smoke_test)}


RECIPES = _recipes()


def get_recipe(name: str, **kw) -> Recipe:
    if name not in RECIPES:
        raise KeyError(f"unknown recipe {name!r}; known: {sorted(RECIPES)}")
    r = RECIPES[name](**kw)
    validate_moe_flags(r.profile.model, r.profile.parallel)
    return r
