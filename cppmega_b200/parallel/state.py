"""Process-group topology: one process per GPU, groups for DP / TP / PP / EP.

Rank order (fastest to slowest varying): ``tp -> ep(within dp) -> dp -> pp``.  The
expert-parallel group is carved out of the data-parallel group: ``dp = ep * edp``
where ``edp`` ("expert data parallel") ranks hold replicas of the same experts.
Context parallelism is reserved (size 1): the mixers refuse CP > 1 exactly as the
reference does (cppmega/megatron/cppmega_mamba3_tp_mixer.py:143-147).

Works with the ``nccl`` backend on GPUs and ``gloo`` on CPU.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ParallelConfig:
    tp: int = 1
    pp: int = 1
    ep: int = 1
    cp: int = 1
    vpp: int = 1
    sequence_parallel: bool = False
    distributed_optimizer: bool = True
    overlap_grad_reduce: bool = True
    overlap_param_gather: bool = True
    fused_collectives: bool = True     # peer-memory compute+collective kernels where available

    def __post_init__(self):
        if min(self.tp, self.pp, self.ep, self.cp, self.vpp) < 1:
            raise ValueError("parallel sizes must be >= 1")
        if self.cp != 1:
            raise ValueError("context parallelism is not supported (cp must be 1)")
        if self.sequence_parallel and self.tp == 1:
            object.__setattr__(self, "sequence_parallel", False)

    def dp(self, world: int) -> int:
        denom = self.tp * self.pp
        if world % denom:
            raise ValueError(f"world size {world} not divisible by tp*pp={denom}")
        dp = world // denom
        if dp % self.ep:
            raise ValueError(f"data-parallel size {dp} not divisible by ep={self.ep}")
        return dp

    def describe(self, world: int) -> str:
        parts = []
        dp = self.dp(world)
        for name, v in (("tp", self.tp), ("pp", self.pp), ("ep", self.ep), ("dp", dp)):
            if v > 1 or name == "dp":
                parts.append(f"{name}{v}")
        return "".join(parts)


@dataclass
class ParallelContext:
    """Groups and coordinates of this rank.  ``None`` groups mean size 1."""

    config: ParallelConfig = field(default_factory=ParallelConfig)
    world_size: int = 1
    rank: int = 0
    local_rank: int = 0
    tp_rank: int = 0
    pp_rank: int = 0
    dp_rank: int = 0
    ep_rank: int = 0
    edp_rank: int = 0
    tp_group: Optional[dist.ProcessGroup] = None
    pp_group: Optional[dist.ProcessGroup] = None
    dp_group: Optional[dist.ProcessGroup] = None
    ep_group: Optional[dist.ProcessGroup] = None
    edp_group: Optional[dist.ProcessGroup] = None
    world_group: Optional[dist.ProcessGroup] = None
    embd_group: Optional[dist.ProcessGroup] = None     # first+last pipeline stage (embedding copies)
    # one group per ORDERED pair of pipeline stages (src, dst): messages src -> dst travel on a communicator that carries
    # nothing else, so pre-posted receives of one direction can never queue in front of sends of the other direction
    pp_directed: dict = field(default_factory=dict)
    tp_ranks: List[int] = field(default_factory=lambda: [0])
    pp_ranks: List[int] = field(default_factory=lambda: [0])
    dp_ranks: List[int] = field(default_factory=lambda: [0])
    ep_ranks: List[int] = field(default_factory=lambda: [0])
    edp_ranks: List[int] = field(default_factory=lambda: [0])

    @property
    def tp(self) -> int:
        return self.config.tp

    @property
    def pp(self) -> int:
        return self.config.pp

    @property
    def ep(self) -> int:
        return self.config.ep

    @property
    def dp(self) -> int:
        return len(self.dp_ranks)

    @property
    def edp(self) -> int:
        return len(self.edp_ranks)

    @property
    def sequence_parallel(self) -> bool:
        return self.config.sequence_parallel and self.tp > 1

    @property
    def is_first_pp(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_pp(self) -> bool:
        return self.pp_rank == self.pp - 1

    @property
    def initialized(self) -> bool:
        return self.world_size > 1


_CTX: Optional[ParallelContext] = None


def single_process_context() -> ParallelContext:
    return ParallelContext()


def rank_coordinates(rank: int, world: int, cfg: ParallelConfig):
    """(tp_rank, ep_rank, edp_rank, dp_rank, pp_rank) of ``rank``."""
    dp = cfg.dp(world)
    tp_rank = rank % cfg.tp
    dp_rank = (rank // cfg.tp) % dp
    pp_rank = rank // (cfg.tp * dp)
    ep_rank = dp_rank % cfg.ep
    edp_rank = dp_rank // cfg.ep
    return tp_rank, ep_rank, edp_rank, dp_rank, pp_rank


def group_rank_lists(world: int, cfg: ParallelConfig):
    """Enumerate the rank lists of every group kind; pure function, CPU-testable."""
    dp = cfg.dp(world)
    tp, pp, ep = cfg.tp, cfg.pp, cfg.ep
    edp = dp // ep

    def r(t, d, p):
        return t + tp * (d + dp * p)

    out = {"tp": [], "dp": [], "pp": [], "ep": [], "edp": []}
    for p in range(pp):
        for d in range(dp):
            out["tp"].append([r(t, d, p) for t in range(tp)])
        for t in range(tp):
            out["dp"].append([r(t, d, p) for d in range(dp)])
            for j in range(edp):
                out["ep"].append([r(t, j * ep + e, p) for e in range(ep)])
            for e in range(ep):
                out["edp"].append([r(t, j * ep + e, p) for j in range(edp)])
    for d in range(dp):
        for t in range(tp):
            out["pp"].append([r(t, d, p) for p in range(pp)])
    return out


def initialize(cfg: ParallelConfig = ParallelConfig(), backend: Optional[str] = None,
               timeout_s: float = 600.0, directed_pp_groups: bool = True) -> ParallelContext:
    """Create (or reuse) the default process group from ``RANK``/``WORLD_SIZE``/``MASTER_*``
    and build every sub-group.  With ``WORLD_SIZE`` unset or 1 returns a single-process context."""
    global _CTX
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world == 1 and not dist.is_initialized():
        cfg.dp(1)
        _CTX = ParallelContext(config=cfg, local_rank=local_rank)
        return _CTX
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    world = dist.get_world_size()
    rank = dist.get_rank()
    lists = group_rank_lists(world, cfg)
    mine = {}
    groups = {}
    for kind, rank_lists in lists.items():
        for ranks in rank_lists:
            # every rank must call new_group for every group, in the same order
            g = dist.new_group(ranks=ranks, backend=backend) if len(ranks) > 1 else None
            if rank in ranks:
                mine[kind] = ranks
                groups[kind] = g
    embd_group = None
    if cfg.pp > 1:
        for ranks in lists["pp"]:
            pair = [ranks[0], ranks[-1]]
            g = dist.new_group(ranks=pair, backend=backend)
            if rank in pair:
                embd_group = g
    pp_directed = {}
    if cfg.pp > 1 and (cfg.vpp > 1 or directed_pp_groups):
        for ranks in lists["pp"]:
            for a in range(cfg.pp):
                for b in range(cfg.pp):
                    if a == b:
                        continue
                    g = dist.new_group(ranks=sorted([ranks[a], ranks[b]]), backend=backend)
                    if rank in (ranks[a], ranks[b]):
                        pp_directed[(a, b)] = g
                        if backend == "nccl":
                            # NCCL creates a point-to-point communicator at the first send / receive of a pair, and that
                            # creation blocks the host until the peer arrives.  The schedules pre-post receives in an
                            # order that differs between ranks, so open every channel here, in one global order.
                            one = torch.zeros(1, device=torch.device("cuda", torch.cuda.current_device()))
                            if rank == ranks[a]:
                                dist.send(one, dst=ranks[b], group=g)
                            else:
                                dist.recv(one, src=ranks[a], group=g)
    if pp_directed and backend == "nccl":
        torch.cuda.synchronize()
    tp_rank, ep_rank, edp_rank, dp_rank, pp_rank = rank_coordinates(rank, world, cfg)
    _CTX = ParallelContext(
        config=cfg, world_size=world, rank=rank, local_rank=local_rank,
        tp_rank=tp_rank, pp_rank=pp_rank, dp_rank=dp_rank, ep_rank=ep_rank, edp_rank=edp_rank,
        tp_group=groups["tp"], pp_group=groups["pp"], dp_group=groups["dp"],
        ep_group=groups["ep"], edp_group=groups["edp"], world_group=dist.group.WORLD, embd_group=embd_group,
        tp_ranks=mine["tp"], pp_ranks=mine["pp"], dp_ranks=mine["dp"],
        ep_ranks=mine["ep"], edp_ranks=mine["edp"], pp_directed=pp_directed,
    )
    return _CTX


def get_context() -> ParallelContext:
    global _CTX
    if _CTX is None:
        _CTX = single_process_context()
    return _CTX


def set_context(ctx: Optional[ParallelContext]) -> None:
    global _CTX
    _CTX = ctx


def destroy() -> None:
    global _CTX
    _CTX = None
    if dist.is_initialized():
        dist.destroy_process_group()
