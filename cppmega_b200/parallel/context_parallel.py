"""Context-parallel plumbing for the sparse-attention layers.

The sequence is cut into contiguous chunks over a context-parallel group; a DSA layer then needs every key the local
queries may select: the index keys, the latent KV and the rope keys are all-gathered along the sequence (gradients
reduce-scattered back), the queries keep their global positions for the causal rule and the rotary tables.  This is
the part of context parallelism the reference carries (CP-group gathers of ``k_idx`` / key / value inside its DSA
patch, cppmega/megatron/index_cache_patch.py:143-147,213-219); like the reference, the Mamba3 / M2RNN mixers do not
support a split sequence, so ``ParallelConfig.cp`` stays 1 and a layer opts in by carrying a :class:`ContextGroup`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ContextGroup:
    group: Optional[dist.ProcessGroup]
    size: int
    rank: int

    def q_offset(self, local_len: int) -> int:
        return self.rank * local_len


def _all_gather_seq(x: torch.Tensor, cg: ContextGroup) -> torch.Tensor:
    parts = [torch.empty_like(x) for _ in range(cg.size)]
    dist.all_gather(parts, x.contiguous(), group=cg.group)
    return torch.cat(parts, dim=1)


class _GatherContext(torch.autograd.Function):
    """[B, S/cp, ...] -> [B, S, ...]; backward: sum of every rank's gradient for this rank's chunk."""

    @staticmethod
    def forward(ctx, x, cg):
        ctx.cg = cg
        return _all_gather_seq(x, cg)

    @staticmethod
    def backward(ctx, g):
        cg = ctx.cg
        g = g.contiguous()
        dist.all_reduce(g, group=cg.group)
        n = g.shape[1] // cg.size
        return g[:, cg.rank * n:(cg.rank + 1) * n].contiguous(), None


def gather_context(x: torch.Tensor, cg: Optional[ContextGroup]) -> torch.Tensor:
    """All-gather along the sequence dimension (dim 1) over the context-parallel group; identity without one."""
    if cg is None or cg.size == 1:
        return x
    return _GatherContext.apply(x, cg)
