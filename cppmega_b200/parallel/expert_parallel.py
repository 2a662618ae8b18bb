"""Expert-parallel token dispatch and combine.

``AllToAllDispatcher`` is the plain-collective path (NCCL on GPUs, gloo on CPU): a
dropless all-to-all(v) of the routed token copies to the ranks that own their experts,
a local sort by expert, and the reverse on the way back.  It is the behaviour the
reference selects with ``--moe-token-dispatcher-type alltoall``
(cppmega/recipes/megatron_args.py:99-135) and the baseline the fused peer-memory
dispatcher in :mod:`cppmega_b200.parallel.fused_moe` is measured against.

All index building is done once per layer call and reused by the backward pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .state import ParallelContext


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits,
                               input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits,
                               input_split_sizes=ctx.out_splits, group=ctx.group)
        return out, None, None, None


@dataclass
class DispatchPlan:
    """Everything needed to undo a dispatch."""

    sort_idx: torch.Tensor                 # [T*k] permutation that groups copies by (dest rank, expert)
    token_of_copy: torch.Tensor            # [T*k] source token of each sorted copy
    send_splits: Optional[List[int]]       # rows sent to each EP rank
    recv_splits: Optional[List[int]]       # rows received from each EP rank
    local_sort: Optional[torch.Tensor]     # permutation of received rows into expert order
    counts_local: torch.Tensor             # [E_local] rows per local expert (device)
    counts_local_host: Optional[List[int]]
    num_tokens: int
    topk: int


class AllToAllDispatcher:
    def __init__(self, pc: ParallelContext, num_experts: int):
        if num_experts % pc.ep:
            raise ValueError(f"num_experts={num_experts} not divisible by ep={pc.ep}")
        self.pc = pc
        self.num_experts = num_experts
        self.e_local = num_experts // pc.ep

    def dispatch(self, x: torch.Tensor, expert_ids: torch.Tensor) -> Tuple[torch.Tensor, DispatchPlan]:
        """x [T,H]; expert_ids [T,k] -> rows sorted by local expert, and the plan."""
        pc, E = self.pc, self.num_experts
        T, k = expert_ids.shape
        flat = expert_ids.reshape(-1)
        sort_idx = torch.argsort(flat, stable=True)
        token_of_copy = torch.div(sort_idx, k, rounding_mode="floor")
        counts = torch.bincount(flat, minlength=E)
        xs = x.index_select(0, token_of_copy)
        if pc.ep == 1:
            ch = None if x.is_cuda else counts.tolist()   # the CUDA grouped GEMM reads device counts
            return xs, DispatchPlan(sort_idx, token_of_copy, None, None, None, counts, ch, T, k)
        # exchange per-expert counts so every rank knows what it receives
        all_counts = torch.empty(pc.ep * E, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(all_counts, counts.contiguous(), group=pc.ep_group)
        all_counts = all_counts.view(pc.ep, E)
        lo = pc.ep_rank * self.e_local
        recv_mat = all_counts[:, lo:lo + self.e_local]                    # [src rank, local expert]
        host = torch.cat([counts.view(pc.ep, self.e_local).sum(1), recv_mat.sum(1), recv_mat.reshape(-1)]).tolist()
        send_splits = [int(v) for v in host[:pc.ep]]
        recv_splits = [int(v) for v in host[pc.ep:2 * pc.ep]]
        recv_flat = host[2 * pc.ep:]
        y = _AllToAll.apply(xs, recv_splits, send_splits, pc.ep_group)
        # received rows are ordered (src rank, expert); regroup to (expert, src rank)
        ids = torch.repeat_interleave(
            torch.arange(self.e_local, device=x.device).repeat(pc.ep),
            torch.tensor(recv_flat, device=x.device, dtype=torch.long))
        local_sort = torch.argsort(ids, stable=True)
        y = y.index_select(0, local_sort)
        counts_local = recv_mat.sum(0)
        ch = [int(sum(recv_flat[s * self.e_local + e] for s in range(pc.ep))) for e in range(self.e_local)]
        return y, DispatchPlan(sort_idx, token_of_copy, send_splits, recv_splits, local_sort, counts_local, ch, T, k)

    def combine(self, y: torch.Tensor, probs: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
        """y rows in local-expert order -> [T,H] weighted sum over each token's k copies."""
        pc = self.pc
        if pc.ep > 1:
            inv = torch.empty_like(plan.local_sort)
            inv[plan.local_sort] = torch.arange(plan.local_sort.numel(), device=y.device)
            y = y.index_select(0, inv)
            y = _AllToAll.apply(y, plan.send_splits, plan.recv_splits, pc.ep_group)
        w = probs.reshape(-1).index_select(0, plan.sort_idx).to(y.dtype).unsqueeze(-1)
        out = torch.zeros(plan.num_tokens, y.shape[1], dtype=y.dtype, device=y.device)
        return out.index_add(0, plan.token_of_copy, y * w)
