"""Tensor parallelism with sequence parallelism: region mappings and sharded linears.

These are the NCCL/gloo collectives the reference reaches through Megatron's mappings
(cppmega/megatron/cppmega_mamba3_tp_mixer.py:217-229,363-375,438-444 and
cppmega/megatron/custom_embedding.py:148-153).  On GPUs with peer access the column /
row linears switch to the fused all-gather->GEMM and GEMM->reduce-scatter kernels
in :mod:`cppmega_b200.parallel.fused_tp`; this file is the plain-collective path and
the fallback on CPU.

Activations are ``[B, S, H]``; sequence parallelism shards dim 1.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .state import ParallelContext

SEQ_DIM = 1


def _world(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def _all_gather_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    n = _world(group)
    if n == 1:
        return x
    x = x.contiguous()
    if dim == 0:
        out = x.new_empty((n * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=dim)


def _reduce_scatter_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    n = _world(group)
    if n == 1:
        return x
    chunks = [c.contiguous() for c in x.chunk(n, dim=dim)]
    out = torch.empty_like(chunks[0])
    if x.device.type == "cpu":
        # gloo has no reduce_scatter: all-reduce then slice
        full = x.contiguous().clone()
        dist.all_reduce(full, group=group)
        return full.chunk(n, dim=dim)[dist.get_rank(group)].contiguous()
    dist.reduce_scatter(out, chunks, group=group)
    return out


def _split_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    n = _world(group)
    if n == 1:
        return x
    return x.chunk(n, dim=dim)[dist.get_rank(group)].contiguous()


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _world(ctx.group) > 1:
            g = g.contiguous()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        if _world(group) > 1:
            x = x.contiguous().clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherSeq(torch.autograd.Function):
    """all-gather along the sequence in forward; reduce-scatter (or slice) in backward."""

    @staticmethod
    def forward(ctx, x, group, reduce_grad):
        ctx.group, ctx.reduce_grad = group, reduce_grad
        return _all_gather_dim(x, SEQ_DIM, group)

    @staticmethod
    def backward(ctx, g):
        if ctx.reduce_grad:
            return _reduce_scatter_dim(g, SEQ_DIM, ctx.group), None, None
        return _split_dim(g, SEQ_DIM, ctx.group), None, None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_dim(x, SEQ_DIM, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, SEQ_DIM, ctx.group), None


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _split_dim(x, SEQ_DIM, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, SEQ_DIM, ctx.group), None


class _GatherLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_dim(x, x.dim() - 1, group)

    @staticmethod
    def backward(ctx, g):
        return _split_dim(g, g.dim() - 1, ctx.group), None


def copy_to_tp(x, pc: ParallelContext):
    return _CopyToTP.apply(x, pc.tp_group) if pc.tp > 1 else x


def reduce_from_tp(x, pc: ParallelContext):
    return _ReduceFromTP.apply(x, pc.tp_group) if pc.tp > 1 else x


def gather_seq(x, pc: ParallelContext, reduce_grad: bool = True):
    return _GatherSeq.apply(x, pc.tp_group, reduce_grad) if pc.tp > 1 else x


def reduce_scatter_seq(x, pc: ParallelContext):
    return _ReduceScatterSeq.apply(x, pc.tp_group) if pc.tp > 1 else x


def scatter_seq(x, pc: ParallelContext):
    return _ScatterSeq.apply(x, pc.tp_group) if pc.tp > 1 else x


def gather_last_dim(x, pc: ParallelContext):
    return _GatherLast.apply(x, pc.tp_group) if pc.tp > 1 else x


def _init_full_then_slice(shape_full, std: float, dim: int, sizes_full: Optional[Sequence[int]],
                          tp: int, tp_rank: int, seed: int, dtype, zero: bool = False) -> torch.Tensor:
    """Deterministic init: draw the full matrix from a CPU generator and keep this
    rank's slice, so TP=1 and TP=n hold the same model
    (the reference does the same for per-head params,
    cppmega/megatron/cppmega_mamba3_tp_mixer.py:282-300)."""
    if zero:
        full = torch.zeros(shape_full, dtype=torch.float32)
    else:
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        full = torch.empty(shape_full, dtype=torch.float32).normal_(0.0, std, generator=gen)
    if tp == 1:
        return full.to(dtype)
    if sizes_full is None:
        return full.chunk(tp, dim=dim)[tp_rank].contiguous().to(dtype)
    pieces, pos = [], 0
    for sz in sizes_full:
        blk = full.narrow(dim, pos, sz)
        pieces.append(blk.chunk(tp, dim=dim)[tp_rank])
        pos += sz
    return torch.cat(pieces, dim=dim).contiguous().to(dtype)


class ColumnParallelLinear(nn.Module):
    """``y = x W^T`` with ``W`` split along its output rows.  ``partition_sizes`` lists the
    *full* widths of packed components so each rank keeps a slice of every component
    (recorded on the weight for checkpoint resharding)."""

    def __init__(self, in_features: int, out_features: int, pc: ParallelContext, *,
                 std: float = 0.02, seed: int = 0, dtype=torch.float32,
                 partition_sizes: Optional[Sequence[int]] = None, gather_output: bool = False,
                 sequence_parallel_input: bool = True, zero_init: bool = False, name: str = ""):
        super().__init__()
        tp = pc.tp
        if out_features % tp:
            raise ValueError(f"{name}: out_features={out_features} not divisible by tp={tp}")
        if partition_sizes is not None:
            if sum(partition_sizes) != out_features or any(s % tp for s in partition_sizes):
                raise ValueError(f"{name}: partition_sizes {partition_sizes} invalid for tp={tp}")
        self.pc, self.gather_output = pc, gather_output
        self.sp_input = sequence_parallel_input
        self.in_features, self.out_features = in_features, out_features
        w = _init_full_then_slice((out_features, in_features), std, 0, partition_sizes, tp, pc.tp_rank,
                                  seed, dtype, zero=zero_init)
        self.weight = nn.Parameter(w)
        self.weight.tensor_model_parallel = tp > 1
        self.weight.partition_dim = 0
        self.weight.partition_sizes = [s // tp for s in partition_sizes] if partition_sizes else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import functional as F_
        pc = self.pc
        y = None
        if pc.tp > 1 and pc.sequence_parallel and self.sp_input and x.is_cuda:
            from . import fused_tp
            y = fused_tp.column_linear(x, self.weight)          # all-gather fused into the GEMM's operand loads
        if y is None:
            if pc.tp > 1:
                x = gather_seq(x, pc) if (pc.sequence_parallel and self.sp_input) else copy_to_tp(x, pc)
            y = F_.linear(x, self.weight)
        if self.gather_output:
            y = gather_last_dim(y, pc)
        return y


class RowParallelLinear(nn.Module):
    """``y = x W^T`` with ``W`` split along its input columns; output is reduced over TP
    (reduce-scatter along the sequence under sequence parallelism)."""

    def __init__(self, in_features: int, out_features: int, pc: ParallelContext, *,
                 std: float = 0.02, seed: int = 0, dtype=torch.float32,
                 sequence_parallel_output: bool = True, zero_init: bool = False, name: str = ""):
        super().__init__()
        tp = pc.tp
        if in_features % tp:
            raise ValueError(f"{name}: in_features={in_features} not divisible by tp={tp}")
        self.pc = pc
        self.sp_output = sequence_parallel_output
        self.in_features, self.out_features = in_features, out_features
        w = _init_full_then_slice((out_features, in_features), std, 1, None, tp, pc.tp_rank, seed, dtype,
                                  zero=zero_init)
        self.weight = nn.Parameter(w)
        self.weight.tensor_model_parallel = tp > 1
        self.weight.partition_dim = 1
        self.weight.partition_sizes = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import functional as F_
        pc = self.pc
        if pc.tp > 1 and pc.sequence_parallel and self.sp_output and x.is_cuda:
            from . import fused_tp
            y = fused_tp.row_linear(x, self.weight)             # reduce-scatter fused into the GEMM's epilogue
            if y is not None:
                return y
        y = F_.linear(x, self.weight)
        if pc.tp > 1:
            y = reduce_scatter_seq(y, pc) if (pc.sequence_parallel and self.sp_output) else reduce_from_tp(y, pc)
        return y


class ReplicatedLinear(nn.Module):
    """A small linear kept whole on every TP rank (e.g. the Mamba3 angle projection,
    cppmega/megatron/cppmega_mamba3_tp_mixer.py:244-262).  Under sequence parallelism its
    input is sequence-sharded, so its weight gradient is a partial sum that the
    trainer all-reduces over TP (flag ``sequence_parallel_grad``)."""

    def __init__(self, in_features: int, out_features: int, pc: ParallelContext, *, std: float = 0.02,
                 seed: int = 0, dtype=torch.float32, uniform_bound: Optional[float] = None,
                 zero_init: bool = False, sp_partial_grad: bool = True):
        super().__init__()
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        w = torch.empty(out_features, in_features, dtype=torch.float32)
        if zero_init:
            w.zero_()
        elif uniform_bound is not None:
            w.uniform_(-uniform_bound, uniform_bound, generator=gen)
        else:
            w.normal_(0.0, std, generator=gen)
        self.weight = nn.Parameter(w.to(dtype))
        self.weight.tensor_model_parallel = False
        self.weight.sequence_parallel_grad = pc.sequence_parallel and sp_partial_grad
        self.pc = pc

    def forward(self, x):
        from ..ops import functional as F_
        return F_.linear(x, self.weight)


def allreduce_sequence_parallel_grads(params: List[nn.Parameter], pc: ParallelContext) -> None:
    """Sum over TP the gradients of replicated parameters that consumed sequence-sharded
    activations (norm weights, replicated linears)."""
    if pc.tp == 1 or not pc.sequence_parallel:
        return
    for p in params:
        if getattr(p, "sequence_parallel_grad", False) and p.grad is not None:
            dist.all_reduce(p.grad, group=pc.tp_group)
