"""Shared building blocks: RMSNorm module, dense SwiGLU MLP, seeded init helpers."""
from __future__ import annotations

import zlib
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as F_
from ..parallel.state import ParallelContext
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear


def seed_for(name: str, base: int = 1234) -> int:
    """Stable per-parameter seed so that every parallel layout initialises the same model."""
    return (zlib.crc32(name.encode()) + 7919 * base) % (2**31 - 1)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=torch.float32, sequence_parallel: bool = False):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.weight.sequence_parallel_grad = sequence_parallel
        self.weight.no_weight_decay = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F_.rmsnorm(x, self.weight, self.eps)


class DenseMLP(nn.Module):
    """SwiGLU MLP: fc1 packs [gate | up]; used by MTP layers, 'D' layers and the MoE shared expert."""

    def __init__(self, hidden: int, ffn: int, pc: ParallelContext, *, std: float, out_std: float,
                 dtype=torch.float32, name: str = "mlp", seed: int = 1234):
        super().__init__()
        self.linear_fc1 = ColumnParallelLinear(hidden, 2 * ffn, pc, std=std, dtype=dtype,
                                               seed=seed_for(name + ".linear_fc1", seed),
                                               partition_sizes=[ffn, ffn], name=name + ".linear_fc1")
        self.linear_fc2 = RowParallelLinear(ffn, hidden, pc, std=out_std, dtype=dtype,
                                            seed=seed_for(name + ".linear_fc2", seed), name=name + ".linear_fc2")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear_fc2(F_.swiglu(self.linear_fc1(x)))


def fp32_param(t: torch.Tensor, *, tp_sharded: bool = False, no_wd: bool = True) -> nn.Parameter:
    """Per-head SSM parameters stay fp32 whatever the model dtype; the scan kernels read
    them as fp32 (the reference needed a restore hook after its bf16 wrapper cast them,
    scripts/cppmega_fp8_shim.py:2892-2940)."""
    p = nn.Parameter(t.float().contiguous())
    p.keep_fp32 = True
    p.tensor_model_parallel = tp_sharded
    p.partition_dim = 0
    p.no_weight_decay = no_wd
    return p


def cast_module_params(module: nn.Module, dtype: torch.dtype) -> nn.Module:
    """Cast floating parameters to ``dtype`` except those flagged ``keep_fp32``."""
    for p in module.parameters():
        if p.is_floating_point() and not getattr(p, "keep_fp32", False):
            p.data = p.data.to(dtype)
    return module


def optional_dropout(x, p: float, training: bool):
    return torch.nn.functional.dropout(x, p, training) if p > 0 else x


_ = Optional


class _SplitLastDim(torch.autograd.Function):
    """``torch.split`` along the last dim whose backward assembles the gradient with one strided copy per piece
    (the library's split backward concatenates with a generic kernel that is several times slower on a few wide and
    a few very narrow pieces, which is exactly the packed in-projection of the Mamba mixer)."""

    @staticmethod
    def forward(ctx, x, sizes):
        ctx.sizes, ctx.shape, ctx.dtype = tuple(sizes), x.shape, x.dtype
        return tuple(x.split(ctx.sizes, dim=-1))

    @staticmethod
    def backward(ctx, *grads):
        ref = next(g for g in grads if g is not None)
        out = torch.empty(ctx.shape, dtype=ctx.dtype, device=ref.device)
        off = 0
        for g, sz in zip(grads, ctx.sizes):
            dst = out[..., off:off + sz]
            if g is None:
                dst.zero_()
            elif g.is_cuda:
                from ..ops.cuda import fast_copy_
                fast_copy_(dst, g)
            else:
                dst.copy_(g)
            off += sz
        return out, None


class _CatLastDim(torch.autograd.Function):
    """``torch.cat`` along the last dim as one vectorised strided copy per piece, both ways (the pieces here are head
    slices with 128-byte runs, which the library's batched cat and slice-backward kernels move far below memory speed)."""

    @staticmethod
    def forward(ctx, *xs):
        from ..ops.cuda import fast_copy_
        ctx.sizes = tuple(x.shape[-1] for x in xs)
        out = torch.empty(*xs[0].shape[:-1], sum(ctx.sizes), dtype=xs[0].dtype, device=xs[0].device)
        off = 0
        for x, sz in zip(xs, ctx.sizes):
            fast_copy_(out[..., off:off + sz], x)
            off += sz
        return out

    @staticmethod
    def backward(ctx, g):
        from ..ops.cuda import fast_contiguous
        grads, off = [], 0
        for need, sz in zip(ctx.needs_input_grad, ctx.sizes):
            grads.append(fast_contiguous(g[..., off:off + sz]) if need else None)
            off += sz
        return tuple(grads)


def cat_last_dim(xs):
    xs = list(xs)
    if xs[0].is_cuda and all(x.dtype == xs[0].dtype and x.shape[:-1] == xs[0].shape[:-1] for x in xs):
        return _CatLastDim.apply(*xs)
    return torch.cat(xs, dim=-1)


def split_last_dim(x: torch.Tensor, sizes):
    if x.is_cuda and x.requires_grad:
        return _SplitLastDim.apply(x, tuple(sizes))
    return torch.split(x, list(sizes), dim=-1)
