"""Cross-entropy over a vocabulary-sharded output layer.

Each tensor-parallel rank holds ``W_local [V/tp, H]``.  Per token chunk: local logits, global max
(all-reduce MAX), global sum of exponentials and the target logit (all-reduce SUM); the backward
pass recomputes the chunk's logits, forms ``softmax - onehot`` for the local vocabulary slice and
accumulates ``dW_local`` and a partial ``dh`` that is all-reduced over the group.  The full
``[tokens, V]`` logits never exist (the scalars the reference's Megatron stack all-reduces for its
vocab-parallel loss).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .state import ParallelContext

CHUNK = 2048


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, group, vocab_start, ignore_index):
        T = hidden.shape[0]
        Vl = weight.shape[0]
        loss = torch.zeros(T, dtype=torch.float32, device=hidden.device)
        lse_all = torch.empty(T, dtype=torch.float32, device=hidden.device)
        wf = weight
        for s in range(0, T, CHUNK):
            e = min(s + CHUNK, T)
            lg = (hidden[s:e] @ wf.t()).float()
            mx = lg.max(dim=-1).values
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
            se = torch.exp(lg - mx.unsqueeze(-1)).sum(-1)
            local = labels[s:e] - vocab_start
            mine = (local >= 0) & (local < Vl) & (labels[s:e] != ignore_index)
            tgt = torch.where(mine, lg.gather(1, local.clamp(0, Vl - 1).unsqueeze(1)).squeeze(1),
                              torch.zeros_like(mx))
            packed = torch.stack([se, tgt])
            dist.all_reduce(packed, group=group)
            lse = mx + torch.log(packed[0])
            lse_all[s:e] = lse
            valid = labels[s:e] != ignore_index
            loss[s:e] = torch.where(valid, lse - packed[1], torch.zeros_like(lse))
        ctx.save_for_backward(hidden, weight, labels, lse_all)
        ctx.group, ctx.vocab_start, ctx.ignore_index = group, vocab_start, ignore_index
        return loss

    @staticmethod
    def backward(ctx, g):
        hidden, weight, labels, lse_all = ctx.saved_tensors
        T = hidden.shape[0]
        Vl = weight.shape[0]
        dh = torch.empty_like(hidden)
        dw = torch.zeros_like(weight, dtype=torch.float32)
        for s in range(0, T, CHUNK):
            e = min(s + CHUNK, T)
            lg = (hidden[s:e] @ weight.t()).float()
            p = torch.exp(lg - lse_all[s:e].unsqueeze(-1))
            local = labels[s:e] - ctx.vocab_start
            mine = (local >= 0) & (local < Vl)
            rows = torch.nonzero(mine, as_tuple=True)[0]
            p[rows, local[rows]] -= 1.0
            valid = (labels[s:e] != ctx.ignore_index).float()
            p = p * (g[s:e].float() * valid).unsqueeze(-1)
            pd = p.to(hidden.dtype)
            dh[s:e] = pd @ weight
            dw += (pd.t() @ hidden[s:e]).float()
        dist.all_reduce(dh, group=ctx.group)
        return dh, dw.to(weight.dtype), None, None, None, None


def vocab_parallel_linear_cross_entropy(hidden, weight, labels, pc: ParallelContext, ignore_index: int = -100):
    """Per-token CE (0 at ignored rows) for ``hidden [T,H]`` replicated over TP and a
    vocabulary-sharded ``weight``."""
    start = pc.tp_rank * weight.shape[0]
    return _VocabParallelCE.apply(hidden, weight, labels, pc.tp_group, start, ignore_index)
