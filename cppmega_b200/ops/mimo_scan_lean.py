"""Memory-lean PyTorch execution of the Mamba3 MIMO scan for GPUs without the fused kernel.

The chunked operator of :mod:`cppmega_b200.ops.mimo_scan_ref` is evaluated one B/C group of heads
at a time (heads of a group share the un-biased Q/K), with bf16 operands for the large
contractions, and wrapped in an autograd Function that keeps only the inputs and recomputes the
group in backward.  Peak memory is one group's intermediates instead of the whole layer's.
"""
from __future__ import annotations

import torch

from . import mimo_scan_ref as R


class _LeanScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div, chunk):
        ctx.save_for_backward(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z)
        ctx.div, ctx.chunk = div, chunk
        G = Q.shape[3]
        H = V.shape[2]
        hpg = H // G
        outs = []
        with torch.no_grad():
            for g in range(G):
                hs = slice(g * hpg, (g + 1) * hpg)
                outs.append(R.mimo_scan_chunked(
                    Q[:, :, :, g:g + 1], K[:, :, :, g:g + 1], V[:, :, hs], ADT[:, hs], DT[:, hs], Trap[:, hs],
                    Qb[hs], Kb[hs], Psi[hs], Zeta[hs], Phi[hs], angles[:, :, hs], D[hs], Z[:, :, hs],
                    div, chunk, mm_dtype=torch.bfloat16))
        return torch.cat(outs, dim=2)

    @staticmethod
    def backward(ctx, dy):
        return lean_backward(ctx.saved_tensors, dy, ctx.div, ctx.chunk)


def lean_backward(saved, dy, div, chunk):
    """Gradients of the scan by recomputing one head group at a time under autograd."""
    if True:
        Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z = saved
        G = Q.shape[3]
        H = V.shape[2]
        hpg = H // G
        grads = [torch.zeros_like(t, dtype=torch.float32) if t.is_floating_point() else None for t in saved]
        # which dim of each input carries heads (None = group dim 3 for Q/K)
        head_dim = [None, None, 2, 1, 1, 1, 0, 0, 0, 0, 0, 2, 0, 2]
        for g in range(G):
            hs = slice(g * hpg, (g + 1) * hpg)
            parts = []
            for t, hd in zip(saved, head_dim):
                if hd is None:
                    p = t[:, :, :, g:g + 1]
                else:
                    idx = [slice(None)] * t.dim()
                    idx[hd] = hs
                    p = t[tuple(idx)]
                parts.append(p.detach().requires_grad_(True))
            with torch.enable_grad():
                y = R.mimo_scan_chunked(*parts, div, chunk, mm_dtype=torch.bfloat16)
            gs = torch.autograd.grad(y, parts, dy[:, :, hs].to(y.dtype), allow_unused=True)
            for i, (gi, hd) in enumerate(zip(gs, head_dim)):
                if gi is None:
                    continue
                if hd is None:
                    grads[i][:, :, :, g:g + 1] += gi.float()
                else:
                    idx = [slice(None)] * grads[i].dim()
                    idx[hd] = hs
                    grads[i][tuple(idx)] += gi.float()
        out = [None if g is None else g.to(t.dtype) for g, t in zip(grads, saved)]
        return (*out, None, None)


def mimo_scan_lean(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div: int = 4, chunk: int = 64):
    return _LeanScan.apply(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div, chunk)
