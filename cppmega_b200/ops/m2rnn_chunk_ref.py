"""Chunk-checkpointed M2RNN scan in plain PyTorch.

The step-by-step definition (:func:`cppmega_b200.ops.reference.m2rnn_scan`) keeps every intermediate state alive for
autograd: O(S) matrices of [B, H, K, V] fp32.  This version saves only the state at chunk boundaries (O(S / C)) and
re-runs one chunk at a time in backward, carrying d(state) from the later chunk into the earlier one - the same
schedule as the CUDA kernel (history at chunk boundaries, recomputation inside a chunk) and the reference's chunked
PyTorch scan (cppmega/megatron/m2rnn_chunk.py:44,431).  It is the CPU path for long sequences and the oracle for the
kernel's checkpointing.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import reference as ref


class _M2RNNChunkedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, W, f, h0, chunk: int):
        B, S = v.shape[:2]
        states = []
        ys = []
        h = h0
        with torch.no_grad():
            for s0 in range(0, S, chunk):
                sl = slice(s0, min(s0 + chunk, S))
                states.append(h)
                y, h = ref.m2rnn_scan(q[:, sl], k[:, sl], v[:, sl], W, f[:, sl], h)
                ys.append(y)
        ctx.save_for_backward(q, k, v, W, f, *[s for s in states if s is not None])
        ctx.chunk, ctx.has_h0, ctx.n_states = chunk, h0 is not None, len(states)
        return torch.cat(ys, dim=1), h

    @staticmethod
    def backward(ctx, dy, dh_last):
        q, k, v, W, f, *saved = ctx.saved_tensors
        states = list(saved) if ctx.has_h0 else [None] + list(saved)
        S, chunk = v.shape[1], ctx.chunk
        dq, dk, dv, df = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v), torch.zeros_like(f)
        dW = torch.zeros_like(W, dtype=torch.float32)
        dh = dh_last
        starts = list(range(0, S, chunk))
        for ci in reversed(range(len(starts))):
            sl = slice(starts[ci], min(starts[ci] + chunk, S))
            with torch.enable_grad():
                leaves = [t[:, sl].detach().requires_grad_() for t in (q, k, v)]
                Wl = W.detach().requires_grad_()
                fl = f[:, sl].detach().requires_grad_()
                h_in = states[ci]
                h_leaf = None if h_in is None else h_in.detach().requires_grad_()
                y, h_out = ref.m2rnn_scan(leaves[0], leaves[1], leaves[2], Wl, fl, h_leaf)
                outs, grads = [y], [dy[:, sl]]
                if dh is not None:
                    outs.append(h_out)
                    grads.append(dh)
                inputs = leaves + [Wl, fl] + ([h_leaf] if h_leaf is not None else [])
                g = torch.autograd.grad(outs, inputs, grads, allow_unused=True)
            dq[:, sl], dk[:, sl], dv[:, sl] = g[0], g[1], g[2]
            dW += g[3].float()
            df[:, sl] = g[4]
            dh = g[5] if h_leaf is not None else None
        dh0 = dh if ctx.has_h0 else None
        return dq, dk, dv, dW.to(W.dtype), df, dh0, None


def m2rnn_scan_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, W: torch.Tensor, f: torch.Tensor,
                       h0: Optional[torch.Tensor] = None, chunk: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same contract as :func:`reference.m2rnn_scan`; memory of the autograd graph is O(S / chunk) states."""
    return _M2RNNChunkedFn.apply(q, k, v, W, f, h0, int(chunk))
