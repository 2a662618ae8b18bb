"""Activation recomputation with an operator-level stash.

``checkpoint(fn, *args)`` runs ``fn`` without a graph in the forward pass and replays it in backward, like the
library's reentrant checkpoint.  The difference is the *stash*: an operator whose forward is expensive but whose
output is small compared with what a full graph would keep (the Mamba3 scan: three kernels for an output and chunk
states; sparse attention: output and log-sum-exp) may park its results during the first pass and pick them up in
the replay instead of running its kernels again.  The stash belongs to the checkpoint instance, so it is freed with
the layer's backward and is correct under any micro-batch schedule.

The reference reaches the same end with Megatron's selective recompute switches and a Mamba-specific recompute flag
(``CPPMEGA_MAMBA_RECOMPUTE``, scripts/remote_smoke_h200_dsa_9_4_m.sh:88-123).
"""
from __future__ import annotations

import threading
from typing import Any, Callable, Dict, Optional

import torch

_TLS = threading.local()
STASH_ENABLED = True


class Stash:
    def __init__(self):
        self.mode = "first"                 # "first" (graph-free forward) | "replay"
        self.items: Dict[Any, Any] = {}
        self._n_put = 0
        self._n_get = 0

    def next_put_key(self, tag: str):
        k = (tag, self._n_put)
        self._n_put += 1
        return k

    def next_get_key(self, tag: str):
        k = (tag, self._n_get)
        self._n_get += 1
        return k

    def nbytes(self) -> int:
        tot = 0
        for v in self.items.values():
            for t in (v if isinstance(v, (tuple, list)) else (v,)):
                if torch.is_tensor(t):
                    tot += t.numel() * t.element_size()
        return tot


def current_stash() -> Optional[Stash]:
    return getattr(_TLS, "stash", None) if STASH_ENABLED else None


def stashed_call(tag: str, compute: Callable[[], Any], wrap: Callable[[Any], Any]):
    """Helper for operators.  First pass: ``compute()`` runs, its result is parked, ``wrap(result)`` is returned.
    Replay: the parked result is handed to ``wrap`` without recomputation.  Outside a checkpoint: plain call."""
    st = current_stash()
    if st is None:
        return wrap(compute())
    if st.mode == "first":
        res = compute()
        st.items[st.next_put_key(tag)] = res
        return wrap(res)
    key = st.next_get_key(tag)
    res = st.items.pop(key, None)
    if res is None:                      # replay reached an op the first pass did not stash (shape-dependent path)
        res = compute()
    return wrap(res)


class _RecomputeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, *args):
        ctx.fn = fn
        ctx.stash = Stash()
        ctx.tensor_idx = [i for i, a in enumerate(args) if torch.is_tensor(a)]
        ctx.other = {i: a for i, a in enumerate(args) if not torch.is_tensor(a)}
        ctx.nargs = len(args)
        ctx.save_for_backward(*[args[i] for i in ctx.tensor_idx])
        prev = getattr(_TLS, "stash", None)
        _TLS.stash = ctx.stash
        try:
            with torch.no_grad():
                out = fn(*args)
        finally:
            _TLS.stash = prev
        return out

    @staticmethod
    def backward(ctx, *gouts):
        tensors = ctx.saved_tensors
        args = [None] * ctx.nargs
        leaves = []
        for i, t in zip(ctx.tensor_idx, tensors):
            d = t.detach()
            if t.requires_grad or t.is_floating_point() and ctx.needs_input_grad[i + 1]:
                d.requires_grad_(ctx.needs_input_grad[i + 1])
            args[i] = d
            leaves.append((i, d))
        for i, a in ctx.other.items():
            args[i] = a
        ctx.stash.mode = "replay"
        prev = getattr(_TLS, "stash", None)
        _TLS.stash = ctx.stash
        try:
            with torch.enable_grad():
                out = ctx.fn(*args)
        finally:
            _TLS.stash = prev
        ctx.stash.items.clear()
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, gouts) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        grads = [None] * (ctx.nargs + 1)
        for i, d in leaves:
            grads[i + 1] = d.grad
        return tuple(grads)


def checkpoint(fn: Callable, *args):
    """Run ``fn(*args)`` with recomputation in backward.  Falls back to a plain call when nothing needs a gradient."""
    if not torch.is_grad_enabled():
        return fn(*args)
    return _RecomputeFn.apply(fn, *args)
