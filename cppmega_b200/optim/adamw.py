"""AdamW update on a flat fp32 master shard, writing the low-precision copy in the same pass.

On CUDA the update is one launch of the fused kernel (``ops.cuda.adamw_shard``); the
PyTorch path below is the definition it is tested against.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


def adamw_reference(master, m, v, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2):
    gf = g.float() * clip
    m.mul_(b1).add_(gf, alpha=1.0 - b1)
    v.mul_(b2).addcmul_(gf, gf, value=1.0 - b2)
    denom = (v / bc2).sqrt_().add_(eps)
    upd = (m / bc1) / denom
    upd.add_(master * wd_mask.to(master.dtype), alpha=wd)
    master.add_(upd, alpha=-lr)
    out.copy_(master.to(out.dtype))


def adamw_shard_update(master, m, v, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2,
                       skip_segments: Sequence[Tuple[int, int, tuple]] = (), gate=None):
    """Update ``master/m/v`` from gradient shard ``g`` (any float dtype) and store the cast
    result in ``out``.  ``clip`` is a 0-dim tensor multiplied into the gradient (stays on
    device: no host sync).  Ranges in ``skip_segments`` were already updated by Muon.  ``gate`` (CUDA only): a device
    int32 word; when it is non-zero the kernel leaves everything untouched."""
    if skip_segments:
        keep = torch.ones_like(wd_mask)
        for s, e, _ in skip_segments:
            keep[s:e] = False
        idx = keep.nonzero(as_tuple=True)[0]
        if idx.numel() == 0:
            return
        mm, m2, v2, g2 = master[idx], m[idx], v[idx], g[idx]
        o2 = out[idx]
        adamw_reference(mm, m2, v2, g2, o2, wd_mask[idx], clip, lr, b1, b2, eps, wd, bc1, bc2)
        master[idx], m[idx], v[idx], out[idx] = mm, m2, v2, o2
        return
    if master.is_cuda:
        from ..ops import functional as F_
        fn = F_._cuda("adamw_shard", master)
        if fn is not None:
            fn(master, m, v, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2, gate=gate)
            return
    adamw_reference(master, m, v, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2)


_ = List
