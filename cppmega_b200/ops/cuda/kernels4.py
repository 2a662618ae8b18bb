"""Wrappers for the small memory-bound kernels around the mixers (rotary-angle prefix sums, ...)."""
from __future__ import annotations

import ctypes

import torch

from .. import functional as F_

ANG_SEG = 512


def declare(L: ctypes.CDLL) -> None:
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    sig = {
        "cm_angle_cumsum_fwd": [vp, vp, i64, i64, i64, vp, i32, i32, i32, i32, vp],
        "cm_angle_cumsum_bwd": [vp, vp, vp, i64, i64, i64, vp, vp, vp, i32, i32, i32, i32, vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = i32


class AngleCumsumFn(torch.autograd.Function):
    """out[b,t,h,a] = sum_{s<=t} raw[b,s,a] * dt[b,h,s]; ``dt`` may be any strided [B,H,S] fp32 view."""

    @staticmethod
    def forward(ctx, raw, dt):
        from . import lib, stream_ptr, _check
        B, S, A = raw.shape
        H = dt.shape[1]
        raw32 = raw.float().contiguous()
        dt32 = dt if dt.dtype == torch.float32 else dt.float()
        out = torch.empty(B, S, H, A, dtype=torch.float32, device=raw.device)
        sb, sh, ss = dt32.stride()
        _check(lib().cm_angle_cumsum_fwd(raw32.data_ptr(), dt32.data_ptr(), sb, sh, ss, out.data_ptr(), B, S, H, A,
                                         stream_ptr()), "cm_angle_cumsum_fwd")
        F_.count_launch("angle_cumsum")
        ctx.save_for_backward(raw32, dt32)
        ctx.raw_dtype, ctx.dt_dtype = raw.dtype, dt.dtype
        return out

    @staticmethod
    def backward(ctx, g):
        from . import lib, stream_ptr, _check
        raw32, dt32 = ctx.saved_tensors
        B, S, A = raw32.shape
        H = dt32.shape[1]
        # the kernel overwrites its input with suffix sums; autograd may still own `g`, so work on a private copy
        # unless the incoming tensor is a temporary nobody else can see
        g = g.float().contiguous().clone() if g._base is not None or g.dtype != torch.float32 or not g.is_contiguous() else g.clone()
        nseg = (S + ANG_SEG - 1) // ANG_SEG
        segsum = torch.empty(B * H * nseg * A, dtype=torch.float32, device=g.device)
        draw = torch.empty(B, S, A, dtype=torch.float32, device=g.device)
        ddt = torch.empty(B, H, S, dtype=torch.float32, device=g.device)
        sb, sh, ss = dt32.stride()
        _check(lib().cm_angle_cumsum_bwd(g.data_ptr(), raw32.data_ptr(), dt32.data_ptr(), sb, sh, ss, segsum.data_ptr(),
                                         draw.data_ptr(), ddt.data_ptr(), B, S, H, A, stream_ptr()), "cm_angle_cumsum_bwd")
        F_.count_launch("angle_cumsum_bwd", 3)
        return draw.to(ctx.raw_dtype), ddt.to(ctx.dt_dtype)


def angle_cumsum(raw, dt):
    if raw.shape[-1] > 32 or dt.dim() != 3:
        return None
    return AngleCumsumFn.apply(raw, dt)


def register() -> None:
    F_.register_cuda("angle_cumsum", angle_cumsum)
