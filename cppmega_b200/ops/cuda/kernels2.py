"""Wrappers for the sequence-mixer, attention and embedding kernels."""
from __future__ import annotations

import ctypes

import torch

from .. import functional as F_


def declare(L: ctypes.CDLL) -> None:
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    sig = {
        "cm_m2rnn_fwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp],
        "cm_m2rnn_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = i32
    from . import kernels3
    kernels3.declare(L)
    _ = (i64, f32)


# ---------------------------------------------------------------------------
# M2RNN
# ---------------------------------------------------------------------------

class M2RNNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, W, f):
        from . import lib, stream_ptr, _check
        B, S, Hq, KD = q.shape
        Hk = k.shape[2]
        H, VD = v.shape[2], v.shape[3]
        q, k, v, W = q.contiguous(), k.contiguous(), v.contiguous(), W.contiguous()
        f = f.float().contiguous()
        need = any(ctx.needs_input_grad)
        y = torch.empty(B, S, H, VD, dtype=torch.bfloat16, device=v.device)
        hist = torch.empty(B, H, S, KD, VD, dtype=torch.float32, device=v.device) if need else None
        ypart = torch.empty(KD // 16, B, S, H, VD, dtype=torch.float32, device=v.device) if KD > 16 else None
        _check(lib().cm_m2rnn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), W.data_ptr(), f.data_ptr(), y.data_ptr(),
                                  None if ypart is None else ypart.data_ptr(), hist.data_ptr() if need else None, None,
                                  B, S, H, Hq, Hk, KD, VD, stream_ptr()),
               "cm_m2rnn_fwd")
        F_.count_launch("m2rnn_fwd")
        if need:
            ctx.save_for_backward(q, k, v, W, f, hist)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import lib, stream_ptr, _check
        q, k, v, W, f, hist = ctx.saved_tensors
        B, S, Hq, KD = q.shape
        Hk = k.shape[2]
        H, VD = v.shape[2], v.shape[3]
        dev = v.device
        dy = dy.to(torch.bfloat16).contiguous()
        dq_h = torch.empty(B, S, H, KD, dtype=torch.float32, device=dev)
        dk_h = torch.empty(B, S, H, KD, dtype=torch.float32, device=dev)
        dv = torch.zeros(B, S, H, VD, dtype=torch.float32, device=dev)      # accumulated over the CTAs of a head
        df = torch.zeros(B, S, H, dtype=torch.float32, device=dev)
        dW = torch.zeros(H, VD, VD, dtype=torch.float32, device=dev)
        _check(lib().cm_m2rnn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), W.data_ptr(), f.data_ptr(), hist.data_ptr(),
                                  dy.data_ptr(), dq_h.data_ptr(), dk_h.data_ptr(), dv.data_ptr(), df.data_ptr(),
                                  dW.data_ptr(), B, S, H, Hq, Hk, KD, VD, stream_ptr()), "cm_m2rnn_bwd")
        F_.count_launch("m2rnn_bwd")
        dq = dq_h.sum(2, keepdim=True) if Hq == 1 else dq_h
        dk = dk_h.sum(2, keepdim=True) if Hk == 1 else dk_h
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dW.to(W.dtype), df


def m2rnn_scan(q, k, v, W, f):
    KD, VD = q.shape[-1], v.shape[-1]
    if (q.dtype != torch.bfloat16 or v.dtype != torch.bfloat16 or W.dtype != torch.bfloat16 or VD != 16
            or KD not in (16, 32, 64) or q.shape[2] not in (1, v.shape[2]) or k.shape[2] not in (1, v.shape[2])):
        from .. import reference as ref
        return ref.m2rnn_scan(q, k, v, W, f)[0]
    return M2RNNFn.apply(q, k, v, W, f)


def register() -> None:
    F_.register_cuda("m2rnn_scan", m2rnn_scan)
    from . import kernels3
    kernels3.register()
