"""Dense causal attention on the tcgen05 kernels of ``ops/csrc/attention.cu`` (q / k head dim 128, v head dim 64)."""
from __future__ import annotations

import ctypes

import torch

from .. import functional as F_


def declare(L: ctypes.CDLL) -> None:
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    sig = {
        "cm_attn_fwd": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp, vp],
        "cm_attn_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp, vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = i32


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and q.dim() == 4 and q.shape == k.shape and q.shape[-1] == 128 and v.shape[-1] == 64
            and v.shape[:3] == q.shape[:3] and q.shape[1] % 128 == 0 and q.numel() > 0)


def attn_fwd_raw(q, k, v, scale: float):
    """q, k [B,S,H,128], v [B,S,H,64] packed bf16 -> (out [B,S,H,64] bf16, lse2 [B,H,S] fp32 in the log2 domain)."""
    from . import lib, err_word, stream_ptr, _check
    B, S, H, _ = q.shape
    out = torch.empty(B, S, H, 64, dtype=torch.bfloat16, device=q.device)
    lse2 = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    _check(lib().cm_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse2.data_ptr(), B, S, H, 128, 64,
                             float(scale), err_word(q.device).data_ptr(), stream_ptr()), "cm_attn_fwd")
    F_.count_launch("causal_attention")
    return out, lse2


class CausalAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        from . import fast_contiguous
        q, k, v = fast_contiguous(q), fast_contiguous(k), fast_contiguous(v)
        out, lse2 = attn_fwd_raw(q, k, v, scale)
        ctx.save_for_backward(q, k, v, out, lse2)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import lib, err_word, stream_ptr, _check, fast_contiguous
        q, k, v, out, lse2 = ctx.saved_tensors
        B, S, H, _ = q.shape
        dev = q.device
        dout = fast_contiguous(dout.to(torch.bfloat16))
        delta = torch.empty(B, H, S, dtype=torch.float32, device=dev)
        dq_acc = torch.zeros(B, S, H, 128, dtype=torch.float32, device=dev)      # the kernel reduces query-gradient rows into it
        dk = torch.empty(B, S, H, 128, dtype=torch.bfloat16, device=dev)
        dv = torch.empty(B, S, H, 64, dtype=torch.bfloat16, device=dev)
        _check(lib().cm_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse2.data_ptr(),
                                 delta.data_ptr(), dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, S, H, 128, 64,
                                 float(ctx.scale), err_word(dev).data_ptr(), stream_ptr()), "cm_attn_bwd")
        F_.count_launch("causal_attention_bwd", 2)
        return dq_acc.to(torch.bfloat16), dk, dv, None


def causal_attention(q, k, v, scale: float):
    if not supported(q, k, v):
        F_._miss("causal_attention(shape/dtype)", q)
        return F_.causal_attention_library(q, k, v, scale)
    return CausalAttentionFn.apply(q, k, v, float(scale))


def register() -> None:
    F_.register_cuda("causal_attention", causal_attention)
