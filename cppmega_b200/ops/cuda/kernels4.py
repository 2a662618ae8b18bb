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
    f32 = ctypes.c_float
    sig["cm_sparse_mla_fwd"] = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, vp]
    sig["cm_sparse_mla_bwd"] = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, vp]
    sig["cm_head_reduce"] = [vp, vp, vp, i64, i32, i32, i32, vp]
    sig["cm_indexer_scores"] = [vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]
    sig["cm_indexer_topk"] = [vp, vp, i32, i32, i32, vp]
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


def sparse_mla_fwd_raw(q, kv, idx, scale, d_v):
    from . import lib, err_word, stream_ptr, _check
    B, S, Hq, Dq = q.shape
    Skv, topk = kv.shape[1], idx.shape[-1]
    q, kv = q.contiguous(), kv.contiguous()
    idx = idx.to(torch.int32).contiguous()
    out = torch.empty(B, S, Hq, d_v, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, S, Hq, dtype=torch.float32, device=q.device)
    _check(lib().cm_sparse_mla_fwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, Skv,
                                   Hq, Dq, topk, d_v, float(scale), err_word(q.device).data_ptr(), stream_ptr()),
           "cm_sparse_mla_fwd")
    F_.count_launch("sparse_mla")
    return out, lse


class SparseMLAFn(torch.autograd.Function):
    """Sparse latent attention on the tcgen05 kernels: q [B,S,32,128], kv [B,Skv,128] bf16, idx [B,S,256] int32."""

    @staticmethod
    def forward(ctx, q, kv, idx, scale, d_v, precomputed=None):
        q, kv = q.contiguous(), kv.contiguous()
        idx = idx.to(torch.int32).contiguous()
        out, lse = precomputed if precomputed is not None else sparse_mla_fwd_raw(q, kv, idx, scale, d_v)
        ctx.save_for_backward(q, kv, idx, out, lse)
        ctx.scale, ctx.d_v = float(scale), d_v
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import lib, err_word, stream_ptr, _check
        q, kv, idx, out, lse = ctx.saved_tensors
        B, S, Hq, Dq = q.shape
        Skv, topk = kv.shape[1], idx.shape[-1]
        dout = dout.to(torch.bfloat16).contiguous()
        dq = torch.empty_like(q)
        dkv = torch.zeros(B, Skv, Dq, dtype=torch.float32, device=q.device)
        _check(lib().cm_sparse_mla_bwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                       lse.data_ptr(), dq.data_ptr(), dkv.data_ptr(), B, S, Skv, Hq, Dq, topk, ctx.d_v,
                                       ctx.scale, err_word(q.device).data_ptr(), stream_ptr()), "cm_sparse_mla_bwd")
        F_.count_launch("sparse_mla_bwd")
        return dq, dkv.to(kv.dtype), None, None, None, None


def sparse_mla(q, kv, idx, scale, d_v):
    if (q.dtype != torch.bfloat16 or kv.dtype != torch.bfloat16 or q.dim() != 4 or q.shape[2] != 32 or q.shape[3] != 128
            or kv.shape[-1] != 128 or idx.shape[-1] != 256 or d_v != 64):
        return None
    from ...utils.recompute import stashed_call
    return stashed_call("sparse_mla", lambda: sparse_mla_fwd_raw(q.detach(), kv.detach(), idx, scale, d_v),
                        lambda res: SparseMLAFn.apply(q, kv, idx, scale, d_v, res))


def head_reduce(dh: torch.Tensor, G: int):
    """dh [B,S,H,R,N] bf16 -> (sum over the heads of each group [B,S,G,R,N] bf16, sum over tokens [H,R,N] fp32)."""
    from . import lib, stream_ptr, _check
    B, S, H, R, N = dh.shape
    dgrp = torch.empty(B, S, G, R, N, dtype=torch.bfloat16, device=dh.device)
    dbias = torch.zeros(H, R, N, dtype=torch.float32, device=dh.device)
    _check(lib().cm_head_reduce(dh.data_ptr(), dgrp.data_ptr(), dbias.data_ptr(), B * S, H, G, R * N, stream_ptr()),
           "cm_head_reduce")
    F_.count_launch("head_reduce")
    return dgrp, dbias


def indexer_topk(q_idx, k_idx, w, topk: int):
    """Causal top-k key positions per query (int32 [B,S,topk], unordered, -1 padded) on the indexer kernels."""
    if (q_idx.dtype != torch.bfloat16 or k_idx.dtype != torch.bfloat16 or q_idx.dim() != 4 or q_idx.shape[2] != 32
            or q_idx.shape[3] != 64 or q_idx.shape[1] % 4 or q_idx.shape[1] > 8192 or k_idx.shape[1] != q_idx.shape[1]
            or topk > 2048):
        return None
    from . import lib, err_word, stream_ptr, _check
    B, S = q_idx.shape[:2]
    q, k = q_idx.contiguous(), k_idx.contiguous()
    wf = w.float().contiguous()
    scores = torch.empty(B, S, S, dtype=torch.float32, device=q.device)
    out = torch.empty(B, S, topk, dtype=torch.int32, device=q.device)
    _check(lib().cm_indexer_scores(q.data_ptr(), k.data_ptr(), wf.data_ptr(), scores.data_ptr(), B, S, 32, 64,
                                   err_word(q.device).data_ptr(), stream_ptr()), "cm_indexer_scores")
    _check(lib().cm_indexer_topk(scores.data_ptr(), out.data_ptr(), B, S, topk, stream_ptr()), "cm_indexer_topk")
    F_.count_launch("indexer_topk", 2)
    return out


def register() -> None:
    F_.register_cuda("indexer_topk", indexer_topk)
    F_.register_cuda("angle_cumsum", angle_cumsum)
    F_.register_cuda("sparse_mla", sparse_mla)
