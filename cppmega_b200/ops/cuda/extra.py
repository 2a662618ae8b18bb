"""Wrappers for the grouped expert GEMMs and the chunked fused linear cross-entropy."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import functional as F_

TILE = 128


def declare(L: ctypes.CDLL) -> None:
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    sig = {
        "cm_ce_fwd_bwd": [vp, vp, vp, vp, vp, i32, i32, i64, i32, i32, vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = i32
    from . import kernels2
    kernels2.declare(L)


# ---------------------------------------------------------------------------
# grouped experts on the padded layout
# ---------------------------------------------------------------------------

def padded_plan(counts: torch.Tensor, total_rows: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """From per-expert row counts (device, no host sync) derive the 128-row aligned layout:
    returns (dst_row [total_rows] for expert-sorted rows, tile_expert [max_tiles] int32,
    seg_offsets [E+1] int32, max_rows)."""
    E = counts.numel()
    max_rows = (total_rows + E * (TILE - 1) + TILE - 1) // TILE * TILE
    c = counts.to(torch.int64)
    padded = (c + (TILE - 1)) // TILE * TILE
    seg_end = torch.cumsum(padded, 0)
    seg_start = seg_end - padded
    un_end = torch.cumsum(c, 0)
    un_start = un_end - c
    rows = torch.arange(total_rows, device=counts.device)
    e_of_row = torch.searchsorted(un_end, rows, right=True).clamp_(max=E - 1)
    dst_row = seg_start[e_of_row] + (rows - un_start[e_of_row])
    tiles = torch.arange(max_rows // TILE, device=counts.device) * TILE
    te = torch.searchsorted(seg_end, tiles, right=True)
    tile_expert = torch.where(te < E, te, torch.full_like(te, -1)).to(torch.int32)
    seg_offsets = torch.cat([seg_start[:1], seg_end]).to(torch.int32)
    return dst_row, tile_expert, seg_offsets, max_rows


class GroupedLinearFn(torch.autograd.Function):
    """y[r] = x[r] @ W[e(r)]^T on the padded layout; W is [E, N, K]."""

    @staticmethod
    def forward(ctx, xp, w, tile_expert, seg_offsets):
        from . import lib, err_word, stream_ptr, _check
        rows, K = xp.shape
        E, N, _ = w.shape
        y = torch.empty(rows, N, dtype=xp.dtype, device=xp.device)
        _check(lib().cm_grouped_gemm_rows_bf16(xp.data_ptr(), w.data_ptr(), y.data_ptr(), rows, N, K, E, 0,
                                               tile_expert.data_ptr(), err_word(xp.device).data_ptr(), stream_ptr()),
               "cm_grouped_gemm_rows_bf16")
        F_.count_launch("grouped_gemm")
        ctx.save_for_backward(xp, w, tile_expert, seg_offsets)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import lib, err_word, stream_ptr, _check
        xp, w, tile_expert, seg_offsets = ctx.saved_tensors
        rows, K = xp.shape
        E, N, _ = w.shape
        dy = dy.contiguous()
        dx = dw = None
        err = err_word(xp.device).data_ptr()
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(xp)
            # reduction over N, output width K: W [E, N, K] is the "MN-major" B operand
            _check(lib().cm_grouped_gemm_rows_bf16(dy.data_ptr(), w.data_ptr(), dx.data_ptr(), rows, K, N, E, 1,
                                                   tile_expert.data_ptr(), err, stream_ptr()),
                   "cm_grouped_gemm_rows_bf16(dgrad)")
            F_.count_launch("grouped_gemm")
        if ctx.needs_input_grad[1]:
            from . import wgrad_into_main_grad

            def run(out, acc):
                out = torch.empty_like(w) if out is None else out
                _check(lib().cm_grouped_gemm_k_bf16(dy.data_ptr(), xp.data_ptr(), out.data_ptr(), rows, N, K, E,
                                                    seg_offsets.data_ptr(), int(out.dtype == torch.float32), int(acc), err,
                                                    stream_ptr()), "cm_grouped_gemm_k_bf16")
                F_.count_launch("grouped_gemm")
                return out
            dw = wgrad_into_main_grad(w, run)
        return dx, dw, None, None


def moe_experts(x_sorted: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, counts: torch.Tensor):
    """Expert-sorted rows -> SwiGLU expert MLP -> rows in the same order."""
    if (x_sorted.dtype != torch.bfloat16 or w1.dtype != torch.bfloat16 or x_sorted.shape[1] % 8
            or w1.shape[1] % 16 or x_sorted.shape[0] == 0):
        return None
    from . import swiglu
    dst_row, tile_expert, seg_offsets, max_rows = padded_plan(counts, x_sorted.shape[0])
    xp = torch.zeros(max_rows, x_sorted.shape[1], dtype=x_sorted.dtype, device=x_sorted.device)
    xp = xp.index_copy(0, dst_row, x_sorted)
    h = GroupedLinearFn.apply(xp, w1, tile_expert, seg_offsets)
    h = swiglu(h)
    y = GroupedLinearFn.apply(h, w2, tile_expert, seg_offsets)
    return y.index_select(0, dst_row)


# ---------------------------------------------------------------------------
# fused linear + cross-entropy (chunked, gradients produced in the forward pass)
# ---------------------------------------------------------------------------

class LinearCEWeightedFn(torch.autograd.Function):
    """L = sum_t weight_t * CE(h_t W^T, label_t).  Returns (L, per-token loss).  Logits exist one
    chunk at a time in bf16; dlogits overwrite them in place and feed the dgrad/wgrad GEMMs, so
    the backward pass only rescales by the upstream scalar."""

    CHUNK = 4096

    @staticmethod
    def forward(ctx, h, w, labels, weights, ignore_index):
        from . import gemm, lib, stream_ptr, _check
        T, H = h.shape
        V = w.shape[0]
        need_grad = h.requires_grad or w.requires_grad
        per_tok = torch.empty(T, dtype=torch.float32, device=h.device)
        dh = torch.empty_like(h) if need_grad else None
        dw = torch.zeros(V, H, dtype=torch.float32, device=h.device) if need_grad else None
        labels = labels.to(torch.int64).contiguous()
        weights = weights.to(torch.float32).contiguous()
        C = LinearCEWeightedFn.CHUNK
        logits = torch.empty(min(C, T), V, dtype=torch.bfloat16, device=h.device)
        for s in range(0, T, C):
            e = min(s + C, T)
            n = e - s
            lg = logits[:n]
            gemm(h[s:e], w, out=lg)
            _check(lib().cm_ce_fwd_bwd(lg.data_ptr(), labels[s:e].data_ptr(), weights[s:e].data_ptr(),
                                       per_tok[s:e].data_ptr(), None, n, V, V, int(ignore_index), int(need_grad),
                                       stream_ptr()), "cm_ce_fwd_bwd")
            F_.count_launch("cross_entropy")
            if need_grad:
                gemm(lg, w, b_mn=True, out=dh[s:e])
                gemm(lg, h[s:e], a_mn=True, b_mn=True, out=dw, accumulate=True)
        total = (per_tok * weights).sum()
        if need_grad:
            ctx.save_for_backward(dh, dw)
        ctx.w_dtype = w.dtype
        ctx.mark_non_differentiable(per_tok)
        return total, per_tok

    @staticmethod
    def backward(ctx, g_total, _g_per_tok):
        dh, dw = ctx.saved_tensors
        return dh * g_total.to(dh.dtype), (dw * g_total).to(ctx.w_dtype), None, None, None


def linear_cross_entropy_weighted(h, w, labels, weights, ignore_index):
    if h.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[0] % 8 or h.shape[1] % 8:
        return None
    return LinearCEWeightedFn.apply(h.contiguous(), w, labels, weights, ignore_index)


def register() -> None:
    F_.register_cuda("moe_experts", moe_experts)
    F_.register_cuda("linear_cross_entropy_weighted", linear_cross_entropy_weighted)
    from . import kernels2
    kernels2.register()


_ = Optional
