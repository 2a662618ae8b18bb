"""MXFP8 tensors and the block-scaled linear.

``quantize_rowwise`` / ``quantize_colwise`` / ``dequantize`` / ``swizzle_scales`` wrap the kernels in
``csrc/mxfp8.cu``.  :class:`Mxfp8LinearFn` is the linear layer of the ``mxfp8`` precision recipe: every operand of
the three products (forward, dgrad, wgrad) is rounded to MXFP8 along the dimension that product reduces over - the
contract of the reference's MXFP8 GEMM wrappers (``tn_gemm`` / ``dgrad_nn_gemm`` / ``wgrad_nt_gemm``,
cppmega/megatron/cutlass_mxfp8_gemm.py:102,249,506) - and the activation saved for the weight gradient is kept as an
MXFP8 tensor (1 byte per value + 1/32 scale), which is what the reference's FP8 activation pack saves
(cppmega/megatron/fp8_activations.py).  The products themselves run on the bf16 tcgen05 GEMM over the dequantised
operands: same numerics as a block-scaled GEMM up to accumulation order, bf16 tensor-core rate.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Tuple

import torch

from .. import functional as F_


@dataclass
class Mxfp8Tensor:
    payload: torch.Tensor          # uint8 (E4M3 bit patterns), [rows, cols] of the *stored* orientation
    scales: torch.Tensor           # uint8 (E8M0), [rows, cols / 32]
    shape: Tuple[int, int]         # logical [rows, cols] of the stored orientation

    def nbytes(self) -> int:
        return self.payload.numel() + self.scales.numel()

    def dequantize(self) -> torch.Tensor:
        return dequantize(self)


def _lib():
    from . import lib
    L = lib()
    if not getattr(L, "_mx_declared", False):
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        L.cm_mxfp8_quantize_rowwise.argtypes = [vp, vp, vp, i64, i32, vp]
        L.cm_mxfp8_quantize_colwise.argtypes = [vp, vp, vp, i64, i32, vp]
        L.cm_mxfp8_dequantize.argtypes = [vp, vp, vp, i64, vp]
        L.cm_mxfp8_swizzle_scales.argtypes = [vp, vp, i64, i32, vp]
        for n in ("cm_mxfp8_quantize_rowwise", "cm_mxfp8_quantize_colwise", "cm_mxfp8_dequantize", "cm_mxfp8_swizzle_scales"):
            getattr(L, n).restype = i32
        L._mx_declared = True
    return L


def _check(rc, what):
    if rc:
        raise RuntimeError(f"{what} failed ({rc})")


def quantize_rowwise(x: torch.Tensor) -> Mxfp8Tensor:
    """Blocks of 32 along the last dimension of a 2-D bf16 tensor."""
    from . import stream_ptr
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.shape[1] % 32 == 0
    x = x.contiguous()
    rows, cols = x.shape
    pay = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    sc = torch.empty(rows, cols // 32, dtype=torch.uint8, device=x.device)
    _check(_lib().cm_mxfp8_quantize_rowwise(x.data_ptr(), pay.data_ptr(), sc.data_ptr(), rows, cols, stream_ptr()),
           "cm_mxfp8_quantize_rowwise")
    F_.count_launch("mxfp8_quantize")
    return Mxfp8Tensor(pay, sc, (rows, cols))


def quantize_colwise(x: torch.Tensor) -> Mxfp8Tensor:
    """Blocks of 32 along the rows; the result is stored transposed: payload [cols, rows], scales [cols, rows/32]."""
    from . import stream_ptr
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.shape[0] % 32 == 0
    x = x.contiguous()
    rows, cols = x.shape
    pay = torch.empty(cols, rows, dtype=torch.uint8, device=x.device)
    sc = torch.empty(cols, rows // 32, dtype=torch.uint8, device=x.device)
    _check(_lib().cm_mxfp8_quantize_colwise(x.data_ptr(), pay.data_ptr(), sc.data_ptr(), rows, cols, stream_ptr()),
           "cm_mxfp8_quantize_colwise")
    F_.count_launch("mxfp8_quantize")
    return Mxfp8Tensor(pay, sc, (cols, rows))


def dequantize(t: Mxfp8Tensor) -> torch.Tensor:
    from . import stream_ptr
    out = torch.empty(t.shape, dtype=torch.bfloat16, device=t.payload.device)
    _check(_lib().cm_mxfp8_dequantize(t.payload.data_ptr(), t.scales.data_ptr(), out.data_ptr(), t.payload.numel(),
                                      stream_ptr()), "cm_mxfp8_dequantize")
    F_.count_launch("mxfp8_dequantize")
    return out


def swizzle_scales(scales: torch.Tensor) -> torch.Tensor:
    """Row-major [rows, kb] scale bytes -> flat 128x4-tiled buffer (padded with the neutral scale 127)."""
    from . import stream_ptr
    rows, kb = scales.shape
    out = torch.empty(((rows + 127) // 128) * ((kb + 3) // 4) * 512, dtype=torch.uint8, device=scales.device)
    _check(_lib().cm_mxfp8_swizzle_scales(scales.contiguous().data_ptr(), out.data_ptr(), rows, kb, stream_ptr()),
           "cm_mxfp8_swizzle_scales")
    return out


def eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    rows = x.numel() // x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2
            and x.shape[-1] % 32 == 0 and w.shape[0] % 32 == 0 and rows % 32 == 0 and rows > 0)


class Mxfp8LinearFn(torch.autograd.Function):
    """y = q_K(x) q_K(W)^T;  dx = q_N(dy) q_N(W);  dW = q_T(dy)^T q_T(x)  (q_D: MXFP8 rounding along D)."""

    @staticmethod
    def forward(ctx, x, w):
        from . import gemm
        x2 = x.reshape(-1, x.shape[-1])
        xq = quantize_rowwise(x2)                       # along K
        wq = quantize_rowwise(w)                        # along K
        y = gemm(dequantize(xq), dequantize(wq))
        x_t = quantize_colwise(x2)                      # [K, T] along tokens: the wgrad operand, kept in 1 byte/value
        ctx.save_for_backward(x_t.payload, x_t.scales, w)
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import gemm, wgrad_into_main_grad
        xt_pay, xt_sc, w = ctx.saved_tensors
        K, T = xt_pay.shape
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq = dequantize(quantize_rowwise(dy2))                      # along N
            w_t = dequantize(quantize_colwise(w))                        # [K, N] along N
            dx = gemm(dyq, w_t).view(ctx.xshape)                          # [T,N] x [K,N]^T
        if ctx.needs_input_grad[1]:
            dy_t = dequantize(quantize_colwise(dy2))                     # [N, T] along tokens
            x_t = dequantize(Mxfp8Tensor(xt_pay, xt_sc, (K, T)))         # [K, T]
            dw = wgrad_into_main_grad(w, lambda out, acc: gemm(dy_t, x_t, out=out, accumulate=acc))
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor):
    if not eligible(x, w):
        return None
    return Mxfp8LinearFn.apply(x, w)
