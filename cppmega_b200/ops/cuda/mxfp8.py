"""MXFP8 tensors and the block-scaled linear.

``quantize_rowwise`` / ``quantize_colwise`` / ``dequantize`` / ``swizzle_scales`` wrap the kernels in
``csrc/mxfp8.cu``.  :class:`Mxfp8LinearFn` is the linear layer of the ``mxfp8`` precision recipe: every operand of
the three products (forward, dgrad, wgrad) is rounded to MXFP8 along the dimension that product reduces over - the
contract of the reference's MXFP8 GEMM wrappers (``tn_gemm`` / ``dgrad_nn_gemm`` / ``wgrad_nt_gemm``,
cppmega/megatron/cutlass_mxfp8_gemm.py:102,249,506) - and the activation saved for the weight gradient is kept as an
MXFP8 tensor (1 byte per value + 1/32 scale), which is what the reference's FP8 activation pack saves
(cppmega/megatron/fp8_activations.py).  The products run on the block-scaled tensor-core GEMM of
``csrc/mxfp8_gemm.cu`` (:func:`gemm_mxfp8`: ``tcgen05.mma.kind::mxf8f6f4.block_scale`` with the scale bytes in TMEM),
every one of them as a "TN" product of two operands quantised along the reduction dimension.
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
    _swizzled: torch.Tensor = None  # scales in the 128x4 tile order the tensor cores read (made on first use)

    def swizzled(self) -> torch.Tensor:
        if self._swizzled is None:
            self._swizzled = swizzle_scales(self.scales)
        return self._swizzled

    def nbytes(self) -> int:
        return self.payload.numel() + self.scales.numel()

    def dequantize(self) -> torch.Tensor:
        return dequantize(self)


def _lib():
    from . import lib
    L = lib()
    if not getattr(L, "_mx_declared", False):
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        L.cm_mxfp8_quantize_rowwise.argtypes = [vp, vp, vp, vp, i64, i32, vp, vp]
        L.cm_mxfp8_quantize_colwise.argtypes = [vp, vp, vp, vp, i64, i32, vp, vp]
        L.cm_amax_bf16.argtypes = [vp, i64, vp, vp]
        L.cm_amax_bf16.restype = i32
        L.cm_mxfp8_dequantize.argtypes = [vp, vp, vp, i64, vp]
        L.cm_mxfp8_swizzle_scales.argtypes = [vp, vp, i64, i32, vp]
        L.cm_mxfp8_quantize_both.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i32, vp, vp]
        L.cm_mxfp8_grouped_rows.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp]
        L.cm_mxfp8_grouped_k.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, i32, i32, vp, vp]
        L.cm_mxfp8_gemm.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, i32, vp, vp]
        for n in ("cm_mxfp8_quantize_rowwise", "cm_mxfp8_quantize_colwise", "cm_mxfp8_dequantize", "cm_mxfp8_swizzle_scales",
                  "cm_mxfp8_gemm", "cm_mxfp8_quantize_both", "cm_mxfp8_grouped_rows", "cm_mxfp8_grouped_k"):
            getattr(L, n).restype = i32
        L._mx_declared = True
    return L


def _check(rc, what):
    if rc:
        raise RuntimeError(f"{what} failed ({rc})")


def _swizzled_buffer(rows: int, kb: int, device) -> torch.Tensor:
    n = ((rows + 127) // 128) * ((kb + 3) // 4) * 512
    if rows % 128 or kb % 4:                       # padding entries keep the neutral scale
        return torch.full((n,), 127, dtype=torch.uint8, device=device)
    return torch.empty(n, dtype=torch.uint8, device=device)


def tensor_amax(x: torch.Tensor) -> torch.Tensor:
    """Device scalar max |x| of a bf16 tensor (one pass, no host sync): the scale source of the tensorwise recipe."""
    from . import stream_ptr
    x = x.contiguous()
    out = torch.zeros(1, dtype=torch.float32, device=x.device)
    if x.numel() % 8:
        out.copy_(x.abs().max().float())
        return out
    _check(_lib().cm_amax_bf16(x.data_ptr(), x.numel(), out.data_ptr(), stream_ptr()), "cm_amax_bf16")
    F_.count_launch("fp8_amax")
    return out


def _amax_ptr(x: torch.Tensor, tensorwise):
    """``tensorwise``: False / None (block scales), True (measure the tensor's amax now), or a device scalar."""
    if tensorwise is None or tensorwise is False:
        return None, None
    am = tensor_amax(x) if tensorwise is True else tensorwise
    return am, am.data_ptr()


def quantize_rowwise(x: torch.Tensor, for_gemm: bool = False, tensorwise=None) -> Mxfp8Tensor:
    """Blocks of 32 along the last dimension of a 2-D bf16 tensor.  ``for_gemm`` also writes the scales in the tile
    order the block-scaled GEMM reads, from the same kernel.  ``tensorwise``: one power-of-two scale for the whole
    tensor (written into every scale byte) instead of one per block."""
    from . import stream_ptr
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.shape[1] % 32 == 0
    x = x.contiguous()
    rows, cols = x.shape
    pay = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    sc = torch.empty(rows, cols // 32, dtype=torch.uint8, device=x.device)
    sw = _swizzled_buffer(rows, cols // 32, x.device) if for_gemm else None
    _am, amp = _amax_ptr(x, tensorwise)
    _check(_lib().cm_mxfp8_quantize_rowwise(x.data_ptr(), pay.data_ptr(), sc.data_ptr(), sw.data_ptr() if for_gemm else None,
                                            rows, cols, amp, stream_ptr()), "cm_mxfp8_quantize_rowwise")
    F_.count_launch("mxfp8_quantize")
    return Mxfp8Tensor(pay, sc, (rows, cols), sw)


def quantize_colwise(x: torch.Tensor, for_gemm: bool = False, tensorwise=None) -> Mxfp8Tensor:
    """Blocks of 32 along the rows; the result is stored transposed: payload [cols, rows], scales [cols, rows/32]."""
    from . import stream_ptr
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.shape[0] % 32 == 0
    x = x.contiguous()
    rows, cols = x.shape
    pay = torch.empty(cols, rows, dtype=torch.uint8, device=x.device)
    sc = torch.empty(cols, rows // 32, dtype=torch.uint8, device=x.device)
    sw = _swizzled_buffer(cols, rows // 32, x.device) if for_gemm else None
    _am, amp = _amax_ptr(x, tensorwise)
    _check(_lib().cm_mxfp8_quantize_colwise(x.data_ptr(), pay.data_ptr(), sc.data_ptr(), sw.data_ptr() if for_gemm else None,
                                            rows, cols, amp, stream_ptr()), "cm_mxfp8_quantize_colwise")
    F_.count_launch("mxfp8_quantize")
    return Mxfp8Tensor(pay, sc, (cols, rows), sw)


def quantize_both(x: torch.Tensor, for_gemm: bool = True, tensorwise=None):
    """Row-wise and transposed column-wise MXFP8 copies of a 2-D bf16 tensor from one read of it."""
    from . import stream_ptr
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.shape[0] % 32 == 0 and x.shape[1] % 32 == 0
    x = x.contiguous()
    rows, cols = x.shape
    dev = x.device
    pay_r = torch.empty(rows, cols, dtype=torch.uint8, device=dev)
    sc_r = torch.empty(rows, cols // 32, dtype=torch.uint8, device=dev)
    pay_t = torch.empty(cols, rows, dtype=torch.uint8, device=dev)
    sc_t = torch.empty(cols, rows // 32, dtype=torch.uint8, device=dev)
    sw_r = _swizzled_buffer(rows, cols // 32, dev) if for_gemm else None
    sw_t = _swizzled_buffer(cols, rows // 32, dev) if for_gemm else None
    ptr = lambda t: t.data_ptr() if t is not None else None
    _am, amp = _amax_ptr(x, tensorwise)
    _check(_lib().cm_mxfp8_quantize_both(x.data_ptr(), pay_r.data_ptr(), sc_r.data_ptr(), ptr(sw_r), pay_t.data_ptr(),
                                         sc_t.data_ptr(), ptr(sw_t), rows, cols, amp, stream_ptr()), "cm_mxfp8_quantize_both")
    F_.count_launch("mxfp8_quantize")
    return Mxfp8Tensor(pay_r, sc_r, (rows, cols), sw_r), Mxfp8Tensor(pay_t, sc_t, (cols, rows), sw_t)


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


def gemm_mxfp8(a: Mxfp8Tensor, b: Mxfp8Tensor, out: torch.Tensor = None, accumulate: bool = False,
               out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``a [M,K] . b [N,K]^T`` with both operands quantised along K; bf16 result, or fp32 (optionally added to ``out``)."""
    from . import err_word, stream_ptr
    (M, K), (N, K2) = a.shape, b.shape
    assert K == K2 and K % 32 == 0
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, dtype=out_dtype, device=a.payload.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    sfa, sfb = a.swizzled(), b.swizzled()
    _check(_lib().cm_mxfp8_gemm(a.payload.data_ptr(), sfa.data_ptr(), b.payload.data_ptr(), sfb.data_ptr(), out.data_ptr(), M, N, K,
                                a.payload.stride(0), b.payload.stride(0), out.stride(0), int(out.dtype == torch.float32),
                                int(accumulate), err_word(out.device).data_ptr(), stream_ptr()), "cm_mxfp8_gemm")
    F_.count_launch("mxfp8_gemm")
    return out


def eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    rows = x.numel() // x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2
            and x.shape[-1] % 32 == 0 and w.shape[0] % 32 == 0 and rows % 32 == 0 and rows > 0)


def quantize_weight(w: torch.Tensor, colwise: bool, tensorwise: bool = False) -> Mxfp8Tensor:
    """FP8 copy of a parameter, kept on the parameter until the optimizer next writes it (``_version`` changes), so
    the replayed forward of a recomputed layer and every micro-batch of a step reuse one quantisation."""
    key = ("_tw_col" if colwise else "_tw_row") if tensorwise else ("_mx_col" if colwise else "_mx_row")
    hit = getattr(w, key, None)
    if hit is not None and hit[0] == w._version:
        return hit[1]
    tw = True if tensorwise else None
    q = quantize_colwise(w.detach(), True, tw) if colwise else quantize_rowwise(w.detach(), True, tw)
    try:
        setattr(w, key, (w._version, q))
    except AttributeError:
        pass
    return q


def quantize_expert_weights(w: torch.Tensor, transposed: bool, tensorwise: bool = False) -> Mxfp8Tensor:
    """FP8 copy of a stacked expert weight [E, N, K], cached until the optimizer writes it.  ``transposed`` False:
    [E * N, K] quantised along K (forward operand).  True: the stack read as [E * N, K] and quantised along its rows,
    stored transposed [K, E * N] - the dgrad operand, whose reduction axis is N and whose expert e occupies the
    columns [e N, (e + 1) N).  ``tensorwise``: one scale for the whole stack."""
    key = ("_tw_ecol" if transposed else "_tw_erow") if tensorwise else ("_mx_ecol" if transposed else "_mx_erow")
    hit = getattr(w, key, None)
    if hit is not None and hit[0] == w._version:
        return hit[1]
    w2 = w.detach().reshape(-1, w.shape[-1])
    tw = True if tensorwise else None
    q = quantize_colwise(w2, True, tw) if transposed else quantize_rowwise(w2, True, tw)
    try:
        setattr(w, key, (w._version, q))
    except AttributeError:
        pass
    return q


def grouped_rows_mxfp8(xq: Mxfp8Tensor, wq: Mxfp8Tensor, tile_expert: torch.Tensor, num_experts: int, n_out: int, dgrad: bool,
                       out: torch.Tensor = None) -> torch.Tensor:
    """Expert forward (``wq`` = stacked [E * n_out, K]) or dgrad (``wq`` = transposed stack [n_out, E * K]) on the padded
    expert-sorted rows of ``xq`` [rows, K]."""
    from . import err_word, stream_ptr
    rows, K = xq.shape
    if out is None:
        out = torch.empty(rows, n_out, dtype=torch.bfloat16, device=xq.payload.device)
    _check(_lib().cm_mxfp8_grouped_rows(xq.payload.data_ptr(), xq.swizzled().data_ptr(), wq.payload.data_ptr(), wq.swizzled().data_ptr(),
                                        out.data_ptr(), rows, n_out, K, num_experts, int(dgrad), tile_expert.data_ptr(),
                                        err_word(out.device).data_ptr(), stream_ptr()), "cm_mxfp8_grouped_rows")
    F_.count_launch("mxfp8_grouped_gemm")
    return out


def grouped_wgrad_mxfp8(dy_t: Mxfp8Tensor, x_t: Mxfp8Tensor, seg_offsets: torch.Tensor, num_experts: int, out: torch.Tensor = None,
                        accumulate: bool = False) -> torch.Tensor:
    """dW[e] [N, K] (+)= dy_e^T x_e from the token-transposed operands dy_t [N, R], x_t [K, R]."""
    from . import err_word, stream_ptr
    (N, R), (K, R2) = dy_t.shape, x_t.shape
    assert R == R2
    if out is None:
        out = torch.empty(num_experts, N, K, dtype=torch.bfloat16, device=dy_t.payload.device)
        accumulate = False
    assert out.is_contiguous() and out.dtype in (torch.bfloat16, torch.float32)
    _check(_lib().cm_mxfp8_grouped_k(dy_t.payload.data_ptr(), dy_t.swizzled().data_ptr(), x_t.payload.data_ptr(), x_t.swizzled().data_ptr(),
                                     out.data_ptr(), R, N, K, num_experts, seg_offsets.data_ptr(), int(out.dtype == torch.float32),
                                     int(accumulate), err_word(out.device).data_ptr(), stream_ptr()), "cm_mxfp8_grouped_k")
    F_.count_launch("mxfp8_grouped_gemm")
    return out


class Mxfp8LinearFn(torch.autograd.Function):
    """y = q_K(x) q_K(W)^T;  dx = q_N(dy) q_N(W);  dW = q_T(dy)^T q_T(x)  (q_D: FP8 rounding along D).  ``tensorwise``:
    one power-of-two scale per tensor (measured from the tensor itself: current scaling) instead of one per 32 values;
    the row-wise and transposed copies of one tensor share the measured amax."""

    @staticmethod
    def forward(ctx, x, w, tensorwise=False):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        tw = tensor_amax(x2) if tensorwise else None
        xq, x_t = quantize_both(x2, True, tw)           # along K, and [K, T] along tokens: the wgrad operand (1 byte/value)
        wq = quantize_weight(w, colwise=False, tensorwise=tensorwise)          # along K
        y = gemm_mxfp8(xq, wq)
        ctx.save_for_backward(x_t.payload, x_t.scales, x_t._swizzled, w)
        ctx.xshape = x.shape
        ctx.tensorwise = tensorwise
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import wgrad_into_main_grad
        xt_pay, xt_sc, xt_sw, w = ctx.saved_tensors
        K, T = xt_pay.shape
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        tw = tensor_amax(dy2) if ctx.tensorwise else None
        dx = dw = None
        dyq = dy_t = None
        if ctx.needs_input_grad[0] and ctx.needs_input_grad[1]:
            dyq, dy_t = quantize_both(dy2, True, tw)                     # one read of dy for both products
        if ctx.needs_input_grad[0]:
            dyq = dyq if dyq is not None else quantize_rowwise(dy2, True, tw)   # along N
            w_t = quantize_weight(w, colwise=True, tensorwise=ctx.tensorwise)   # [K, N] along N
            dx = gemm_mxfp8(dyq, w_t).view(ctx.xshape)                   # [T,N] x [K,N]^T
        if ctx.needs_input_grad[1]:
            dy_t = dy_t if dy_t is not None else quantize_colwise(dy2, True, tw)   # [N, T] along tokens
            x_t = Mxfp8Tensor(xt_pay, xt_sc, (K, T), xt_sw)              # [K, T]
            dw = wgrad_into_main_grad(w, lambda out, acc: _wgrad(dy_t, x_t, out, acc))
        return dx, dw, None


def _wgrad(dy_t: Mxfp8Tensor, x_t: Mxfp8Tensor, out, accumulate: bool):
    """dW [N,K] = dy^T x over tokens, written or accumulated into ``out`` (fp32 or bf16 main grad) or returned as bf16."""
    if out is None:
        return gemm_mxfp8(dy_t, x_t)
    return gemm_mxfp8(dy_t, x_t, out=out, accumulate=accumulate)


def linear(x: torch.Tensor, w: torch.Tensor, tensorwise: bool = False):
    if not eligible(x, w):
        return None
    return Mxfp8LinearFn.apply(x, w, tensorwise)
