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
    _declare_head_linear(L)


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
    F_.register_cuda("head_linear", head_linear)
    F_.register_cuda("causal_conv1d_silu", causal_conv1d_silu)


# ---------------------------------------------------------------------------
# per-head linear maps of the absorbed sparse-attention path (ops/csrc/head_linear.cu)
# ---------------------------------------------------------------------------

def _declare_head_linear(L: ctypes.CDLL) -> None:
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    for name, args in (("cm_head_linear", [vp, vp, vp, i32, i32, i64, i64, i64, i64, i32, vp, vp]),
                       ("cm_head_linear_wgrad", [vp, vp, vp, i32, i32, i64, i64, i64, i64, vp, vp])):
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = i32


def _token_view(x: torch.Tensor):
    """(tensor, tokens, token stride, head stride) of a [..., H, 64] bf16 operand the kernel can read in place: the
    leading dimensions must collapse to one stride; otherwise the operand is copied to a packed tensor."""
    from . import fast_contiguous
    H = x.shape[-2]
    T = x.numel() // (H * 64)
    lead_sizes, lead_strides = x.shape[:-2], x.stride()[:-2]
    ok = x.stride(-1) == 1 and x.stride(-2) % 8 == 0 and x.data_ptr() % 16 == 0
    tok = None
    if ok:
        tok = lead_strides[-1] if lead_sizes else H * 64
        expect = tok
        for n, s in zip(reversed(lead_sizes), reversed(lead_strides)):
            if n != 1 and s != expect:
                ok = False
                break
            expect *= n
        ok = ok and tok % 8 == 0 and tok >= 64
    if not ok:
        x = fast_contiguous(x)
        return x, T, H * 64, 64
    return x, T, tok, x.stride(-2)


def head_linear_raw(x: torch.Tensor, w: torch.Tensor, transposed: bool) -> torch.Tensor:
    """``y[..., h, :] = x[..., h, :] @ w[h].T`` (``transposed`` False, ``w`` [H, 64 out, 64 in]) or ``x @ w[h]``."""
    from . import lib, err_word, stream_ptr, _check
    xs, T, x_tok, x_head = _token_view(x)
    H = x.shape[-2]
    y = torch.empty(*x.shape[:-1], 64, dtype=torch.bfloat16, device=x.device)
    _check(lib().cm_head_linear(xs.data_ptr(), w.data_ptr(), y.data_ptr(), T, H, x_tok, x_head, H * 64, 64, int(transposed),
                                err_word(x.device).data_ptr(), stream_ptr()), "cm_head_linear")
    F_.count_launch("head_linear")
    return y


class HeadLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        wc = w.contiguous()
        ctx.save_for_backward(x, wc)
        return head_linear_raw(x, wc, False)

    @staticmethod
    def backward(ctx, dy):
        from . import lib, err_word, stream_ptr, _check
        x, wc = ctx.saved_tensors
        dy = dy.to(torch.bfloat16)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = head_linear_raw(dy, wc, True)
        if ctx.needs_input_grad[1]:
            H = x.shape[-2]
            dys, T, dy_tok, dy_head = _token_view(dy)
            xs, _, x_tok, x_head = _token_view(x)
            dw32 = torch.zeros(H, 64, 64, dtype=torch.float32, device=x.device)
            _check(lib().cm_head_linear_wgrad(dys.data_ptr(), xs.data_ptr(), dw32.data_ptr(), T, H, dy_tok, dy_head, x_tok, x_head,
                                              err_word(x.device).data_ptr(), stream_ptr()), "cm_head_linear_wgrad")
            F_.count_launch("head_linear_wgrad")
            dw = dw32.to(wc.dtype)
        return dx, dw


def head_linear(x: torch.Tensor, w: torch.Tensor):
    if (not x.is_cuda or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() < 3 or x.shape[-1] != 64
            or w.dim() != 3 or tuple(w.shape[1:]) != (64, 64) or w.shape[0] != x.shape[-2] or x.numel() == 0):
        return None
    return HeadLinearFn.apply(x, w)


# ---------------------------------------------------------------------------
# depthwise causal conv1d + SiLU, channels-last (ops/csrc/conv1d.cu)
# ---------------------------------------------------------------------------

def _declare_conv(L: ctypes.CDLL) -> None:
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    if getattr(L, "_conv_declared", False):
        return
    L.cm_causal_conv1d_silu_fwd.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i64, vp]
    L.cm_causal_conv1d_silu_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, vp]
    L.cm_causal_conv1d_silu_fwd.restype = L.cm_causal_conv1d_silu_bwd.restype = i32
    L._conv_declared = True


def _conv_view(x: torch.Tensor):
    """(tensor, token stride) for a [B, S, C] bf16 operand the kernel can read in place: channels contiguous, batch stride
    = S * token stride, 16-byte aligned rows; anything else is copied to a packed tensor."""
    B, S, C = x.shape
    sb, ss, sc = x.stride()
    if sc == 1 and ss >= C and ss % 8 == 0 and (B == 1 or sb == S * ss) and x.data_ptr() % 16 == 0:
        return x, ss
    x = x.contiguous()
    return x, C


class CausalConv1dSiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        from . import lib, stream_ptr, _check
        L = lib()
        _declare_conv(L)
        B, S, C = x.shape
        xv, ldx = _conv_view(x)
        wc = w.contiguous()
        bc = None if bias is None else bias.contiguous()
        y = torch.empty(B, S, C, dtype=torch.bfloat16, device=x.device)
        _check(L.cm_causal_conv1d_silu_fwd(xv.data_ptr(), wc.data_ptr(), None if bc is None else bc.data_ptr(), y.data_ptr(),
                                           B, S, C, wc.shape[1], ldx, stream_ptr()), "cm_causal_conv1d_silu_fwd")
        F_.count_launch("causal_conv1d_silu")
        ctx.save_for_backward(x, wc, bc if bc is not None else wc.new_empty(0))
        ctx.has_bias = bc is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import lib, stream_ptr, _check
        L = lib()
        x, w, bias = ctx.saved_tensors
        B, S, C = x.shape
        k = w.shape[1]
        xv, ldx = _conv_view(x)
        dy = dy.contiguous()
        g = torch.empty(B, S, C, dtype=torch.bfloat16, device=x.device)
        dx = torch.empty(B, S, C, dtype=torch.bfloat16, device=x.device)
        dw = torch.zeros(C, k, dtype=torch.float32, device=x.device)
        db = torch.zeros(C, dtype=torch.float32, device=x.device)
        _check(L.cm_causal_conv1d_silu_bwd(xv.data_ptr(), w.data_ptr(), bias.data_ptr() if ctx.has_bias else None, dy.data_ptr(),
                                           g.data_ptr(), dx.data_ptr(), dw.data_ptr(), db.data_ptr(), B, S, C, k, ldx, C,
                                           stream_ptr()), "cm_causal_conv1d_silu_bwd")
        F_.count_launch("causal_conv1d_silu_bwd", 2)
        return dx, dw.to(w.dtype), (db.to(bias.dtype) if ctx.has_bias else None)


def causal_conv1d_silu(x, w, bias):
    """x [B, S, C] bf16 (may be a column slice of a wider projection), w [C, k] bf16, bias [C] bf16 or None."""
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16)
            or x.dim() != 3 or x.shape[2] % 8 or not 1 <= w.shape[1] <= 8 or x.numel() == 0):
        F_._miss("causal_conv1d_silu(shape/dtype)", x)
        return None
    return CausalConv1dSiluFn.apply(x, w, bias)
