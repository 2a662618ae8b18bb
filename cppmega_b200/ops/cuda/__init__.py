"""ctypes front-end of the sm_100a kernel library and its autograd wrappers.

Importing this module loads ``libcppmega_b200_kernels.so`` (built in-tree by
``python -m cppmega_b200.ops.cuda.build``) and registers the CUDA implementations with
:mod:`cppmega_b200.ops.functional`.  If a GPU is present and the library is missing, the
import raises: there is no silent PyTorch fallback on a GPU box.
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Optional

import torch

from .. import functional as F_

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libcppmega_b200_kernels.so"
_lib: Optional[ctypes.CDLL] = None
_err_words = {}

ERROR_NAMES = {1: "TMA stage never arrived", 2: "pipeline stage never released", 3: "accumulator never completed",
               4: "accumulator never released", 5: "peer flag never set", 6: "bad argument"}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH.name} is missing; run `python -m cppmega_b200.ops.cuda.build` (needs nvcc, no GPU)")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    sig = {
        "cm_gemm_bf16": [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, i32, i32, i32, vp, vp],
        "cm_grouped_gemm_rows_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp],
        "cm_grouped_gemm_k_bf16": [vp, vp, vp, i32, i32, i32, i32, vp, i32, i32, vp, vp],
        "cm_rmsnorm_fwd": [vp, vp, vp, vp, i32, i32, f32, vp],
        "cm_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, i32, i32, vp],
        "cm_swiglu_fwd": [vp, vp, i64, i32, vp],
        "cm_swiglu_bwd": [vp, vp, vp, i64, i32, vp],
        "cm_swiglu_fwd_rows": [vp, vp, i64, i32, vp, vp],
        "cm_swiglu_bwd_rows": [vp, vp, vp, i64, i32, vp, vp],
        "cm_adamw": [vp, vp, vp, vp, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, f32, i32, i32, vp],
        "cm_adamw_gated": [vp, vp, vp, vp, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, f32, i32, i32, vp, vp],
        "cm_sumsq": [vp, i64, vp, i32, vp],
        "cm_strided_copy": [vp, vp, vp, vp, vp, i64, vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = i32
    from . import attention, extra, kernels4
    extra.declare(L)
    kernels4.declare(L)
    attention.declare(L)


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def err_word(device: Optional[torch.device] = None) -> torch.Tensor:
    """Per-device int32 that kernels write when a bounded wait runs out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _err_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _err_words[key] = t
    return t


def check_errors(device: Optional[torch.device] = None) -> None:
    """Synchronising read of the error word; raises :class:`KernelError` if a kernel gave up."""
    t = err_word(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise KernelError(f"sm_100a kernel aborted: {ERROR_NAMES.get(code, code)} (code {code})")


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------

def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, accumulate: bool = False) -> torch.Tensor:
    """``C[M,N] = op(A) op(B)``.  ``a`` is [M,K] (or [K,M] when ``a_mn``); ``b`` is [N,K] (or [K,N]
    when ``b_mn``).  bf16 inputs, fp32 accumulation in TMEM, bf16 or fp32 output."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    K, M = (a.shape if a_mn else a.shape[::-1])
    Kb, N = (b.shape if b_mn else b.shape[::-1])
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    assert out.stride(1) == 1
    rc = lib().cm_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                            out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate),
                            err_word(a.device).data_ptr(), stream_ptr())
    _check(rc, "cm_gemm_bf16")
    F_.count_launch("gemm")
    return out


def _gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
            and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0 and x.numel() > 0)


class LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        y = gemm(x2, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = wgrad_into_main_grad(w, lambda out, acc: gemm(dy2, x2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        return dx, dw


def _collapse(sizes, sstr, dstr):
    """Drop unit dimensions and merge neighbours that are contiguous in both tensors."""
    dims = [(n, a, b) for n, a, b in zip(sizes, sstr, dstr) if n != 1]
    out = []
    for n, a, b in dims:
        if out and out[-1][1] == a * n and out[-1][2] == b * n:
            pn, _, _ = out[-1]
            out[-1] = (pn * n, a, b)
        else:
            out.append((n, a, b))
    return out


def fast_copy_(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``dst.copy_(src)`` for same-dtype CUDA tensors whose innermost run is contiguous on both sides, as one launch
    of 16-byte vector moves.  The library's generic strided copy moves such views (slices of a packed projection,
    head splits) element by element at a fraction of the memory bandwidth.  Anything else falls through to ``copy_``."""
    if (not (dst.is_cuda and src.is_cuda) or dst.dtype != src.dtype or dst.shape != src.shape or dst.numel() == 0
            or dst.device != src.device):
        return dst.copy_(src)
    es = dst.element_size()
    dims = _collapse(dst.shape, src.stride(), dst.stride())
    if not dims:
        return dst.copy_(src)
    n_in, s_in, d_in = dims[-1]
    outer = dims[:-1]
    if (s_in != 1 or d_in != 1 or (n_in * es) % 16 or len(outer) > 4 or src.data_ptr() % 16 or dst.data_ptr() % 16
            or dst.numel() * es >= 2 ** 35
            or any((a * es) % 16 or (b * es) % 16 for _, a, b in outer)):
        return dst.copy_(src)
    outer = [(1, 0, 0)] * (4 - len(outer)) + outer
    arr = ctypes.c_longlong * 4
    sizes = arr(*[n for n, _, _ in outer])
    sstr = arr(*[a * es for _, a, _ in outer])
    dstr = arr(*[b * es for _, _, b in outer])
    _check(lib().cm_strided_copy(src.data_ptr(), dst.data_ptr(), sizes, sstr, dstr, n_in * es, stream_ptr()), "cm_strided_copy")
    F_.count_launch("strided_copy")
    return dst


def fast_contiguous(x: torch.Tensor) -> torch.Tensor:
    if x.is_contiguous() or not x.is_cuda:
        return x.contiguous()
    return fast_copy_(torch.empty(x.shape, dtype=x.dtype, device=x.device), x)


def wgrad_into_main_grad(w: torch.Tensor, run):
    """Weight gradient either as a fresh tensor or, when the optimizer asked for it (``w.fuse_wgrad_accumulation``),
    accumulated by the GEMM epilogue straight into the parameter's slice of the flat gradient buffer.  In the fused
    case autograd still gets a tensor of the right shape (uninitialised, never read): the optimizer's hook sees
    ``grad_added_to_main_grad`` and drops it.  ``run(out, accumulate)`` launches the GEMM."""
    mg = getattr(w, "main_grad", None)
    if (mg is not None and getattr(w, "fuse_wgrad_accumulation", False) and mg.dtype in (torch.bfloat16, torch.float32)
            and mg.is_contiguous() and mg.shape == w.shape):
        run(mg, True)
        w.grad_added_to_main_grad = True
        return torch.empty(w.shape, dtype=w.dtype, device=w.device)
    return run(None, False)


def linear(x: torch.Tensor, w: torch.Tensor):
    if not _gemm_ok(x, w):
        return None
    return LinearFn.apply(x, w)


class LinearFp32OutFn(torch.autograd.Function):
    """``y = x W^T`` with bf16 operands on the tensor cores and an fp32 result, for fp32 parameters whose
    consumers want fp32 (router logits).  ``w`` is the fp32 parameter; it is rounded to bf16 for the products and
    receives an fp32 gradient."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        wb = w.to(torch.bfloat16)
        ctx.save_for_backward(x2, wb)
        ctx.xshape = x.shape
        y = gemm(x2, wb, out_dtype=torch.float32)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wb = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, wb, b_mn=True).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)
        return dx, dw


def linear_fp32out(x: torch.Tensor, w: torch.Tensor):
    if (x.dtype != torch.bfloat16 or w.dtype != torch.float32 or w.dim() != 2 or x.shape[-1] % 8 or w.shape[0] % 8
            or x.numel() == 0):
        return None
    return LinearFp32OutFn.apply(x, w)


# ---------------------------------------------------------------------------
# RMSNorm / SwiGLU
# ---------------------------------------------------------------------------

class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        H = x.shape[-1]
        x2 = fast_contiguous(x).view(-1, H)
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        _check(lib().cm_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), x2.shape[0], H,
                                    float(eps), stream_ptr()), "cm_rmsnorm_fwd")
        F_.count_launch("rmsnorm")
        ctx.save_for_backward(x2, w, rstd)
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        H = x2.shape[-1]
        dy2 = fast_contiguous(dy).view(-1, H)
        dx = torch.empty_like(x2)
        dw = torch.zeros(H, dtype=torch.float32, device=x2.device)
        _check(lib().cm_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                    dw.data_ptr(), x2.shape[0], H, stream_ptr()), "cm_rmsnorm_bwd")
        F_.count_launch("rmsnorm_bwd")
        return dx.view(ctx.xshape), dw.to(w.dtype), None


def rmsnorm(x, w, eps):
    H = x.shape[-1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or H % 8 or H > 16384 or x.numel() == 0:
        from .. import reference as ref
        F_._miss("rmsnorm(shape/dtype)", x)
        return ref.rmsnorm(x, w, eps)
    return RMSNormFn.apply(x, w, eps)


class SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        out = torch.empty(g2.shape[0], F2 // 2, dtype=gu.dtype, device=gu.device)
        _check(lib().cm_swiglu_fwd(g2.data_ptr(), out.data_ptr(), g2.shape[0], F2 // 2, stream_ptr()), "cm_swiglu_fwd")
        F_.count_launch("swiglu")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        F = g2.shape[-1] // 2
        d2 = dout.reshape(-1, F)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        din = torch.empty_like(g2)
        _check(lib().cm_swiglu_bwd(g2.data_ptr(), d2.data_ptr(), din.data_ptr(), g2.shape[0], F, stream_ptr()),
               "cm_swiglu_bwd")
        F_.count_launch("swiglu_bwd")
        return din.view(ctx.shape)


def swiglu_rows(h: torch.Tensor, rows_limit: torch.Tensor) -> torch.Tensor:
    """``silu(h[:, :F]) * h[:, F:]`` on the first ``rows_limit[0]`` rows of a 2-D bf16 tensor (a device int32: the rows in use
    of a worst-case-sized buffer); the rows after them are left unwritten.  No autograd."""
    out = torch.empty(h.shape[0], h.shape[1] // 2, dtype=h.dtype, device=h.device)
    _check(lib().cm_swiglu_fwd_rows(h.data_ptr(), out.data_ptr(), h.shape[0], h.shape[1] // 2, rows_limit.data_ptr(), stream_ptr()),
           "cm_swiglu_fwd_rows")
    F_.count_launch("swiglu")
    return out


def swiglu_bwd_rows(h: torch.Tensor, da: torch.Tensor, rows_limit: torch.Tensor) -> torch.Tensor:
    """Gradient of :func:`swiglu_rows` with respect to ``h`` (same row limit)."""
    dh = torch.empty_like(h)
    _check(lib().cm_swiglu_bwd_rows(h.data_ptr(), da.data_ptr(), dh.data_ptr(), h.shape[0], h.shape[1] // 2, rows_limit.data_ptr(),
                                    stream_ptr()), "cm_swiglu_bwd_rows")
    F_.count_launch("swiglu_bwd")
    return dh


def swiglu(gu):
    if gu.dtype != torch.bfloat16 or (gu.shape[-1] // 2) % 8 or gu.numel() == 0:
        from .. import reference as ref
        F_._miss("swiglu(shape/dtype)", gu)
        return ref.swiglu(gu)
    return SwiGLUFn.apply(gu)


# ---------------------------------------------------------------------------
# optimizer
# ---------------------------------------------------------------------------

def adamw_shard(master, m, v, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2, gate=None):
    """``gate``: optional device int32 word; the update is skipped on the device when it is non-zero."""
    gk = {torch.float32: 0, torch.bfloat16: 1}.get(g.dtype)
    ok = {torch.float32: 0, torch.bfloat16: 1}.get(out.dtype)
    if gk is None or ok is None:
        from ...optim.adamw import adamw_reference
        return adamw_reference(master, m, v, g, out, wd_mask, clip, lr, b1, b2, eps, wd, bc1, bc2)
    clip_t = clip if torch.is_tensor(clip) else torch.tensor(float(clip), device=master.device)
    clip_t = clip_t.reshape(1).float()
    _check(lib().cm_adamw_gated(master.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), out.data_ptr(),
                                wd_mask.data_ptr(), clip_t.data_ptr(), master.numel(), float(lr), float(b1), float(b2),
                                float(eps), float(wd), float(bc1), float(bc2), gk, ok,
                                None if gate is None else gate.data_ptr(), stream_ptr()), "cm_adamw")
    F_.count_launch("adamw")


def sumsq(g: torch.Tensor, out: torch.Tensor) -> None:
    kind = {torch.float32: 0, torch.bfloat16: 1}[g.dtype]
    _check(lib().cm_sumsq(g.data_ptr(), g.numel(), out.data_ptr(), kind, stream_ptr()), "cm_sumsq")
    F_.count_launch("sumsq")


def _register() -> None:
    F_.register_cuda("linear", linear)
    F_.register_cuda("linear_fp32out", linear_fp32out)
    F_.register_cuda("rmsnorm", rmsnorm)
    F_.register_cuda("swiglu", swiglu)
    F_.register_cuda("adamw_shard", adamw_shard)
    from . import attention, extra, kernels4
    extra.register()
    kernels4.register()
    attention.register()


if torch.cuda.is_available():
    lib()            # raises if the library was not built: no silent fallback on a GPU box
    _register()
