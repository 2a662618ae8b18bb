"""Wrappers for the Mamba3 MIMO scan kernels."""
from __future__ import annotations

import ctypes

import torch

from .. import functional as F_

LT = 32


def declare(L: ctypes.CDLL) -> None:
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    fn = getattr(L, "cm_mimo_scan_fwd", None)
    if fn is not None:
        fn.argtypes = [vp] * 19 + [i32] * 5 + [i64, i64] + [vp, vp]
        fn.restype = i32
    fn = getattr(L, "cm_mimo_scan_bwd", None)
    if fn is not None:
        fn.argtypes = [vp] * 31 + [i32] * 5 + [i64, i64] + [vp, vp]
        fn.restype = i32


def supported(Q, K, V, Zeta, Phi, D, Z, div) -> bool:
    B, S, R, G, N = Q.shape
    H, P = V.shape[2], V.shape[3]
    return (V.is_cuda and V.dtype == torch.bfloat16 and Q.dtype == torch.bfloat16 and K.dtype == torch.bfloat16
            and R == 4 and N == 128 and P == 64 and div == 4 and S % LT == 0 and H % G == 0
            and None not in (Zeta, Phi, D, Z) and Z.dtype == torch.bfloat16)


class _ShapeOnly:
    """Stand-in that answers ``shape`` / ``dtype`` like tensor ``x`` would after padding its last dimension to ``n``."""

    def __init__(self, x: torch.Tensor, n: int):
        self.shape, self.dtype = (*x.shape[:-1], n), x.dtype


def _as_bsgrn(x: torch.Tensor) -> torch.Tensor:
    """[B,S,R,G,N] (possibly a permuted view) -> contiguous [B,S,G,R,N]."""
    y = x.permute(0, 1, 3, 2, 4)
    return y if y.is_contiguous() else y.contiguous()


def token_strided(x: torch.Tensor):
    """(tensor, token stride) for a [B,S,H,P] bf16 operand that the kernels can read in place: the last two dims packed,
    batch stride = S * token stride, 16-byte aligned rows.  Anything else is copied to a packed tensor."""
    B, S, H, P = x.shape
    sb, ss, sh, sp = x.stride()
    if sp == 1 and sh == P and sb == S * ss and ss >= H * P and ss % 8 == 0 and x.data_ptr() % 16 == 0:
        return x, ss
    x = x.contiguous()
    return x, H * P


def mimo_fwd_raw(Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, want_state: bool = False):
    """Qn/Kn are [B,S,G,R,N] contiguous bf16.  Returns (y, states, tot[, final_state])."""
    from . import lib, err_word, stream_ptr, _check
    B, S, G, R, N = Qn.shape
    H, P = V.shape[2], V.shape[3]
    C = S // LT
    dev = V.device
    local = torch.empty(B, H, C, N, P, dtype=torch.float32, device=dev)
    tot = torch.empty(B, H, C, dtype=torch.float32, device=dev)
    states = torch.empty(B, H, C, N, P, dtype=torch.bfloat16, device=dev)
    final = torch.empty(B, H, N, P, dtype=torch.float32, device=dev) if want_state else None
    y = torch.empty(B, S, H, P, dtype=torch.bfloat16, device=dev)
    f32 = lambda t: t.float().contiguous()
    Vs, ldV = token_strided(V)
    Zs, ldZ = token_strided(Z)
    args = [Qn, Kn, Vs, Zs, f32(ADT), f32(DT), f32(Trap), f32(Qb), f32(Kb), f32(Psi), f32(Zeta),
            f32(Phi), f32(angles), f32(D)]
    _check(lib().cm_mimo_scan_fwd(*[t.data_ptr() for t in args], local.data_ptr(), tot.data_ptr(), states.data_ptr(),
                                  final.data_ptr() if want_state else None, y.data_ptr(), B, S, H, G, N, ldV, ldZ,
                                  err_word(dev).data_ptr(), stream_ptr()), "cm_mimo_scan_fwd")
    F_.count_launch("mimo_scan_fwd", 3)
    return (y, states, tot, final) if want_state else (y, states, tot)


class MimoScanFn(torch.autograd.Function):
    """Fused forward; the backward uses the fused backward kernels when the library has them and
    otherwise recomputes group by group in PyTorch."""

    @staticmethod
    def forward(ctx, Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div, chunk, precomputed=None):
        if precomputed is None:
            precomputed = mimo_fwd_raw(_as_bsgrn(Q), _as_bsgrn(K), V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D)
        y, states, tot = precomputed
        ctx.save_for_backward(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, states, tot)
        ctx.div, ctx.chunk = div, 64          # chunk length of the PyTorch recomputation, not of the kernel
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import lib
        *saved, states, tot = ctx.saved_tensors
        if getattr(lib(), "cm_mimo_scan_bwd", None) is not None and "mimo_scan_bwd" not in F_._DISABLED:
            from .mimo_bwd import mimo_bwd
            return (*mimo_bwd(saved, dy, states, tot), None, None, None)
        from ..mimo_scan_lean import lean_backward
        F_._FALLBACKS["mimo_scan_bwd"] += 1
        return (*lean_backward(saved, dy, ctx.div, ctx.chunk), None)


def _pad_state_dim(x: torch.Tensor, n: int, to: int = 128) -> torch.Tensor:
    """[..., n] -> [..., to]: each half of the state dimension keeps its place at the start of the wider half
    (``[first half | 0 | second half | 0]``), so the rotary pairs ``(i, n/2 + i)`` become ``(i, to/2 + i)``."""
    h, z = n // 2, x.new_zeros(*x.shape[:-1], to // 2 - n // 2)
    return torch.cat([x[..., :h], z, x[..., h:], z], dim=-1)


def _pad_launch(ins, outs, specs, inverse: bool) -> None:
    """One launch of ``cm_pad_state_dims`` over several tensors; ``specs``: (n, w, split) per tensor."""
    from . import lib, stream_ptr, _check
    L = lib()
    k = len(ins)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    if not getattr(L, "_pad_declared", False):
        L.cm_pad_state_dims.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, vp]
        L.cm_pad_state_dims.restype = i32
        L._pad_declared = True
    narrow = outs if inverse else ins
    rows = (i64 * k)(*[t.numel() // spec[0] for t, spec in zip(narrow, specs)])
    _check(L.cm_pad_state_dims((vp * k)(*[t.data_ptr() for t in ins]), (vp * k)(*[t.data_ptr() for t in outs]), rows,
                               (i32 * k)(*[sp[0] for sp in specs]), (i32 * k)(*[sp[1] for sp in specs]),
                               (i32 * k)(*[t.element_size() for t in ins]), (i32 * k)(*[int(sp[2]) for sp in specs]),
                               k, int(inverse), stream_ptr()), "cm_pad_state_dims")
    F_.count_launch("pad_state_dims")


class PadStateFn(torch.autograd.Function):
    """(Q, K, Qb, Kb, angles) with state dimension n -> the same tensors widened to 128 (angles to 32) by one kernel; the
    backward is one launch of its adjoint."""

    @staticmethod
    def forward(ctx, Q, K, Qb, Kb, angles):
        n, a = Q.shape[-1], angles.shape[-1]
        ins = [t.contiguous() for t in (Q, K, Qb, Kb, angles)]
        specs = [(n, 128, True)] * 4 + [(a, 32, False)]
        outs = [torch.empty(*t.shape[:-1], sp[1], dtype=t.dtype, device=t.device) for t, sp in zip(ins, specs)]
        _pad_launch(ins, outs, specs, False)
        ctx.specs, ctx.shapes = specs, [t.shape for t in ins]
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        specs, shapes = [], []
        ins, slots = [], []
        for i, (g, sp, shp) in enumerate(zip(grads, ctx.specs, ctx.shapes)):
            if g is not None and ctx.needs_input_grad[i]:
                ins.append(g.contiguous())
                specs.append(sp)
                shapes.append(shp)
                slots.append(i)
        outs = [torch.empty(shp, dtype=g.dtype, device=g.device) for g, shp in zip(ins, shapes)]
        if ins:
            _pad_launch(ins, outs, specs, True)
        res = [None] * 5
        for i, o in zip(slots, outs):
            res[i] = o
        return tuple(res)


def _padded_to_128(Q, K, Qb, Kb, angles):
    """A scan with state dimension 32 or 64 is the scan with state dimension 128 on zero-padded Q / K / biases: the
    padded state rows stay zero, the padded rotary pairs get angle 0.  The kernels are instantiated for 128."""
    N = Q.shape[-1]
    if (Q.is_cuda and Q.dtype == K.dtype and Q.element_size() in (2, 4) and Qb.dtype == Kb.dtype == torch.float32
            and angles.dtype == torch.float32 and N % 2 == 0):
        return PadStateFn.apply(Q, K, Qb, Kb, angles)
    ang = torch.cat([angles, angles.new_zeros(*angles.shape[:-1], 32 - angles.shape[-1])], dim=-1)
    return _pad_state_dim(Q, N), _pad_state_dim(K, N), _pad_state_dim(Qb, N), _pad_state_dim(Kb, N), ang


def mimo_scan(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div, chunk):
    N = Q.shape[-1]
    if (N in (32, 64) and div == 4 and angles.shape[-1] == N // 4 and V.is_cuda
            and supported(_ShapeOnly(Q, 128), K, V, Zeta, Phi, D, Z, div)):
        Qp, Kp, Qbp, Kbp, angp = _padded_to_128(Q, K, Qb, Kb, angles)
        return mimo_scan(Qp, Kp, V, ADT, DT, Trap, Qbp, Kbp, Psi, Zeta, Phi, angp, D, Z, div, chunk)
    if not supported(Q, K, V, Zeta, Phi, D, Z, div):
        from ..mimo_scan_lean import mimo_scan_lean
        F_._FALLBACKS["mimo_scan"] += 1
        if None in (Zeta, Phi, D, Z):
            from .. import mimo_scan_ref as R
            return R.mimo_scan_chunked(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div, chunk)
        return mimo_scan_lean(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div, 64)
    from ...utils.recompute import stashed_call
    # inside a recomputed layer the three forward kernels run once: the replay picks up (y, chunk states, totals)
    return stashed_call(
        "mimo_scan",
        lambda: mimo_fwd_raw(_as_bsgrn(Q), _as_bsgrn(K), V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D),
        lambda res: MimoScanFn.apply(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z, div, chunk, res))


def register() -> None:
    F_.register_cuda("mimo_scan", mimo_scan)
