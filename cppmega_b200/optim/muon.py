"""Muon for matrix parameters, with optional int8 (q8) momentum.

Per matrix ``W [rows, cols]`` with gradient ``G``:

    m   <- beta * m + (1 - beta) * G                    (fp32, or q8: int8 payload + fp32 absmax per 256 values)
    U   <- NewtonSchulz5(m / ||m||_F)                   (bf16 GEMMs; per normalisation group for fused projections)
    W   <- W * (1 - lr * wd) - lr * scale * U,          scale = 0.2 * sqrt(max(rows, cols))

Scalars, embeddings and the output layer stay on AdamW (``muon_scalar_optimizer``).  Stacked expert weights
``[E, rows, cols]`` are E separate matrices.  Under ZeRO-1 a matrix whose elements all lie in one rank's shard is
updated there; for a matrix cut by a shard boundary every owner updates its piece of the momentum, the bucket's
momentum is all-gathered, and each owner applies its rows of the orthogonalised full matrix
(:func:`muon_update_cut_matrices`), so the update is the same for every data-parallel size and bucket size.

The q8 state and its kernels follow the reference's contract (cppmega/megatron/quantized_muon_momentum.py:29-46 state,
:97-185 norm plan for fused-QKV segments, :287-676 update entry points; kernel arithmetic at
cppmega/megatron/cuda_ext/quantized_muon_momentum.cu:283-340); the Newton-Schulz driver replaces the one the reference
takes from Megatron's emerging-optimizers fork (cppmega/recipes/run_profiles.py:167-195).
"""
from __future__ import annotations

import atexit
import collections
import ctypes
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import reference as ref

QBLOCK = 256


# ---------------------------------------------------------------------------
# q8 momentum state
# ---------------------------------------------------------------------------

@dataclass
class QuantizedMomentum:
    """int8 payload + one fp32 absmax per 256 values (flat, padded to a whole block)."""

    data: torch.Tensor            # int8 [n]
    absmax: torch.Tensor          # fp32 [ceil(n / 256)]
    shape: Tuple[int, ...]

    @classmethod
    def zeros(cls, shape: Sequence[int], device) -> "QuantizedMomentum":
        n = int(math.prod(shape))
        return cls(torch.zeros(n, dtype=torch.int8, device=device),
                   torch.zeros((n + QBLOCK - 1) // QBLOCK, dtype=torch.float32, device=device), tuple(shape))

    def dequantize(self) -> torch.Tensor:
        n = self.data.numel()
        sc = (self.absmax / 127.0).repeat_interleave(QBLOCK)[:n]
        return (self.data.float() * sc).view(self.shape)

    def nbytes(self) -> int:
        return self.data.numel() + 4 * self.absmax.numel()


@dataclass
class NormPlan:
    """Which 256-blocks of a flat matrix normalise together.  A fused projection (e.g. QKV stacked along rows) is cut
    into row segments that each get their own Frobenius norm; segments must start on a block boundary."""

    block_group: torch.Tensor     # int32 [nblocks]
    num_groups: int
    row_splits: Tuple[int, ...] = field(default_factory=tuple)


def build_norm_plan(shape: Sequence[int], row_splits: Optional[Sequence[int]] = None, device="cpu") -> NormPlan:
    rows, cols = int(shape[0]), int(shape[1])
    n = rows * cols
    nblocks = (n + QBLOCK - 1) // QBLOCK
    if not row_splits:
        return NormPlan(torch.zeros(nblocks, dtype=torch.int32, device=device), 1, (rows,))
    if sum(row_splits) != rows:
        raise ValueError(f"row_splits {tuple(row_splits)} do not add up to {rows} rows")
    bg = torch.empty(nblocks, dtype=torch.int32)
    start = 0
    for gi, r in enumerate(row_splits):
        s, e = start * cols, (start + r) * cols
        if s % QBLOCK:
            raise ValueError(f"segment {gi} starts at element {s}, not on a {QBLOCK}-value block boundary")
        bg[s // QBLOCK:(e + QBLOCK - 1) // QBLOCK] = gi
        start += r
    return NormPlan(bg.to(device), len(row_splits), tuple(int(r) for r in row_splits))


_AUDIT: "collections.Counter[str]" = collections.Counter()
_audit_on = False


def enable_dtype_audit(print_at_exit: bool = True) -> None:
    """Count elements per dtype that pass through the momentum update and Newton-Schulz
    (cppmega/megatron/muon_dtype_audit.py:61-116)."""
    global _audit_on
    if not _audit_on and print_at_exit:
        atexit.register(lambda: print("[muon dtype audit] " + ", ".join(f"{k}={v}" for k, v in sorted(_AUDIT.items()))))
    _audit_on = True


def dtype_audit() -> Dict[str, int]:
    return dict(_AUDIT)


def _note(tag: str, t: torch.Tensor) -> None:
    if _audit_on:
        _AUDIT[f"{tag}:{str(t.dtype).replace('torch.', '')}"] += t.numel()


def _cuda_lib():
    from ..ops import cuda as cu
    L = cu.lib()
    if not getattr(L, "_qmuon_declared", False):
        vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        L.cm_qmuon_update.argtypes = [vp, vp, vp, vp, vp, vp, i64, f32, i32, vp]
        L.cm_qmuon_scale.argtypes = [vp, vp, vp, i64, f32, i32, vp]
        L.cm_qmuon_emit_mxfp8.argtypes = [vp, vp, vp, vp, vp, i64, vp]
        for n in ("cm_qmuon_update", "cm_qmuon_scale", "cm_qmuon_emit_mxfp8"):
            getattr(L, n).restype = i32
        L._qmuon_declared = True
    return L


def qmuon_update_(state: QuantizedMomentum, grad: torch.Tensor, beta: float, plan: Optional[NormPlan] = None,
                  eps: float = 1e-7, tp_group=None) -> torch.Tensor:
    """In place: momentum update + requantisation; ``grad`` is overwritten with the new momentum divided by the
    Frobenius norm of its normalisation group (the Newton-Schulz input).  Returns the per-group sums of squares."""
    n = grad.numel()
    plan = plan or build_norm_plan((1, n), device=grad.device)
    _note("momentum", state.data)
    _note("grad", grad)
    gflat = grad.view(-1)
    group_ss = torch.zeros(plan.num_groups, dtype=torch.float32, device=grad.device)
    use_cuda = grad.is_cuda and grad.dtype in (torch.float32, torch.bfloat16) and grad.is_contiguous()
    if use_cuda:
        from ..ops import cuda as cu
        from ..ops import functional as F_
        L = _cuda_lib()
        kind = 0 if grad.dtype == torch.float32 else 1
        rc = L.cm_qmuon_update(state.data.data_ptr(), state.absmax.data_ptr(), gflat.data_ptr(), None, group_ss.data_ptr(),
                               plan.block_group.data_ptr(), n, float(beta), kind, cu.stream_ptr())
        if rc:
            raise RuntimeError(f"cm_qmuon_update failed ({rc})")
        F_.count_launch("qmuon_update")
    else:
        qn, am, m, ss = ref.qmuon_update(state.data, state.absmax, gflat, beta)
        state.data.copy_(qn)
        state.absmax.copy_(am)
        gflat.copy_(m.to(grad.dtype))
        group_ss.index_add_(0, plan.block_group.long(), ss)
    if tp_group is not None and torch.distributed.is_initialized():
        torch.distributed.all_reduce(group_ss, group=tp_group)
    if use_cuda:
        rc = L.cm_qmuon_scale(gflat.data_ptr(), group_ss.data_ptr(), plan.block_group.data_ptr(), n, float(eps), kind,
                              cu.stream_ptr())
        if rc:
            raise RuntimeError(f"cm_qmuon_scale failed ({rc})")
        F_.count_launch("qmuon_scale")
    else:
        inv = torch.rsqrt(torch.clamp(group_ss, min=eps * eps))
        per_elem = inv[plan.block_group.long()].repeat_interleave(QBLOCK)[:n]
        gflat.mul_(per_elem.to(grad.dtype))
    return group_ss


def emit_mxfp8_carrier(state: QuantizedMomentum, inv_norm: Optional[torch.Tensor] = None):
    """q8 momentum -> (E4M3 payload uint8 [n], E8M0 scales uint8 [n/32]) for a block-scaled Newton-Schulz GEMM."""
    n = state.data.numel()
    if n % 32:
        raise ValueError("carrier emission needs a multiple of 32 values")
    if state.data.is_cuda:
        from ..ops import cuda as cu
        L = _cuda_lib()
        payload = torch.empty(n, dtype=torch.uint8, device=state.data.device)
        scales = torch.empty(n // 32, dtype=torch.uint8, device=state.data.device)
        rc = L.cm_qmuon_emit_mxfp8(state.data.data_ptr(), state.absmax.data_ptr(),
                                   None if inv_norm is None else inv_norm.data_ptr(), payload.data_ptr(),
                                   scales.data_ptr(), n, cu.stream_ptr())
        if rc:
            raise RuntimeError(f"cm_qmuon_emit_mxfp8 failed ({rc})")
        return payload, scales
    v = state.dequantize().reshape(-1) * (1.0 if inv_norm is None else float(inv_norm))
    q, s = ref.mxfp8_quantize(v.view(1, -1))
    return q.view(torch.uint8).view(-1), s.view(-1)


# ---------------------------------------------------------------------------
# Newton-Schulz and the per-matrix update
# ---------------------------------------------------------------------------

def newton_schulz(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    _note("newton_schulz", G)
    return ref.newton_schulz(G, steps)


def muon_scale(shape: Sequence[int]) -> float:
    return 0.2 * math.sqrt(max(int(shape[0]), int(shape[1])))


def muon_update_segments(st: dict, g: torch.Tensor, clip: torch.Tensor, lr: float, cfg) -> None:
    """Muon step for every whole matrix inside one optimizer shard (``st`` is a state entry of the distributed
    optimizer: ``master``, ``m`` fp32 flat shards and ``muon`` = [(start, end, shape)]).  The low-precision copy of the
    parameter is written by the caller's AdamW pass, which skips these ranges and then casts."""
    buf = st["buf"]
    out = buf.param_buffer[st["lo"]:st["hi"]]
    qstates: Dict[int, QuantizedMomentum] = st.setdefault("muon_q", {})
    for (s, e, shape) in st["muon"]:
        grad = (g[s:e].float() * clip).view(shape)
        if cfg.muon_quantized_momentum:
            q = qstates.get(s)
            if q is None:
                q = qstates[s] = QuantizedMomentum.zeros(shape, grad.device)
            work = grad.contiguous()
            qmuon_update_(q, work, cfg.muon_momentum)
            upd_in = work                                    # already divided by its Frobenius norm
        else:
            m = st["m"][s:e].view(shape)
            m.mul_(cfg.muon_momentum).add_(grad, alpha=1.0 - cfg.muon_momentum)
            upd_in = m
        U = newton_schulz(upd_in, cfg.muon_ns_steps).float()
        w = st["master"][s:e].view(shape)
        if cfg.weight_decay > 0:
            w.mul_(1.0 - lr * cfg.weight_decay)
        w.add_(U, alpha=-lr * muon_scale(shape))
        out[s:e].copy_(w.reshape(-1).to(out.dtype))


def _all_gather_flat(x: torch.Tensor, group, n: int) -> torch.Tensor:
    import torch.distributed as dist
    if x.device.type == "cpu":
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts)
    out = torch.empty(n * x.numel(), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def muon_update_cut_matrices(st: dict, g: torch.Tensor, clip: torch.Tensor, lr: float, cfg) -> None:
    """Muon for the matrices of one bucket that a shard boundary cuts.  The momentum update is elementwise, so every
    rank updates the piece it owns; Newton-Schulz needs the whole matrix, so the bucket's momentum shards are
    all-gathered (one collective per such bucket, issued by every rank of the group whether or not it owns a piece),
    each owner orthogonalises the full matrix and applies its own rows.  The result does not depend on where the
    shard boundaries fall.  Momentum of these matrices stays fp32 (the q8 blocks do not line up with the cuts)."""
    buf = st["buf"]
    out = buf.param_buffer[st["lo"]:st["hi"]]
    for c in st["muon_cross"]:
        s, e = c["local"]
        grad = g[s:e].float() * clip
        st["m"][s:e].mul_(cfg.muon_momentum).add_(grad, alpha=1.0 - cfg.muon_momentum)
    full = _all_gather_flat(st["m"], buf.group, buf.n)          # [bucket numel], rank-major = bucket order
    for c in st["muon_cross"]:
        s, e = c["local"]
        a, b_ = c["bucket"]
        i0, i1 = c["inner"]
        shape = c["shape"]
        U = newton_schulz(full[a:b_].view(shape), cfg.muon_ns_steps).float().reshape(-1)[i0:i1]
        w = st["master"][s:e]
        if cfg.weight_decay > 0:
            w.mul_(1.0 - lr * cfg.weight_decay)
        w.add_(U, alpha=-lr * muon_scale(shape))
        out[s:e].copy_(w.to(out.dtype))


def momentum_bytes(shapes: Sequence[Sequence[int]], quantized: bool) -> int:
    """Optimizer-state estimate used by the memory report."""
    tot = 0
    for sh in shapes:
        n = int(math.prod(sh))
        tot += (n + 4 * ((n + QBLOCK - 1) // QBLOCK)) if quantized else 4 * n
    return tot


_ = List
