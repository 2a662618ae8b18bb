"""Python side of the fused Mamba3 MIMO scan backward: launches the kernels and finishes the small
reductions (heads -> groups, per-head biases, trapezoid coefficients -> DT / Trap)."""
from __future__ import annotations

import torch

from .. import functional as F_
from .kernels3 import LT, _as_bsgrn, token_strided


def mimo_bwd(saved, dy, states, tot):
    from . import lib, err_word, stream_ptr, _check
    Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, D, Z = saved
    B, S, R, G, N = Q.shape
    H, P = V.shape[2], V.shape[3]
    C = S // LT
    dev = V.device
    hpg = H // G
    Qn, Kn = _as_bsgrn(Q), _as_bsgrn(K)
    f32 = lambda t: t.float().contiguous()
    ADTf, DTf, Trapf = f32(ADT), f32(DT), f32(Trap)
    dyc = dy.to(torch.bfloat16).contiguous()
    gbuf = torch.empty(B, H, C, N, P, dtype=torch.float32, device=dev)
    dend = torch.empty(B, H, C, N, P, dtype=torch.bfloat16, device=dev)
    dQh = torch.empty(B, S, H, R, N, dtype=torch.bfloat16, device=dev)
    dKh = torch.empty(B, S, H, R, N, dtype=torch.bfloat16, device=dev)
    dV = torch.empty(B, S, H, P, dtype=torch.bfloat16, device=dev)
    dZ = torch.empty(B, S, H, P, dtype=torch.bfloat16, device=dev)
    dAng = torch.empty(B, S, H, N // 4, dtype=torch.float32, device=dev)
    dADT = torch.empty(B, H, S, dtype=torch.float32, device=dev)
    dTs = torch.empty(B, H, S, dtype=torch.float32, device=dev)
    dGam = torch.empty(B, H, S, dtype=torch.float32, device=dev)
    dPsi = torch.zeros(H, R, P, dtype=torch.float32, device=dev)
    dZeta = torch.zeros(H, R, P, dtype=torch.float32, device=dev)
    dPhi = torch.zeros(H, R, P, dtype=torch.float32, device=dev)
    dD = torch.zeros(H, dtype=torch.float32, device=dev)
    Vs, ldV = token_strided(V)
    Zs, ldZ = token_strided(Z)
    ins = [Qn, Kn, Vs, Zs, dyc, ADTf, DTf, Trapf, f32(Qb), f32(Kb), f32(Psi), f32(Zeta), f32(Phi),
           f32(angles), f32(D), states, tot]
    outs = [gbuf, dend, dQh, dKh, dV, dZ, dAng, dADT, dTs, dGam, dPsi, dZeta, dPhi, dD]
    _check(lib().cm_mimo_scan_bwd(*[t.data_ptr() for t in ins], *[t.data_ptr() for t in outs], B, S, H, G, N, ldV, ldZ,
                                  err_word(dev).data_ptr(), stream_ptr()), "cm_mimo_scan_bwd")
    F_.count_launch("mimo_scan_bwd", 3)
    del gbuf, dend
    # heads -> groups (Q/K are shared by the heads of a group) and per-head biases, one pass per tensor
    from .kernels4 import head_reduce
    if hpg in (1, 2, 4, 8, 16):
        dQg, dQb = head_reduce(dQh, G)
        dKg, dKb = head_reduce(dKh, G)
        dQ, dK = dQg.permute(0, 1, 3, 2, 4), dKg.permute(0, 1, 3, 2, 4)
    else:
        dQ = dQh.view(B, S, G, hpg, R, N).sum(3, dtype=torch.float32).permute(0, 1, 3, 2, 4)
        dK = dKh.view(B, S, G, hpg, R, N).sum(3, dtype=torch.float32).permute(0, 1, 3, 2, 4)
        dQb = dQh.sum((0, 1), dtype=torch.float32)
        dKb = dKh.sum((0, 1), dtype=torch.float32)
    del dQh, dKh
    # trapezoid coefficients: gamma_t = DT_t sig(Trap_t), ts_t = gamma_t + DT_{t+1} sig(-Trap_{t+1})
    sg = torch.sigmoid(Trapf)
    dgt = dGam + dTs
    prev = torch.zeros_like(dTs)
    prev[..., 1:] = dTs[..., :-1]
    dDT = dgt * sg + prev * (1.0 - sg)
    dTrap = (dgt - prev) * DTf * sg * (1.0 - sg)
    return (dQ.to(Q.dtype), dK.to(K.dtype), dV.to(V.dtype), dADT.to(ADT.dtype), dDT.to(DT.dtype), dTrap.to(Trap.dtype),
            dQb.to(Qb.dtype), dKb.to(Kb.dtype), dPsi.to(Psi.dtype), dZeta.to(Zeta.dtype), dPhi.to(Phi.dtype),
            dAng.to(angles.dtype), dD.to(D.dtype), dZ.to(Z.dtype))
