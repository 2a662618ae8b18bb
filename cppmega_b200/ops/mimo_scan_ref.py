"""Mamba3 MIMO scan: plain-PyTorch definitions.

Two functions compute the same operator:

* :func:`mimo_scan_sequential` walks the sequence one token at a time.  It is
  the ground truth that every other implementation (the chunked PyTorch form
  below and the sm_100a kernels) is tested against.
* :func:`mimo_scan_chunked` is the block-parallel form (intra-chunk masked
  products + chunk states + a short recurrence over chunks).  It is
  differentiable by autograd and is the CPU / fallback path.

Operator (per batch ``b`` and head ``h``; ``g = h // (H/G)``; ``r`` indexes the MIMO
rank; state ``S`` is ``[N, P]`` in fp32):

    q[t,r] = rot(Q[t,r,g] + Qb[h,r]),  k[t,r] = rot(K[t,r,g] + Kb[h,r])
    PsiV[t,r] = V[t] * Psi[h,r]
    gamma_t = DT_t * sigmoid(Trap_t)
    ts_t    = gamma_t + DT_{t+1} * sigmoid(-Trap_{t+1})          (second term 0 at t = S-1)
    Sdec    = exp(ADT_t) * S_{t-1}
    o[t,r]  = q[t,r] . Sdec + gamma_t * sum_r' (q[t,r].k[t,r']) PsiV[t,r'] + D_h PsiV[t,r]
    S_t     = Sdec + ts_t * sum_r k[t,r]^T PsiV[t,r]
    y[t]    = sum_r o[t,r] * Phi[h,r] * silu(Z[t] * Zeta[h,r])

``rot`` rotates the pairs ``(i, N/2 + i)`` for ``i < N / rotary_dim_divisor`` by the
per-(token, head) angle.  The definition is independent of any chunk size.  The
reference states the same computation chunk-wise
(cppmega/megatron/cute_dsl_mimo/cute_dsl_mimo_fwd.py:89-267); its backward
(cppmega/megatron/cute_dsl_mimo/full_bwd_bwd_epilogue.py:163-166) shows that the state
update consumes the trapezoid-scaled K, which is what makes the operator
chunk-size invariant and is what is implemented here.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _rot(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot: int) -> torch.Tensor:
    """Rotate pairs (i, N/2+i), i < n_rot.  x: [..., N]; cos/sin broadcastable [..., n_rot]."""
    n = x.shape[-1]
    half = n // 2
    a = x[..., :n_rot]
    b = x[..., half:half + n_rot]
    out_a = cos * a - sin * b
    out_b = sin * a + cos * b
    pieces = [out_a]
    if n_rot < half:
        pieces.append(x[..., n_rot:half])
    pieces.append(out_b)
    if half + n_rot < n:
        pieces.append(x[..., half + n_rot:])
    return torch.cat(pieces, dim=-1)


def trapezoid_coeffs(dt: torch.Tensor, trap: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Return ``(gamma, ts)`` with shapes of ``dt`` ([B,H,S])."""
    dt = dt.float()
    trap = trap.float()
    gamma = dt * torch.sigmoid(trap)
    nxt = dt * torch.sigmoid(-trap)
    shifted = torch.cat([nxt[..., 1:], torch.zeros_like(nxt[..., :1])], dim=-1)
    return gamma, gamma + shifted


def _prep(Q, K, V, Q_bias, K_bias, angles, rotary_dim_divisor):
    B, S, R, G, N = Q.shape
    H = V.shape[2]
    hpg = H // G
    # [B,S,R,G,N] -> [B,S,H,R,N] with head h reading group h // hpg
    qh = Q.float().permute(0, 1, 3, 2, 4).repeat_interleave(hpg, dim=2) + Q_bias.float()
    kh = K.float().permute(0, 1, 3, 2, 4).repeat_interleave(hpg, dim=2) + K_bias.float()
    n_rot = N // rotary_dim_divisor
    ang = angles.float()
    cos = torch.cos(ang).unsqueeze(3)   # [B,S,H,1,n_rot]
    sin = torch.sin(ang).unsqueeze(3)
    return _rot(qh, cos, sin, n_rot), _rot(kh, cos, sin, n_rot)


def _gate(o, Z, Zeta, Phi, out_dtype):
    """o: [B,S,H,R,P] fp32 -> y [B,S,H,P] (Phi given) or [B,S,R,H,P] (Phi None)."""
    if Z is not None:
        zz = Z.float().unsqueeze(3) * Zeta.float()       # [B,S,H,R,P]
        o = o * (zz * torch.sigmoid(zz))
    if Phi is not None:
        return (o * Phi.float()).sum(dim=3).to(out_dtype)
    return o.permute(0, 1, 3, 2, 4).to(out_dtype)


def mimo_scan_sequential(
    Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor,
    ADT: torch.Tensor, DT: torch.Tensor, Trap: torch.Tensor,
    Q_bias: torch.Tensor, K_bias: torch.Tensor,
    Psi: torch.Tensor, Zeta: Optional[torch.Tensor], Phi: Optional[torch.Tensor],
    angles: torch.Tensor, D: Optional[torch.Tensor], Z: Optional[torch.Tensor],
    rotary_dim_divisor: int = 4,
    initial_state: Optional[torch.Tensor] = None,
    return_state: bool = False,
):
    """Token-by-token ground truth.  Shapes: Q,K [B,S,R,G,N]; V,Z [B,S,H,P];
    ADT,DT,Trap [B,H,S]; biases [H,R,N]; Psi,Zeta,Phi [H,R,P]; angles [B,S,H,N/div]; D [H]."""
    B, S, R, G, N = Q.shape
    H, P = V.shape[2], V.shape[3]
    q, k = _prep(Q, K, V, Q_bias, K_bias, angles, rotary_dim_divisor)   # [B,S,H,R,N]
    gamma, ts = trapezoid_coeffs(DT, Trap)                               # [B,H,S]
    psiv = V.float().unsqueeze(3) * Psi.float()                          # [B,S,H,R,P]
    state = (initial_state.float().clone() if initial_state is not None
             else torch.zeros(B, H, N, P, dtype=torch.float32, device=Q.device))
    outs = []
    for t in range(S):
        dec = torch.exp(ADT[:, :, t].float())[..., None, None]
        sdec = state * dec
        o = torch.einsum("bhrn,bhnp->bhrp", q[:, t], sdec)
        qk = torch.einsum("bhrn,bhsn->bhrs", q[:, t], k[:, t])
        o = o + gamma[:, :, t, None, None] * torch.einsum("bhrs,bhsp->bhrp", qk, psiv[:, t])
        if D is not None:
            o = o + D.float()[None, :, None, None] * psiv[:, t]
        state = sdec + ts[:, :, t, None, None] * torch.einsum("bhrn,bhrp->bhnp", k[:, t], psiv[:, t])
        outs.append(o)
    o = torch.stack(outs, dim=1)                                         # [B,S,H,R,P]
    y = _gate(o, Z, Zeta, Phi, V.dtype)
    return (y, state) if return_state else y


def mimo_scan_chunked(
    Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Psi, Zeta, Phi, angles, D, Z,
    rotary_dim_divisor: int = 4, chunk_size: int = 16,
    initial_state: Optional[torch.Tensor] = None, return_state: bool = False,
    mm_dtype: Optional[torch.dtype] = None,
):
    """Block-parallel form of the same operator; differentiable.  ``mm_dtype`` (e.g. bf16)
    rounds the operands of the large contractions, as a tensor-core kernel would."""
    B, S, R, G, N = Q.shape
    H, P = V.shape[2], V.shape[3]
    L = min(chunk_size, S)
    pad = (-S) % L
    q, k = _prep(Q, K, V, Q_bias, K_bias, angles, rotary_dim_divisor)   # [B,S,H,R,N]
    gamma, ts = trapezoid_coeffs(DT, Trap)
    psiv = V.float().unsqueeze(3) * Psi.float()
    adt = ADT.float()
    if pad:
        zp = lambda x, d: torch.nn.functional.pad(x, [0, 0] * (x.dim() - 1 - d) + [0, pad])
        q, k, psiv = zp(q, 1), zp(k, 1), zp(psiv, 1)
        gamma, ts, adt = zp(gamma, 2), zp(ts, 2), zp(adt, 2)
    Sp = S + pad
    C = Sp // L
    # [B,H,C,L,...]
    qc = q.view(B, C, L, H, R, N).permute(0, 3, 1, 2, 4, 5)
    kc = k.view(B, C, L, H, R, N).permute(0, 3, 1, 2, 4, 5)
    pc = psiv.view(B, C, L, H, R, P).permute(0, 3, 1, 2, 4, 5)
    gam = gamma.view(B, H, C, L)
    tsc = ts.view(B, H, C, L)
    cs = torch.cumsum(adt.view(B, H, C, L), dim=-1)                       # inclusive
    tot = cs[..., -1]                                                     # [B,H,C]
    ks = kc * tsc[..., None, None]
    if mm_dtype is not None:
        def mm(eq, a, b):
            return torch.einsum(eq, a.to(mm_dtype), b.to(mm_dtype)).float()
    else:
        mm = torch.einsum
    # intra-chunk, strictly causal in tokens
    scores = mm("bhcirn,bhcjsn->bhcirjs", qc, ks)
    seg = cs[..., :, None] - cs[..., None, :]                             # [B,H,C,L,L]
    mask = torch.ones(L, L, dtype=torch.bool, device=Q.device).tril(-1)
    decay = torch.where(mask, torch.exp(torch.where(mask, seg, torch.zeros_like(seg))), torch.zeros_like(seg))
    scores = scores * decay[..., :, None, :, None]
    o = mm("bhcirjs,bhcjsp->bhcirp", scores, pc)
    # same-token term
    qk = torch.einsum("bhcirn,bhcisn->bhcirs", qc, kc)
    o = o + gam[..., None, None] * torch.einsum("bhcirs,bhcisp->bhcirp", qk, pc)
    if D is not None:
        o = o + D.float()[None, :, None, None, None, None] * pc
    # chunk-local end states and recurrence over chunks
    w = torch.exp(tot[..., None] - cs)                                    # [B,H,C,L]
    local = mm("bhcjrn,bhcjrp->bhcnp", ks * w[..., None, None], pc)
    state = (initial_state.float() if initial_state is not None
             else torch.zeros(B, H, N, P, dtype=torch.float32, device=Q.device))
    starts = []
    dec_c = torch.exp(tot)
    for c in range(C):
        starts.append(state)
        state = state * dec_c[:, :, c, None, None] + local[:, :, c]
    start = torch.stack(starts, dim=2)                                    # [B,H,C,N,P]
    o = o + torch.exp(cs)[..., None, None] * mm("bhcirn,bhcnp->bhcirp", qc, start)
    o = o.permute(0, 2, 3, 1, 4, 5).reshape(B, Sp, H, R, P)[:, :S]
    y = _gate(o, Z, Zeta, Phi, V.dtype)
    return (y, state) if return_state else y


def angle_cumsum(angles_raw: torch.Tensor, dt: torch.Tensor) -> torch.Tensor:
    """Cumulative rotary angle: ``cumsum_t(angle[b,t,:] * DT[b,h,t])`` -> [B,S,H,A] fp32.

    ``angles_raw`` is [B,S,A] (replicated across heads); ``dt`` is [B,H,S]
    (cppmega/megatron/noconv_mamba_mixer.py:326-333)."""
    prod = angles_raw.float().unsqueeze(2) * dt.float().permute(0, 2, 1).unsqueeze(-1)
    return torch.cumsum(prod, dim=1)
