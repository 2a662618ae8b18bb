"""Plain-PyTorch fp32 definitions of the framework's fused operators.

Every CUDA kernel in :mod:`cppmega_b200.ops` is tested against the function of
the same name here, and the CPU (gloo) configuration runs on these directly.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------
# normalisation / activation
# ---------------------------------------------------------------------------

def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-5,
            residual: Optional[torch.Tensor] = None):
    """``y = x * rsqrt(mean(x^2) + eps) * w`` computed in fp32; with ``residual`` the
    sum ``x + residual`` is normalised and also returned."""
    if residual is not None:
        x = x + residual
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    y = y.to(x.dtype)
    return (y, x) if residual is not None else y


def rmsnorm_gated(x: torch.Tensor, weight: torch.Tensor, z: Optional[torch.Tensor] = None,
                  eps: float = 1e-5, group_size: Optional[int] = None, norm_before_gate: bool = True):
    """Grouped RMS norm with an optional SiLU gate
    (semantics of the gated norm used at cppmega/megatron/cppmega_mamba3_tp_mixer.py:341-357)."""
    xf = x.float()
    if z is not None and not norm_before_gate:
        xf = xf * F.silu(z.float())
    d = xf.shape[-1]
    g = group_size or d
    xg = xf.reshape(*xf.shape[:-1], d // g, g)
    y = (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + eps)).reshape(xf.shape)
    y = y * weight.float()
    if z is not None and norm_before_gate:
        y = y * F.silu(z.float())
    return y.to(x.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(a) * b`` for ``gate_up = [a | b]`` along the last dim."""
    a, b = gate_up.chunk(2, dim=-1)
    return (F.silu(a.float()) * b.float()).to(gate_up.dtype)


# ---------------------------------------------------------------------------
# rotary embedding (attention)
# ---------------------------------------------------------------------------

def rope_tables(seq: int, dim: int, base: float, device=None, offset: int = 0):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    t = torch.arange(offset, offset + seq, device=device, dtype=torch.float32)
    fr = torch.outer(t, inv)
    return torch.cos(fr), torch.sin(fr)     # [S, dim/2]


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on the last dim.  x: [B,S,...,D]; cos/sin: [S, D/2]."""
    d2 = x.shape[-1] // 2
    shape = [1, x.shape[1]] + [1] * (x.dim() - 3) + [d2]
    c, s = cos.view(shape), sin.view(shape)
    xf = x.float()
    a, b = xf[..., :d2], xf[..., d2:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1).to(x.dtype)


# ---------------------------------------------------------------------------
# ngram hash
# ---------------------------------------------------------------------------

def ngram_hash_indices(token_ids: torch.Tensor, mults: torch.Tensor, bias: torch.Tensor,
                       table_sizes: torch.Tensor, table_offsets: torch.Tensor,
                       order_of_table: torch.Tensor) -> torch.Tensor:
    """Row index into the unified table for every (batch, position, table).

    ``hash = ((xor_{p < order} mult[t,p] * tok[s-p]) xor bias[t]) mod size[t] + offset[t]`` with
    positions before the start of the sequence reading token 0
    (cppmega/features/engram/ngram_hash.py:117-141).  Returns int64 [B,S,T].
    """
    tok = token_ids.long()
    B, S = tok.shape
    T, max_order = mults.shape
    h = torch.zeros(B, S, T, dtype=torch.long, device=tok.device)
    for p in range(max_order):
        shifted = torch.zeros_like(tok)
        if p == 0:
            shifted = tok
        elif p < S:
            shifted[:, p:] = tok[:, :-p]
        use = (order_of_table > p).long()                  # [T]
        h = h ^ (shifted.unsqueeze(-1) * mults[:, p].long() * use)
    h = h ^ bias.long()
    h = h % table_sizes.long()
    return h + table_offsets.long()


def ngram_hash_embed(token_ids, table, mults, bias, table_sizes, table_offsets, order_of_table):
    idx = ngram_hash_indices(token_ids, mults, bias, table_sizes, table_offsets, order_of_table)
    B, S, T = idx.shape
    return F.embedding(idx, table).reshape(B, S, T * table.shape[1])


# ---------------------------------------------------------------------------
# M2RNN
# ---------------------------------------------------------------------------

def m2rnn_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, W: torch.Tensor, f: torch.Tensor,
               h0: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Matrix-state recurrence ``h <- f h + (1-f) tanh(h W + k (x) v)``, ``y = q . h``.

    q,k: [B,S,Hq|Hk,K]; v: [B,S,H,V]; W: [H,V,V]; f: [B,S,H]; head counts of 1
    broadcast.  Returns (y [B,S,H,V], h_last [B,H,K,V])
    (cppmega/megatron/m2rnn_spec.py:57-99)."""
    B, S, _, Kd = q.shape
    H, Vd = v.shape[2], v.shape[3]
    qf = q.float().expand(B, S, H, Kd) if q.shape[2] == 1 else q.float()
    kf = k.float().expand(B, S, H, Kd) if k.shape[2] == 1 else k.float()
    vf, Wf, ff = v.float(), W.float(), f.float()
    h = torch.zeros(B, H, Kd, Vd, dtype=torch.float32, device=q.device) if h0 is None else h0.float()
    ys = []
    for t in range(S):
        x = kf[:, t, :, :, None] * vf[:, t, :, None, :]
        hn = torch.tanh(torch.matmul(h, Wf) + x)
        ft = ff[:, t, :, None, None]
        h = ft * h + (1.0 - ft) * hn
        ys.append(torch.einsum("bhk,bhkv->bhv", qf[:, t], h))
    return torch.stack(ys, dim=1).to(v.dtype), h


# ---------------------------------------------------------------------------
# DSA: indexer scores, top-k, sparse MLA
# ---------------------------------------------------------------------------

def indexer_scores(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``score[b,i,j] = sum_h w[b,i,h] relu(q_idx[b,i,h,:] . k_idx[b,j,:])`` in fp32
    (cppmega/megatron/dsa_indexer_fused_patch.py:71-133)."""
    qf, kf, wf = q_idx.float(), k_idx.float(), w.float()
    out = None
    for h in range(qf.shape[2]):        # one head at a time: never holds [B,S,H,S]
        s = F.relu(torch.einsum("bid,bjd->bij", qf[:, :, h], kf)) * wf[:, :, h].unsqueeze(-1)
        out = s if out is None else out + s
    return out


def indexer_topk(q_idx, k_idx, w, topk: int, q_offset: Optional[int] = None) -> torch.Tensor:
    """Causal top-k key positions per query; int32 [B,S,topk], -1 where fewer than
    ``topk`` keys are visible.  Query ``i`` sits at sequence position ``q_offset + i`` and sees the keys at positions
    ``<=`` its own (default: the queries are the last ``S`` positions of the key sequence)."""
    sc = indexer_scores(q_idx, k_idx, w)
    B, S, Sk = sc.shape
    off = Sk - S if q_offset is None else int(q_offset)
    causal = torch.ones(S, Sk, dtype=torch.bool, device=sc.device).tril(off)
    sc = sc.masked_fill(~causal, float("-inf"))
    kk = min(topk, Sk)
    vals, idx = torch.topk(sc, kk, dim=-1)
    idx = torch.where(torch.isinf(vals), torch.full_like(idx, -1), idx).to(torch.int32)
    if kk < topk:
        idx = F.pad(idx, (0, topk - kk), value=-1)
    return idx


def sparse_mla(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, scale: float, d_v: int):
    """Sparse latent attention.  q [B,S,Hq,D]; kv [B,Skv,D] (one shared KV head; V is
    the first ``d_v`` channels); indices int [B,S,topk] with -1 = masked.
    Returns (out [B,S,Hq,d_v], lse [B,S,Hq] natural log)
    (contract at cppmega/megatron/sparse_mla_ops/sparse_mla.py:17-39)."""
    B, S, Hq, Dq = q.shape
    valid = indices >= 0
    idx = indices.clamp(min=0).long()
    T = idx.shape[-1]
    # gather rows of the (un-expanded) KV so that the backward scatter-adds into [B,Skv,D]
    g = torch.gather(kv.float(), 1, idx.reshape(B, S * T, 1).expand(B, S * T, Dq)).view(B, S, T, Dq)
    s = torch.einsum("bshd,bstd->bsht", q.float(), g) * scale
    s = s.masked_fill(~valid.unsqueeze(2), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    out = torch.einsum("bsht,bstd->bshd", p, g[..., :d_v])
    return out.to(q.dtype), lse


def indexer_kl_loss(attn_q, attn_k, scale, q_idx, k_idx, w, coeff: float = 1.0):
    """``coeff * mean_{b,i} KL(mean_h softmax(q k^T scale) || softmax(index scores))`` with
    causal masking (cppmega/megatron/dsa_splitk_indexer_loss.py:313-321)."""
    B, S = attn_q.shape[:2]
    causal = torch.ones(S, S, dtype=torch.bool, device=attn_q.device).tril()
    a = torch.einsum("bihd,bjhd->bhij", attn_q.float(), attn_k.float()) * scale
    a = a.masked_fill(~causal, float("-inf"))
    p = torch.softmax(a, dim=-1).mean(dim=1)                                      # [B,S,S]
    sc = indexer_scores(q_idx, k_idx, w).masked_fill(~causal, float("-inf"))
    logq = torch.log_softmax(sc, dim=-1)
    kl = torch.where(p > 0, p * (torch.log(p.clamp_min(1e-30)) - logq), torch.zeros_like(p)).sum(-1)
    return coeff * kl.mean()


def indexer_kl_loss_chunked(attn_q, attn_k, scale, q_idx, k_idx, w, coeff: float = 1.0, rows: int = 512):
    """Same value and gradients as :func:`indexer_kl_loss`, evaluated ``rows`` query positions at a time with each
    block recomputed in backward: the transient is ``[B, H, rows, S]`` instead of ``[B, H, S, S]`` (7 GiB per layer
    at the NAM56R shape), which is what the reference's two-stage split kernels and its fused warm-up kernel buy
    (cppmega/megatron/dsa_splitk_indexer_loss.py:56-321, cppmega/megatron/lemyx_dsa_warmup.py:77-178)."""
    from torch.utils.checkpoint import checkpoint
    B, S = attn_q.shape[:2]
    Sk = attn_k.shape[1]

    def block(aq, ak, qi, ki, wi, r0):
        n = aq.shape[1]
        pos = torch.arange(r0, r0 + n, device=aq.device)
        causal = torch.arange(Sk, device=aq.device)[None, :] <= (pos + (Sk - S))[:, None]              # [n, Sk]
        a = torch.einsum("bihd,bjhd->bhij", aq.float(), ak.float()) * scale
        p = torch.softmax(a.masked_fill(~causal, float("-inf")), dim=-1).mean(dim=1)                  # [B, n, Sk]
        sc = indexer_scores(qi, ki, wi).masked_fill(~causal, float("-inf"))
        logq = torch.log_softmax(sc, dim=-1)
        return torch.where(p > 0, p * (torch.log(p.clamp_min(1e-30)) - logq), torch.zeros_like(p)).sum()

    total = attn_q.new_zeros((), dtype=torch.float32)
    for r0 in range(0, S, rows):
        r1 = min(S, r0 + rows)
        args = (attn_q[:, r0:r1], attn_k, q_idx[:, r0:r1], k_idx, w[:, r0:r1], r0)
        needs = any(torch.is_tensor(t) and t.requires_grad for t in args)
        total = total + (checkpoint(block, *args, use_reentrant=False) if needs else block(*args))
    return coeff * total / (B * S)


def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[b, s, c] = silu(bias[c] + sum_j weight[c, j] * x[b, s - (k-1) + j, c])`` with zeros before the sequence start:
    the depthwise ``nn.Conv1d(C, C, k, groups=C, padding=k-1)`` truncated to S outputs, on a channels-last tensor."""
    S, k = x.shape[1], weight.shape[1]
    y = F.conv1d(x.transpose(1, 2), weight.unsqueeze(1).to(x.dtype), None if bias is None else bias.to(x.dtype),
                 padding=k - 1, groups=x.shape[2])[..., :S]
    return F.silu(y).transpose(1, 2)


def dsa_warmup_attention_and_kl(q, k, v, scale, q_idx, k_idx, w, coeff: float = 1.0, rows: int = 512):
    """Indexer warm-up in one pass: dense causal attention output AND the indexer KL loss from the same score blocks.

    During warm-up the sparse layers attend to every key (the indexer is not trusted yet) while the indexer is trained
    to imitate the head-averaged attention distribution.  Per block of ``rows`` queries the scores ``q k^T`` are formed
    once; their softmax gives the output ``P v`` and, detached and averaged over heads, the target of
    ``KL(target || softmax(index scores))``.  Blocks are recomputed in backward, so the transient is
    ``[B, H, rows, S]``.  q / k [B,S,H,Dqk], v [B,S,H,Dv]; returns (out [B,S,H,Dv], loss).  Same value as
    :func:`indexer_kl_loss` on detached q / k plus ordinary dense attention; the reference reaches this through an external
    fused FlashAttention + lightning-indexer + KL kernel (cppmega/megatron/lemyx_dsa_warmup.py:77-178)."""
    from torch.utils.checkpoint import checkpoint
    B, S, H, _ = q.shape

    def block(qb, kk, vv, qi, ki, wi, r0):
        n = qb.shape[1]
        pos = torch.arange(r0, r0 + n, device=qb.device)
        causal = torch.arange(S, device=qb.device)[None, :] <= pos[:, None]                           # [n, S]
        a = torch.einsum("bihd,bjhd->bhij", qb.float(), kk.float()) * scale
        p = torch.softmax(a.masked_fill(~causal, float("-inf")), dim=-1)                              # [B, H, n, S]
        out = torch.einsum("bhij,bjhd->bihd", p, vv.float()).to(vv.dtype)
        target = p.detach().mean(dim=1)                                                               # [B, n, S]
        sc = indexer_scores(qi, ki, wi).masked_fill(~causal, float("-inf"))
        logq = torch.log_softmax(sc, dim=-1)
        kl = torch.where(target > 0, target * (torch.log(target.clamp_min(1e-30)) - logq), torch.zeros_like(target)).sum()
        return out, kl

    outs = []
    total = q.new_zeros((), dtype=torch.float32)
    for r0 in range(0, S, rows):
        r1 = min(S, r0 + rows)
        args = (q[:, r0:r1], k, v, q_idx[:, r0:r1], k_idx, w[:, r0:r1], r0)
        needs = any(torch.is_tensor(t) and t.requires_grad for t in args)
        o, kl = checkpoint(block, *args, use_reentrant=False) if needs else block(*args)
        outs.append(o)
        total = total + kl
    return torch.cat(outs, dim=1), coeff * total / (B * S)


# ---------------------------------------------------------------------------
# fused linear + cross entropy
# ---------------------------------------------------------------------------

def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                         ignore_index: int = -100, reduction: str = "none") -> torch.Tensor:
    """CE of ``hidden @ weight^T`` against ``labels`` without exposing logits.
    hidden [T,H]; weight [V,H]; labels [T].  ``none`` gives per-token loss with 0 at
    ignored rows; ``sum``/``mean`` reduce over non-ignored rows
    (contract at cppmega/megatron/apply_linear_ce_patch.py:263-310)."""
    logits = hidden.float() @ weight.float().t()
    loss = F.cross_entropy(logits, labels.long(), ignore_index=ignore_index, reduction="none")
    if reduction == "none":
        return loss
    if reduction == "sum":
        return loss.sum()
    if reduction == "mean":
        n = (labels != ignore_index).sum().clamp_min(1)
        return loss.sum() / n
    raise ValueError(f"unknown reduction {reduction!r}")


# ---------------------------------------------------------------------------
# MoE routing
# ---------------------------------------------------------------------------

def router_topk(logits: torch.Tensor, topk: int, score_function: str = "sigmoid",
                expert_bias: Optional[torch.Tensor] = None, norm_topk_prob: bool = True):
    """Return (probs [T,k] fp32, expert ids [T,k] int64, scores [T,E]).  Selection uses
    ``scores + expert_bias``; the combine weights use the unbiased scores
    (cppmega/recipes/nam56r_nemo_recipe.py:321-337)."""
    lf = logits.float()
    scores = torch.sigmoid(lf) if score_function == "sigmoid" else torch.softmax(lf, dim=-1)
    sel = scores + expert_bias.float() if expert_bias is not None else scores
    _, ids = torch.topk(sel, topk, dim=-1)
    probs = torch.gather(scores, 1, ids)
    if norm_topk_prob and (score_function == "sigmoid" or topk > 1):
        probs = probs / probs.sum(-1, keepdim=True).clamp_min(1e-20)
    return probs, ids, scores


def moe_aux_loss(scores: torch.Tensor, ids: torch.Tensor, num_experts: int, topk: int, coeff: float):
    """Switch-style load-balancing loss ``coeff * E * sum_e f_e * P_e``."""
    T = scores.shape[0]
    counts = torch.zeros(num_experts, dtype=torch.float32, device=scores.device)
    counts.scatter_add_(0, ids.reshape(-1), torch.ones(ids.numel(), dtype=torch.float32, device=scores.device))
    f = counts / max(T * topk, 1)
    p = (scores / scores.sum(-1, keepdim=True).clamp_min(1e-20)).mean(0)
    return coeff * num_experts * (f * p).sum()


def grouped_gemm(x: torch.Tensor, w: torch.Tensor, counts: Sequence[int]) -> torch.Tensor:
    """Rows of ``x`` are sorted by expert; ``w`` is [E, K, N]; ``counts[e]`` rows use ``w[e]``."""
    outs, pos = [], 0
    for e, n in enumerate(counts):
        n = int(n)
        outs.append(x[pos:pos + n] @ w[e])
        pos += n
    return torch.cat(outs, dim=0) if outs else x.new_zeros(0, w.shape[-1])


# ---------------------------------------------------------------------------
# MXFP8 (E4M3 payload + E8M0 1x32 scales)
# ---------------------------------------------------------------------------

E4M3_MAX = 448.0


def e8m0_from_amax(amax: torch.Tensor) -> torch.Tensor:
    """Scale byte ``clamp(ceil(log2(amax / 448)) + 127, 1, 254)``; zero blocks get 127
    (cppmega/megatron/cuda_ext/quantized_muon_momentum.cu:75-91)."""
    a = amax.float()
    e = torch.ceil(torch.log2(a.clamp_min(1e-38) / E4M3_MAX)) + 127.0
    e = torch.where(a > 0, e, torch.full_like(e, 127.0))
    return e.clamp(1, 254).to(torch.uint8)


def mxfp8_quantize(x: torch.Tensor, axis: int = -1):
    """Block-scale ``x`` along ``axis`` in groups of 32.  Returns (payload float8_e4m3fn,
    scale uint8 with the block axis divided by 32)."""
    xf = x.float().movedim(axis, -1)
    shp = xf.shape
    assert shp[-1] % 32 == 0, "MXFP8 needs the scaled axis to be a multiple of 32"
    blk = xf.reshape(*shp[:-1], shp[-1] // 32, 32)
    sc = e8m0_from_amax(blk.abs().amax(-1))
    mult = torch.exp2(127.0 - sc.float()).unsqueeze(-1)
    pay = (blk * mult).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).reshape(shp)
    return pay.movedim(-1, axis).contiguous(), sc.movedim(-1, axis).contiguous()


def mxfp8_dequantize(payload: torch.Tensor, scale: torch.Tensor, axis: int = -1) -> torch.Tensor:
    p = payload.float().movedim(axis, -1)
    s = scale.movedim(axis, -1).float()
    shp = p.shape
    out = p.reshape(*shp[:-1], shp[-1] // 32, 32) * torch.exp2(s - 127.0).unsqueeze(-1)
    return out.reshape(shp).movedim(-1, axis).contiguous()


def swizzle_scales_128x4(scale: torch.Tensor) -> torch.Tensor:
    """Rearrange row-major ``[rows, kb]`` scales into the 128x4 tile order that
    block-scaled tensor-core instructions read: tiles of 128 rows x 4 blocks stored as
    ``[32][4][4]`` (row%32, row//32, kb%4), tiles ordered row-tile major
    (index map at cppmega/megatron/flashinfer_mxfp8_gemm.py:146-160)."""
    rows, kb = scale.shape
    pr, pk = (-rows) % 128, (-kb) % 4
    s = F.pad(scale, (0, pk, 0, pr), value=127) if (pr or pk) else scale
    R, Kb = s.shape
    s = s.view(R // 128, 4, 32, Kb // 4, 4).permute(0, 3, 2, 1, 4)
    return s.contiguous().view(-1)


# ---------------------------------------------------------------------------
# q8 Muon momentum
# ---------------------------------------------------------------------------

def qmuon_update(q: torch.Tensor, absmax: torch.Tensor, grad: torch.Tensor, beta: float):
    """Blockwise (256) int8 momentum: ``m = beta * deq(q) + (1-beta) g``; requantise; return
    (q_new int8, absmax_new fp32, m fp32, per-block sum of squares)
    (kernel math at cppmega/megatron/cuda_ext/quantized_muon_momentum.cu:283-340)."""
    n = grad.numel()
    nb = (n + 255) // 256
    g = F.pad(grad.float().reshape(-1), (0, nb * 256 - n)).view(nb, 256)
    qq = F.pad(q.reshape(-1).float(), (0, nb * 256 - n)).view(nb, 256)
    m = beta * qq * (absmax.float().view(nb, 1) / 127.0) + (1.0 - beta) * g
    am = m.abs().amax(-1)
    inv = torch.where(am > 0, 127.0 / am, torch.zeros_like(am)).unsqueeze(-1)
    r = m * inv
    qn = (torch.sign(r) * torch.floor(r.abs() + 0.5)).clamp(-127, 127).to(torch.int8)
    ss = (m * m).sum(-1)
    return qn.view(-1)[:n].view(q.shape), am, m.view(-1)[:n].view(grad.shape), ss


def newton_schulz(G: torch.Tensor, steps: int = 5, coeffs=(3.4445, -4.7750, 2.0315), eps: float = 1e-7):
    """Quintic Newton-Schulz orthogonalisation used by Muon; bf16 matmuls on GPU."""
    a, b, c = coeffs
    X = G.to(torch.bfloat16 if G.is_cuda else torch.float32)
    t = X.shape[-2] > X.shape[-1]
    if t:
        X = X.transpose(-1, -2)
    X = X / (X.float().norm(dim=(-2, -1), keepdim=True) + eps).to(X.dtype)
    for _ in range(steps):
        A = X @ X.transpose(-1, -2)
        Bm = b * A + c * (A @ A)
        X = a * X + Bm @ X
    if t:
        X = X.transpose(-1, -2)
    return X.to(G.dtype)


_ = math
