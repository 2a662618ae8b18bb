"""Wrappers for the small memory-bound kernels around the mixers (rotary-angle prefix sums, ...)."""
from __future__ import annotations

import ctypes

import torch

from .. import functional as F_

ANG_SEG = 512


def declare(L: ctypes.CDLL) -> None:
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    sig = {
        "cm_angle_cumsum_fwd": [vp, vp, i64, i64, i64, vp, vp, i32, i32, i32, i32, vp],
        "cm_angle_cumsum_bwd": [vp, vp, vp, i64, i64, i64, vp, vp, vp, i32, i32, i32, i32, vp],
    }
    f32 = ctypes.c_float
    sig["cm_sparse_mla_fwd"] = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, vp]
    sig["cm_sparse_mla_bwd"] = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, vp, vp]
    sig["cm_router_topk_fwd"] = [vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, vp]
    sig["cm_router_topk_bwd"] = [vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, vp]
    sig["cm_embedding_fwd"] = [vp, vp, vp, i64, i64, i32, vp]
    sig["cm_embedding_bwd"] = [vp, vp, vp, i64, i64, i32, i32, vp]
    sig["cm_ngram_embed_fwd"] = [vp] * 8 + [i32] * 6 + [vp]
    sig["cm_ngram_embed_bwd"] = [vp] * 8 + [i32] * 6 + [vp]
    sig["cm_rope"] = [vp, vp, vp, vp, i64, i32, i32, i32, i64, i64, ctypes.c_float, vp]
    sig["cm_head_reduce"] = [vp, vp, vp, i64, i32, i32, i32, vp]
    sig["cm_indexer_scores"] = [vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]
    sig["cm_indexer_topk"] = [vp, vp, i32, i32, i32, vp]
    for name, args in sig.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = i32


class AngleCumsumFn(torch.autograd.Function):
    """out[b,t,h,a] = sum_{s<=t} raw[b,s,a] * dt[b,h,s]; ``dt`` may be any strided [B,H,S] fp32 view."""

    @staticmethod
    def forward(ctx, raw, dt):
        from . import lib, stream_ptr, _check
        B, S, A = raw.shape
        H = dt.shape[1]
        raw32 = raw.float().contiguous()
        dt32 = dt if dt.dtype == torch.float32 else dt.float()
        out = torch.empty(B, S, H, A, dtype=torch.float32, device=raw.device)
        sb, sh, ss = dt32.stride()
        seg_tot = torch.empty(B * H * ((S + 255) // 256) * A, dtype=torch.float32, device=raw.device)
        _check(lib().cm_angle_cumsum_fwd(raw32.data_ptr(), dt32.data_ptr(), sb, sh, ss, out.data_ptr(), seg_tot.data_ptr(), B, S, H, A,
                                         stream_ptr()), "cm_angle_cumsum_fwd")
        F_.count_launch("angle_cumsum")
        ctx.save_for_backward(raw32, dt32)
        ctx.raw_dtype, ctx.dt_dtype = raw.dtype, dt.dtype
        return out

    @staticmethod
    def backward(ctx, g):
        from . import lib, stream_ptr, _check
        raw32, dt32 = ctx.saved_tensors
        B, S, A = raw32.shape
        H = dt32.shape[1]
        # the kernel overwrites its input with suffix sums; autograd may still own `g`, so work on a private copy
        # unless the incoming tensor is a temporary nobody else can see
        g = g.float().contiguous().clone() if g._base is not None or g.dtype != torch.float32 or not g.is_contiguous() else g.clone()
        nseg = (S + ANG_SEG - 1) // ANG_SEG
        segsum = torch.empty(B * H * nseg * A, dtype=torch.float32, device=g.device)
        draw = torch.empty(B, S, A, dtype=torch.float32, device=g.device)
        ddt = torch.empty(B, H, S, dtype=torch.float32, device=g.device)
        sb, sh, ss = dt32.stride()
        _check(lib().cm_angle_cumsum_bwd(g.data_ptr(), raw32.data_ptr(), dt32.data_ptr(), sb, sh, ss, segsum.data_ptr(),
                                         draw.data_ptr(), ddt.data_ptr(), B, S, H, A, stream_ptr()), "cm_angle_cumsum_bwd")
        F_.count_launch("angle_cumsum_bwd", 3)
        return draw.to(ctx.raw_dtype), ddt.to(ctx.dt_dtype)


def angle_cumsum(raw, dt):
    if raw.shape[-1] > 32 or dt.dim() != 3:
        return None
    return AngleCumsumFn.apply(raw, dt)


def sparse_mla_fwd_raw(q, kv, idx, scale, d_v):
    from . import lib, err_word, stream_ptr, _check
    B, S, Hq, Dq = q.shape
    Skv, topk = kv.shape[1], idx.shape[-1]
    q, kv = q.contiguous(), kv.contiguous()
    idx = idx.to(torch.int32).contiguous()
    out = torch.empty(B, S, Hq, d_v, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, S, Hq, dtype=torch.float32, device=q.device)
    _check(lib().cm_sparse_mla_fwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, Skv,
                                   Hq, Dq, topk, d_v, float(scale), err_word(q.device).data_ptr(), stream_ptr()),
           "cm_sparse_mla_fwd")
    F_.count_launch("sparse_mla")
    return out, lse


class SparseMLAFn(torch.autograd.Function):
    """Sparse latent attention on the tcgen05 kernels: q [B,S,32,128], kv [B,Skv,128] bf16, idx [B,S,256] int32."""

    @staticmethod
    def forward(ctx, q, kv, idx, scale, d_v, precomputed=None):
        q, kv = q.contiguous(), kv.contiguous()
        idx = idx.to(torch.int32).contiguous()
        out, lse = precomputed if precomputed is not None else sparse_mla_fwd_raw(q, kv, idx, scale, d_v)
        ctx.save_for_backward(q, kv, idx, out, lse)
        ctx.scale, ctx.d_v = float(scale), d_v
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import lib, err_word, stream_ptr, _check
        q, kv, idx, out, lse = ctx.saved_tensors
        B, S, Hq, Dq = q.shape
        Skv, topk = kv.shape[1], idx.shape[-1]
        dout = dout.to(torch.bfloat16).contiguous()
        dq = torch.empty_like(q)
        dkv = torch.zeros(B, Skv, Dq, dtype=torch.float32, device=q.device)
        _check(lib().cm_sparse_mla_bwd(q.data_ptr(), kv.data_ptr(), idx.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                       lse.data_ptr(), dq.data_ptr(), dkv.data_ptr(), B, S, Skv, Hq, Dq, topk, ctx.d_v,
                                       ctx.scale, err_word(q.device).data_ptr(), stream_ptr()), "cm_sparse_mla_bwd")
        F_.count_launch("sparse_mla_bwd")
        return dq, dkv.to(kv.dtype), None, None, None, None


def sparse_mla(q, kv, idx, scale, d_v):
    if (q.dtype != torch.bfloat16 or kv.dtype != torch.bfloat16 or q.dim() != 4 or q.shape[2] != 32 or q.shape[3] != 128
            or kv.shape[-1] != 128 or idx.shape[-1] != 256 or d_v != 64):
        return None
    from ...utils.recompute import stashed_call
    return stashed_call("sparse_mla", lambda: sparse_mla_fwd_raw(q.detach(), kv.detach(), idx, scale, d_v),
                        lambda res: SparseMLAFn.apply(q, kv, idx, scale, d_v, res))


def head_reduce(dh: torch.Tensor, G: int):
    """dh [B,S,H,R,N] bf16 -> (sum over the heads of each group [B,S,G,R,N] bf16, sum over tokens [H,R,N] fp32)."""
    from . import lib, stream_ptr, _check
    B, S, H, R, N = dh.shape
    dgrp = torch.empty(B, S, G, R, N, dtype=torch.bfloat16, device=dh.device)
    dbias = torch.zeros(H, R, N, dtype=torch.float32, device=dh.device)
    _check(lib().cm_head_reduce(dh.data_ptr(), dgrp.data_ptr(), dbias.data_ptr(), B * S, H, G, R * N, stream_ptr()),
           "cm_head_reduce")
    F_.count_launch("head_reduce")
    return dgrp, dbias


def indexer_topk(q_idx, k_idx, w, topk: int):
    """Causal top-k key positions per query (int32 [B,S,topk], unordered, -1 padded) on the indexer kernels."""
    if (q_idx.dtype != torch.bfloat16 or k_idx.dtype != torch.bfloat16 or q_idx.dim() != 4 or q_idx.shape[2] != 32
            or q_idx.shape[3] != 64 or q_idx.shape[1] % 4 or q_idx.shape[1] > 32768 or k_idx.shape[1] != q_idx.shape[1]
            or topk > 2048):
        return None
    from . import lib, err_word, stream_ptr, _check
    B, S = q_idx.shape[:2]
    q, k = q_idx.contiguous(), k_idx.contiguous()
    wf = w.float().contiguous()
    scores = torch.empty(B, S, S, dtype=torch.float32, device=q.device)
    out = torch.empty(B, S, topk, dtype=torch.int32, device=q.device)
    _check(lib().cm_indexer_scores(q.data_ptr(), k.data_ptr(), wf.data_ptr(), scores.data_ptr(), B, S, 32, 64,
                                   err_word(q.device).data_ptr(), stream_ptr()), "cm_indexer_scores")
    _check(lib().cm_indexer_topk(scores.data_ptr(), out.data_ptr(), B, S, topk, stream_ptr()), "cm_indexer_topk")
    F_.count_launch("indexer_topk", 2)
    return out


class RouterTopkFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, topk, sigmoid, norm):
        from . import lib, stream_ptr, _check
        T, E = logits.shape
        lf = logits.float().contiguous()
        probs = torch.empty(T, topk, dtype=torch.float32, device=logits.device)
        ids = torch.empty(T, topk, dtype=torch.int64, device=logits.device)
        scores = torch.empty(T, E, dtype=torch.float32, device=logits.device)
        bf = None if bias is None else bias.float().contiguous()
        _check(lib().cm_router_topk_fwd(lf.data_ptr(), None if bf is None else bf.data_ptr(), probs.data_ptr(), ids.data_ptr(),
                                        scores.data_ptr(), T, E, topk, int(sigmoid), int(norm), stream_ptr()),
               "cm_router_topk_fwd")
        F_.count_launch("router_topk")
        ctx.save_for_backward(scores, ids)
        ctx.cfg = (topk, sigmoid, norm, logits.dtype)
        ctx.mark_non_differentiable(ids)
        return probs, ids, scores

    @staticmethod
    def backward(ctx, dprobs, _dids, dscores):
        from . import lib, stream_ptr, _check
        scores, ids = ctx.saved_tensors
        topk, sigmoid, norm, dtype = ctx.cfg
        T, E = scores.shape
        dp = None if dprobs is None else dprobs.float().contiguous()
        dsc = None if dscores is None else dscores.float().contiguous()
        dl = torch.empty(T, E, dtype=torch.float32, device=scores.device)
        _check(lib().cm_router_topk_bwd(scores.data_ptr(), ids.data_ptr(), None if dp is None else dp.data_ptr(),
                                        None if dsc is None else dsc.data_ptr(), dl.data_ptr(), T, E, topk, int(sigmoid),
                                        int(norm), stream_ptr()), "cm_router_topk_bwd")
        F_.count_launch("router_topk_bwd")
        return dl.to(dtype), None, None, None, None


def router_topk(logits, topk, score_function, expert_bias, norm_topk_prob):
    if logits.dim() != 2 or logits.shape[1] > 64 or topk > 8 or score_function not in ("sigmoid", "softmax"):
        return None
    return RouterTopkFn.apply(logits, expert_bias, topk, score_function == "sigmoid", bool(norm_topk_prob))


class NgramEmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, token_ids, mults, bias, sizes, offsets, order):
        from . import lib, stream_ptr, _check
        B, S = token_ids.shape
        NT, max_order = mults.shape
        D = table.shape[1]
        tok = token_ids.long().contiguous()
        tab = table.contiguous()
        consts = [t.long().contiguous() for t in (mults, bias, sizes, offsets, order)]
        out = torch.empty(B, S, NT * D, dtype=table.dtype, device=table.device)
        kind = 0 if table.dtype == torch.float32 else 1
        _check(lib().cm_ngram_embed_fwd(tok.data_ptr(), tab.data_ptr(), *[c.data_ptr() for c in consts], out.data_ptr(),
                                        B, S, NT, D, max_order, kind, stream_ptr()), "cm_ngram_embed_fwd")
        F_.count_launch("ngram_hash_embed")
        ctx.save_for_backward(tok, *consts)
        ctx.meta = (table.shape, table.dtype, kind)
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import lib, stream_ptr, _check
        tok, *consts = ctx.saved_tensors
        shape, dtype, kind = ctx.meta
        B, S = tok.shape
        NT, max_order = consts[0].shape
        dtable = torch.zeros(shape, dtype=torch.float32, device=dout.device)
        dout = dout.to(dtype).contiguous()
        _check(lib().cm_ngram_embed_bwd(tok.data_ptr(), dout.data_ptr(), *[c.data_ptr() for c in consts], dtable.data_ptr(),
                                        B, S, NT, shape[1], max_order, kind, stream_ptr()), "cm_ngram_embed_bwd")
        F_.count_launch("ngram_hash_embed_bwd")
        return dtable.to(dtype), None, None, None, None, None, None


def ngram_hash_embed(token_ids, table, mults, bias, sizes, offsets, order):
    if table.dtype not in (torch.float32, torch.bfloat16) or token_ids.dim() != 2:
        return None
    return NgramEmbedFn.apply(table, token_ids, mults, bias, sizes, offsets, order)


class RopeFn(torch.autograd.Function):
    """Rotate-half RoPE on the last dim of a bf16 tensor [B, S, ..., D] whose last dim is contiguous and whose rows
    (everything but the last dim) are evenly strided, e.g. a column slice of a wider head vector."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        return _rope_launch(x, cos, sin, 1.0)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        return _rope_launch(g, cos, sin, -1.0), None, None


def _row_stride(x: torch.Tensor):
    """Element stride between consecutive rows when ``x`` can be read as [rows, D] with one stride, else None."""
    D = x.shape[-1]
    if x.stride(-1) != 1:
        return None
    st = None
    expect = None
    for size, stride in zip(reversed(x.shape[:-1]), reversed(x.stride()[:-1])):
        if size == 1:
            continue
        if st is None:
            st, expect = stride, stride * size
        elif stride != expect:
            return None
        else:
            expect = stride * size
    return D if st is None else st


def _rope_launch(x, cos, sin, sign):
    from . import lib, stream_ptr, _check
    ld = _row_stride(x)
    if ld is None or ld < x.shape[-1]:
        x = x.contiguous()
        ld = x.shape[-1]
    B, S, D = x.shape[0], x.shape[1], x.shape[-1]
    rows = x.numel() // D
    R = rows // (B * S)
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _check(lib().cm_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), out.data_ptr(), rows, S, R, D, ld, D, sign, stream_ptr()),
           "cm_rope")
    F_.count_launch("rope")
    return out


def apply_rope(x, cos, sin):
    if x.dtype != torch.bfloat16 or x.dim() < 3 or x.shape[-1] % 2 or cos.shape != (x.shape[1], x.shape[-1] // 2):
        return None
    return RopeFn.apply(x, cos.float().contiguous(), sin.float().contiguous())


class EmbeddingFn(torch.autograd.Function):
    """Row gather; the backward adds the output-gradient rows straight into the weight's flat gradient buffer when the
    optimizer allows it (``w.fuse_wgrad_accumulation``), else into a fresh fp32 tensor."""

    @staticmethod
    def forward(ctx, ids, w):
        from . import lib, stream_ptr, _check
        flat = ids.reshape(-1).long().contiguous()
        V, H = w.shape
        out = torch.empty(flat.numel(), H, dtype=torch.bfloat16, device=w.device)
        _check(lib().cm_embedding_fwd(flat.data_ptr(), w.data_ptr(), out.data_ptr(), flat.numel(), V, H, stream_ptr()),
               "cm_embedding_fwd")
        F_.count_launch("embedding")
        ctx.save_for_backward(flat)
        ctx.w = w
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        from . import lib, stream_ptr, _check, wgrad_into_main_grad
        (flat,) = ctx.saved_tensors
        w = ctx.w
        V, H = w.shape
        d2 = dout.reshape(-1, H)
        if d2.dtype != torch.bfloat16 or not d2.is_contiguous():
            d2 = d2.to(torch.bfloat16).contiguous()

        def run(out, acc):
            fresh = out is None
            if fresh:
                out = torch.zeros(V, H, dtype=torch.float32, device=w.device)
            _check(lib().cm_embedding_bwd(flat.data_ptr(), d2.data_ptr(), out.data_ptr(), flat.numel(), V, H,
                                          0 if out.dtype == torch.float32 else 1, stream_ptr()), "cm_embedding_bwd")
            F_.count_launch("embedding_bwd")
            return out.to(w.dtype) if fresh else out

        return None, wgrad_into_main_grad(w, run)


def embedding(ids, w):
    if w.dtype != torch.bfloat16 or w.dim() != 2 or w.shape[1] % 8 or not w.is_contiguous() or ids.numel() == 0:
        F_._miss("embedding(shape/dtype)", w)
        return None
    return EmbeddingFn.apply(ids, w)


def register() -> None:
    F_.register_cuda("embedding", embedding)
    F_.register_cuda("router_topk", router_topk)
    F_.register_cuda("ngram_hash_embed", ngram_hash_embed)
    F_.register_cuda("apply_rope", apply_rope)
    F_.register_cuda("indexer_topk", indexer_topk)
    F_.register_cuda("angle_cumsum", angle_cumsum)
    F_.register_cuda("sparse_mla", sparse_mla)
