"""This package's kernels against the reference project's own runnable kernels, same GPU, same harness.

    python -m cppmega_b200.tools.kernel_bench_reference <case> [--small] [--out file.json]
    cases: m2rnn  sparse_mla  indexer  linear_ce  gemm

The reference's end-to-end training stack (Megatron-LM fork, TransformerEngine fork, mamba_ssm) cannot be installed
offline, but several of its hot kernels need nothing except ``triton`` / ``tilelang`` / ``liger_kernel`` and ``torch``.
They are imported UNMODIFIED from ``baseline/_ref`` (``pip install --target baseline/_ref <reference tree>``) and timed
with the same CUDA-event harness, shapes, warm-up and L2 flush as this package's kernel:

* ``m2rnn``       Triton M2RNN scan fwd + bwd (cppmega/megatron/m2rnn_triton.py:1316) vs ``ops/csrc/m2rnn.cu``;
* ``sparse_mla``  TileLang SparseMLA fwd / bwd (cppmega/megatron/sparse_mla_ops/sparse_mla.py:356-411 over
                  tilelang_sparse_mla_fwd.py:293 and tilelang_sparse_mla_bwd.py:422) vs ``ops/csrc/sparse_mla.cu``;
* ``indexer``     per-head bmm index scores + ``torch.topk`` (cppmega/megatron/dsa_indexer_fused_patch.py:71-133) vs
                  ``ops/csrc/indexer.cu``;
* ``linear_ce``   Liger fused linear cross-entropy as the reference's MTP head calls it
                  (cppmega/megatron/mtp_liger_ce.py:51-53) vs the LM + MTP head of ``ops/csrc/cross_entropy.cu``;
* ``gemm``        ``torch.matmul`` (cuBLASLt, what TE linears run) vs ``ops/csrc/gemm_tcgen05.cu``.

Run ONE case per process: a reference kernel that fails to compile or faults must not take the other measurements
with it.  A case whose reference side cannot run prints ``"reference_unavailable": "<why>"`` beside this package's time.
Each record carries ``ours_ms``, ``reference_ms`` and ``speedup`` = reference_ms / ours_ms (> 1: this package is faster).
"""
from __future__ import annotations

import json
import os
import sys
import traceback
from typing import Callable, List, Optional

import torch

from .kernel_bench import ROOT, time_ms

REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _ref_import(module: str):
    import importlib
    if not os.path.isdir(os.path.join(REF_DIR, "cppmega")):
        raise ImportError("baseline/_ref/cppmega is not installed")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module(module)


def _try(fn: Callable[[], float]):
    """(milliseconds, None) or (None, one-line reason)."""
    try:
        return fn(), None
    except Exception as e:                      # compile errors of the JIT kernels, missing packages
        tb = traceback.format_exc().strip().splitlines()
        return None, f"{type(e).__name__}: {str(e).splitlines()[0][:200] if str(e) else tb[-1][:200]}"


def _rec(kernel: str, shape: dict, ours_ms: float, ref_ms: Optional[float], why: Optional[str], **extra) -> dict:
    r = {"kernel": kernel, **shape, "ours_ms": ours_ms}
    if ref_ms is not None:
        r["reference_ms"] = ref_ms
        r["speedup"] = ref_ms / ours_ms
    else:
        r["reference_unavailable"] = why
    r.update(extra)
    return r


def bench_m2rnn(small: bool) -> List[dict]:
    """R-layer shape of NAM56R: 51 value heads (hidden 4096 / (64 + 16)), one shared q / k head, B4 x S4096."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels2
    B, S, H, Kd, Vd = (1, 512, 8, 64, 16) if small else (4, 4096, 51, 64, 16)
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    q, k = (rn(B, S, 1, Kd) * 0.3).bfloat16(), (rn(B, S, 1, Kd) * 0.3).bfloat16()
    v = rn(B, S, H, Vd).bfloat16()
    W = (rn(H, Vd, Vd) * 0.2).bfloat16()
    f = torch.sigmoid(rn(B, S, H))
    out = []

    def ours(with_bwd: bool):
        a = [t.detach().clone().requires_grad_(with_bwd) for t in (q, k, v, W, f)]

        def step():
            y = kernels2.m2rnn_scan(*a)
            if with_bwd:
                for t in a:
                    t.grad = None
                y.backward(dy)
        y0 = kernels2.m2rnn_scan(*a)
        dy = torch.ones_like(y0)
        return time_ms(step, iters=5)

    def ref(with_bwd: bool):
        fn = _ref_import("cppmega.megatron.m2rnn_triton").m2rnn_scan_triton
        a = [t.detach().clone().requires_grad_(with_bwd) for t in (q, k, v, W.to(q.dtype), f.to(q.dtype))]

        def step():
            y, _ = fn(*a)
            if with_bwd:
                for t in a:
                    t.grad = None
                y.backward(dy)
        y0, _ = fn(*a)
        dy = torch.ones_like(y0)
        return time_ms(step, iters=5)

    shape = {"B": B, "S": S, "heads": H, "k_dim": Kd, "v_dim": Vd}
    for wb, name in ((False, "m2rnn scan fwd"), (True, "m2rnn scan fwd+bwd")):
        o = ours(wb)
        cu.check_errors()
        r, why = _try(lambda: ref(wb))
        out.append(_rec(name, shape, o, r, why, reference="Triton m2rnn_scan_triton"))
    return out


def bench_sparse_mla(small: bool) -> List[dict]:
    """Absorbed DSA attention of NAM56R: 32 heads, latent 64 + rope 64 = 128, V = first 64 channels, top-k 256."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels4
    out = []
    for B, S in ([(1, 1024)] if small else [(4, 4096), (1, 16384)]):
        g = torch.Generator(device="cuda").manual_seed(1)
        q = (torch.randn(B, S, 32, 128, device="cuda", generator=g) * 0.3).bfloat16()
        kv = (torch.randn(B, S, 128, device="cuda", generator=g) * 0.3).bfloat16()
        qi = torch.randn(B, S, 32, 64, device="cuda", generator=g).bfloat16()
        ki = torch.randn(B, S, 64, device="cuda", generator=g).bfloat16()
        wi = torch.rand(B, S, 32, device="cuda", generator=g)
        idx = kernels4.indexer_topk(qi, ki, wi, 256)                      # causal, -1 where fewer than 256 keys are visible
        scale = 128 ** -0.5
        shape = {"B": B, "S": S, "heads": 32, "dim": 128, "d_v": 64, "topk": 256}

        qo, kvo = q.clone().requires_grad_(), kv.clone().requires_grad_()
        o = kernels4.SparseMLAFn.apply(qo, kvo, idx, scale, 64)
        go = torch.randn_like(o)
        ours_f = time_ms(lambda: kernels4.sparse_mla_fwd_raw(q, kv, idx, scale, 64), iters=5)
        ours_b = time_ms(lambda: torch.autograd.grad(o, (qo, kvo), go, retain_graph=True), iters=5)
        cu.check_errors()

        def ref_pair():
            Fn = _ref_import("cppmega.megatron.sparse_mla_ops.sparse_mla").SparseMLA
            qr, kvr = q.clone().requires_grad_(), kv.view(B, S, 1, 128).clone().requires_grad_()
            idr = idx.view(B, S, 1, 256).contiguous()
            with torch.no_grad():
                f_ms = time_ms(lambda: Fn.apply(qr, kvr, idr, scale, 64), iters=5)
            orf, _ = Fn.apply(qr, kvr, idr, scale, 64)
            b_ms = time_ms(lambda: torch.autograd.grad(orf, (qr, kvr), go, retain_graph=True), iters=5)
            err = float((orf.float() - o.float()).norm() / o.float().norm())
            return f_ms, b_ms, err
        res, why = _try(ref_pair)
        rf, rb, err = res if res is not None else (None, None, None)
        out.append(_rec("sparse_mla fwd", shape, ours_f, rf, why, reference="TileLang sparse_mla_fwd_interface",
                        rel_diff_vs_reference=err))
        out.append(_rec("sparse_mla bwd", shape, ours_b, rb, why, reference="TileLang sparse_mla_bwd"))
        del q, kv, qo, kvo, o, go
        torch.cuda.empty_cache()
    return out


def bench_indexer(small: bool) -> List[dict]:
    """Index scores + top-k 256 with 32 index heads x 64 (NAM56R), at the training shape and the long-context points."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels4
    out = []
    for B, S in ([(1, 1024)] if small else [(4, 4096), (1, 8192), (1, 16384), (1, 32768)]):
        g = torch.Generator(device="cuda").manual_seed(2)
        qi = torch.randn(B, S, 32, 64, device="cuda", generator=g).bfloat16()
        ki = torch.randn(B, S, 64, device="cuda", generator=g).bfloat16()
        wi = torch.rand(B, S, 32, device="cuda", generator=g)
        ours = time_ms(lambda: kernels4.indexer_topk(qi, ki, wi, 256), iters=5)
        cu.check_errors()

        def ref():
            score = _ref_import("cppmega.megatron.dsa_indexer_fused_patch").compute_index_scores_fused_bf16
            qs, ks, ws = qi.transpose(0, 1).contiguous(), ki.transpose(0, 1).contiguous(), wi.transpose(0, 1).contiguous().bfloat16()
            causal = torch.ones(S, S, dtype=torch.bool, device="cuda").tril()

            def step():
                sc = score(qs, ws, ks)                                     # [B, S, S] fp32
                sc.masked_fill_(~causal, float("-inf"))
                return torch.topk(sc, 256, dim=-1).indices
            return time_ms(step, iters=3, warmup=1)
        r, why = _try(ref)
        out.append(_rec("indexer scores + top-k", {"B": B, "S": S, "index_heads": 32, "index_dim": 64, "topk": 256}, ours, r, why,
                        reference="per-head bmm (compute_index_scores_fused_bf16) + torch.topk"))
        del qi, ki, wi
        torch.cuda.empty_cache()
    return out


def bench_linear_ce(small: bool) -> List[dict]:
    """LM head + 2 MTP heads of one micro-batch: T = 3 x 16384 rows, hidden 4096, vocabulary 131072, fwd + bwd."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import extra
    T, H, V = (4096, 1024, 32768) if small else (49152, 4096, 131072)
    g = torch.Generator(device="cuda").manual_seed(3)
    h = (torch.randn(T, H, device="cuda", generator=g)).bfloat16()
    w = (torch.randn(V, H, device="cuda", generator=g) * 0.02).bfloat16()
    lab = torch.randint(0, V, (T,), device="cuda", generator=g)
    rw = torch.full((T,), 1.0 / T, device="cuda")

    def ours():
        hh, ww = h.clone().requires_grad_(), w.clone().requires_grad_()

        def step():
            hh.grad = ww.grad = None
            loss, _ = extra.linear_cross_entropy_weighted(hh, ww, lab, rw, -100)
            loss.backward()
        return time_ms(step, iters=3, warmup=1)

    def ref():
        from liger_kernel.ops.fused_linear_cross_entropy import LigerFusedLinearCrossEntropyFunction as Fn
        _ref_import("cppmega.megatron.mtp_liger_ce")                       # the reference module that makes this call
        hh, ww = h.clone().requires_grad_(), w.clone().requires_grad_()

        def step():
            hh.grad = ww.grad = None
            res = Fn.apply(hh, ww, lab, None, None, -100, 0.0, 0.0, "mean", None, False)     # the reference's argument list
            loss = res[0] if isinstance(res, (tuple, list)) else res
            loss.backward()
        return time_ms(step, iters=3, warmup=1)
    o = ours()
    cu.check_errors()
    r, why = _try(ref)
    return [_rec("fused linear cross-entropy fwd+bwd", {"rows": T, "hidden": H, "vocab": V}, o, r, why,
                 reference="Liger LigerFusedLinearCrossEntropyFunction (reduction mean)")]


def bench_gemm(small: bool) -> List[dict]:
    from cppmega_b200.ops import cuda as cu
    shapes = [(16384, 24960, 4096, False, False, "mamba in_proj fwd"), (16384, 4096, 8192, False, False, "mamba out_proj fwd"),
              (16384, 4096, 24960, False, True, "mamba in_proj dgrad"), (24960, 4096, 16384, True, True, "mamba in_proj wgrad"),
              (8192, 8192, 8192, False, False, "square 8192"), (4096, 131072, 4096, False, False, "lm head chunk fwd")]
    if small:
        shapes = [(2048, 2048, 2048, False, False, "square 2048")]
    out = []
    for M, N, K, a_mn, b_mn, label in shapes:
        A = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        Bm = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        o = time_ms(lambda: cu.gemm(A, Bm, a_mn=a_mn, b_mn=b_mn, out=C))
        At, Bt = (A.t() if a_mn else A), (Bm if b_mn else Bm.t())
        r = time_ms(lambda: torch.matmul(At, Bt, out=C))
        cu.check_errors()
        out.append(_rec("bf16 GEMM " + label, {"M": M, "N": N, "K": K}, o, r, None, reference="torch.matmul (cuBLASLt)",
                        ours_tflops=2.0 * M * N * K / o / 1e9, reference_tflops=2.0 * M * N * K / r / 1e9))
    return out


CASES = {"m2rnn": bench_m2rnn, "sparse_mla": bench_sparse_mla, "indexer": bench_indexer, "linear_ce": bench_linear_ce,
         "gemm": bench_gemm}


def main(argv: List[str]) -> int:
    small = "--small" in argv
    out_path = None
    names = []
    it = iter(a for a in argv if a != "--small")
    for a in it:
        if a == "--out":
            out_path = next(it)
        else:
            names.append(a)
    if not names or any(n not in CASES for n in names):
        print(f"usage: python -m cppmega_b200.tools.kernel_bench_reference {{{','.join(CASES)}}} [--small] [--out f.json]")
        return 2
    results = []
    for n in names:
        for rec in CASES[n](small):
            print(json.dumps(rec), flush=True)
            results.append(rec)
    if out_path:
        with open(out_path, "w") as f:
            json.dump(results, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
