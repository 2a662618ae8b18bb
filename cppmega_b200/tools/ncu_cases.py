"""Small, self-terminating workloads for Nsight Compute captures of single kernels.

    python -m cppmega_b200.tools.ncu_cases {gemm,gemm_wgrad,attention,head_linear,scan_fwd,scan_bwd,m2rnn,m2rnn_bwd,sparse_mla,indexer,ce,rmsnorm,rmsnorm_bwd,adamw,quantize,strided_copy,moe_local,mxfp8_gemm}

Each case launches its kernel three times on inputs that exceed the 126 MB L2 but hold at most a few GB, so a
``--set full`` capture of one launch finishes in a minute or two:

    ncu --set full --clock-control none -k regex:<kernel> -s 1 -c 1 -o out python -m cppmega_b200.tools.ncu_cases <case>
"""
from __future__ import annotations

import sys

import torch


def case_gemm(a_mn=False, b_mn=False):
    from cppmega_b200.ops import cuda as cu
    M = N = K = 8192
    A = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    B = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        cu.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=C)
    torch.cuda.synchronize()
    cu.check_errors()


def case_mxfp8_gemm():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import mxfp8
    M = N = K = 8192
    a = mxfp8.quantize_rowwise(torch.randn(M, K, device="cuda").bfloat16())
    b = mxfp8.quantize_rowwise(torch.randn(N, K, device="cuda").bfloat16())
    for _ in range(3):
        mxfp8.gemm_mxfp8(a, b)
    torch.cuda.synchronize()
    cu.check_errors()


def _scan_inputs(B=1, S=4096, H=32, G=2, N=128, P=64, R=4):
    dev = "cuda"
    Qn = (torch.randn(B, S, G, R, N, device=dev) * 0.5).bfloat16()
    Kn = (torch.randn(B, S, G, R, N, device=dev) * 0.5).bfloat16()
    V = torch.randn(B, S, H, P, device=dev).bfloat16()
    Z = torch.randn(B, S, H, P, device=dev).bfloat16()
    DT = torch.rand(B, H, S, device=dev) * 0.1
    ADT = -DT * torch.rand(B, H, S, device=dev)
    Trap = torch.randn(B, H, S, device=dev)
    Qb, Kb = torch.randn(H, R, N, device=dev), torch.randn(H, R, N, device=dev)
    Psi, Zeta, Phi = (torch.randn(H, R, P, device=dev) for _ in range(3))
    ang = torch.randn(B, S, H, N // 4, device=dev)
    D = torch.randn(H, device=dev)
    return Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D


def case_scan_fwd():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels3
    args = _scan_inputs()
    for _ in range(3):
        kernels3.mimo_fwd_raw(*args)
    torch.cuda.synchronize()
    cu.check_errors()


def case_scan_bwd():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels3
    from cppmega_b200.ops.cuda.mimo_bwd import mimo_bwd
    Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _scan_inputs()
    y, states, tot = kernels3.mimo_fwd_raw(Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D)
    saved = [Qn.permute(0, 1, 3, 2, 4), Kn.permute(0, 1, 3, 2, 4), V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z]
    dy = torch.randn_like(y)
    for _ in range(3):
        mimo_bwd(saved, dy, states, tot)
    torch.cuda.synchronize()
    cu.check_errors()


def case_m2rnn():
    from cppmega_b200.ops.cuda import kernels2
    B, S, H = 4, 4096, 51
    q = torch.randn(B, S, 1, 64, device="cuda").bfloat16()
    k = torch.randn(B, S, 1, 64, device="cuda").bfloat16()
    v = torch.randn(B, S, H, 16, device="cuda").bfloat16()
    W = torch.eye(16, device="cuda").repeat(H, 1, 1).bfloat16()
    f = torch.rand(B, S, H, device="cuda")
    with torch.no_grad():
        for _ in range(3):
            kernels2.m2rnn_scan(q, k, v, W, f)
    torch.cuda.synchronize()


def case_m2rnn_bwd():
    from cppmega_b200.ops.cuda import kernels2
    B, S, H = 2, 4096, 51
    q = torch.randn(B, S, 1, 64, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(B, S, 1, 64, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(B, S, H, 16, device="cuda").bfloat16().requires_grad_()
    W = torch.eye(16, device="cuda").repeat(H, 1, 1).bfloat16().requires_grad_()
    f = torch.rand(B, S, H, device="cuda").requires_grad_()
    for _ in range(3):
        y = kernels2.m2rnn_scan(q, k, v, W, f)
        y = y[0] if isinstance(y, tuple) else y
        y.backward(torch.ones_like(y))
    torch.cuda.synchronize()


def _sparse_inputs(B=2, S=4096):
    q = (torch.randn(B, S, 32, 128, device="cuda") * 0.3).bfloat16()
    kv = (torch.randn(B, S, 128, device="cuda") * 0.3).bfloat16()
    t = torch.arange(S, device="cuda")
    idx = (torch.rand(B, S, 256, device="cuda") * (t[None, :, None] + 1)).long().clamp_max(S - 1).int()
    return q, kv, idx


def case_sparse_mla():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels4
    q, kv, idx = _sparse_inputs()
    q.requires_grad_()
    kv.requires_grad_()
    for _ in range(3):
        out = kernels4.SparseMLAFn.apply(q, kv, idx, 128 ** -0.5, 64)
        out.backward(torch.ones_like(out))
    torch.cuda.synchronize()
    cu.check_errors()


def case_indexer():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels4
    B, S = 2, 4096
    q = torch.randn(B, S, 32, 64, device="cuda").bfloat16()
    k = torch.randn(B, S, 64, device="cuda").bfloat16()
    w = torch.rand(B, S, 32, device="cuda")
    for _ in range(3):
        kernels4.indexer_topk(q, k, w, 256)
    torch.cuda.synchronize()
    cu.check_errors()


def case_ce():
    from cppmega_b200.ops.cuda import extra
    T, H, V = 4096, 4096, 131072
    h = torch.randn(T, H, device="cuda").bfloat16()
    w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16()
    lab = torch.randint(0, V, (T,), device="cuda")
    rw = torch.full((T,), 1.0 / T, device="cuda")
    for _ in range(2):
        extra.linear_cross_entropy_weighted(h, w, lab, rw, -100)
    torch.cuda.synchronize()


def case_rmsnorm():
    from cppmega_b200.ops import cuda as cu
    x = torch.randn(65536, 4096, device="cuda").bfloat16()
    w = torch.ones(4096, device="cuda").bfloat16()
    with torch.no_grad():
        for _ in range(3):
            cu.rmsnorm(x, w, 1e-5)
    torch.cuda.synchronize()


def case_rmsnorm_bwd():
    from cppmega_b200.ops import cuda as cu
    x = torch.randn(65536, 4096, device="cuda").bfloat16().requires_grad_()
    w = torch.ones(4096, device="cuda").bfloat16().requires_grad_()
    g = torch.randn(65536, 4096, device="cuda").bfloat16()
    for _ in range(3):
        cu.rmsnorm(x, w, 1e-5).backward(g)
    torch.cuda.synchronize()


def case_adamw():
    from cppmega_b200.ops import cuda as cu
    n = 256 * 1024 * 1024
    master, m, v = (torch.randn(n, device="cuda") * 0.01 for _ in range(3))
    v.abs_()
    g = torch.randn(n, device="cuda").bfloat16()
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    wd = torch.ones(n, device="cuda", dtype=torch.bool)
    clip = torch.tensor(1.0, device="cuda")
    for _ in range(3):
        cu.adamw_shard(master, m, v, g, out, wd, clip, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05)
    torch.cuda.synchronize()


def case_quantize():
    from cppmega_b200.ops.cuda import mxfp8
    x = torch.randn(16384, 24960, device="cuda").bfloat16()
    for _ in range(3):
        mxfp8.quantize_both(x)
    torch.cuda.synchronize()


def case_strided_copy():
    from cppmega_b200.ops.cuda import fast_contiguous
    packed = torch.randn(4, 4096, 24960, device="cuda").bfloat16()
    view = packed[..., 8192:16384]
    for _ in range(3):
        fast_contiguous(view)
    torch.cuda.synchronize()


def case_moe_local():
    """One MoE layer of the NAM56R recipe on one GPU (16 local experts): the permute-fused push / pull kernels and the
    grouped GEMMs, forward + backward."""
    import dataclasses
    from cppmega_b200.config.model import nam56r_full
    from cppmega_b200.models.moe import MoELayer
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.parallel import fused_moe
    from cppmega_b200.parallel import state as pstate
    from cppmega_b200.parallel.state import ParallelConfig
    pc = pstate.initialize(ParallelConfig())
    mcfg = nam56r_full()
    mcfg = dataclasses.replace(mcfg, moe=dataclasses.replace(mcfg.moe, aux_loss_coeff=0.0))
    dev = torch.device("cuda", 0)
    layer = MoELayer(mcfg.hidden_size, mcfg.moe, pc, "case.layer", dtype=torch.bfloat16, seed=1).to(dev)

    class _M(torch.nn.Module):
        cfg = mcfg

        def moe_layers(self):
            return [layer]

    fused_moe.attach(_M(), pc, dev, tokens_per_rank=0)
    x = (torch.randn(4, 4096, mcfg.hidden_size, device=dev) * 0.5).bfloat16().requires_grad_()
    g = torch.randn_like(x)
    for _ in range(3):
        layer(x).backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    pstate.destroy()


def case_attention():
    """Dense causal MLA attention (qk 128, v 64) at the model's shape: batch 4, seq 4096, 32 heads; forward + backward."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    B, S, H = 4, 4096, 32
    q = (torch.randn(B, S, H, 128, device="cuda") * 0.5).bfloat16().requires_grad_()
    k = (torch.randn(B, S, H, 128, device="cuda") * 0.5).bfloat16().requires_grad_()
    v = torch.randn(B, S, H, 64, device="cuda").bfloat16().requires_grad_()
    g = torch.randn(B, S, H, 64, device="cuda").bfloat16()
    for _ in range(3):
        F_.causal_attention(q, k, v, 128 ** -0.5).backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    assert not F_.fallback_counts(), F_.fallback_counts()


def case_head_linear():
    """Per-head 64 x 64 maps of the absorbed sparse-attention path: 16,384 tokens x 32 heads, forward + backward."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    x = torch.randn(4, 4096, 32, 64, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(32, 64, 64, device="cuda") * 0.1).bfloat16().requires_grad_()
    g = torch.randn_like(x)
    for _ in range(3):
        F_.head_linear(x, w).backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    assert not F_.fallback_counts(), F_.fallback_counts()


CASES = {"gemm": case_gemm, "attention": case_attention, "head_linear": case_head_linear, "gemm_wgrad": lambda: case_gemm(True, True), "scan_fwd": case_scan_fwd,
         "scan_bwd": case_scan_bwd, "m2rnn": case_m2rnn, "ce": case_ce, "rmsnorm": case_rmsnorm, "mxfp8_gemm": case_mxfp8_gemm,
         "m2rnn_bwd": case_m2rnn_bwd, "sparse_mla": case_sparse_mla, "indexer": case_indexer,
         "rmsnorm_bwd": case_rmsnorm_bwd, "adamw": case_adamw, "quantize": case_quantize, "strided_copy": case_strided_copy, "moe_local": case_moe_local}

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else ""
    if name not in CASES:
        raise SystemExit(f"usage: python -m cppmega_b200.tools.ncu_cases {{{','.join(CASES)}}}")
    CASES[name]()
    print(f"{name}: done")
