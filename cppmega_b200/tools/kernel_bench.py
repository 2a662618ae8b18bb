"""Per-kernel micro-benchmarks with roofline fractions.

    python -m cppmega_b200.tools.kernel_bench [gemm] [grouped] [rmsnorm] [ce] [scan] ... [--out file.json]

Each case is timed with CUDA events after warm-up, with an L2 flush (a write larger than
the 126 MB L2) between timed iterations, and reported against the measured peaks in
``MEASURED_PEAKS.json`` at the repository root (copy bandwidth and cuBLAS bf16 throughput)
or, if that file is absent, against 6.65 TB/s and 1.59 PFLOP/s.
(Counterpart of the reference's micro-benchmarks, e.g. scripts/bench_m2rnn.py and
tools/probes/speed_harness.py.)
"""
from __future__ import annotations

import json
import os
import sys
from typing import Callable, Dict, List

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> Dict[str, float]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn: Callable, iters: int = 10, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm() -> List[dict]:
    from cppmega_b200.ops import cuda as cu
    pk = peaks()
    out = []
    shapes = [  # (M, N, K, a_mn, b_mn, label)
        (16384, 24960, 4096, False, False, "mamba in_proj fwd"),
        (16384, 4096, 8192, False, False, "mamba out_proj fwd"),
        (16384, 4096, 24960, False, True, "mamba in_proj dgrad"),
        (24960, 4096, 16384, True, True, "mamba in_proj wgrad"),
        (8192, 8192, 8192, False, False, "square 8192"),
        (4096, 131072, 4096, False, False, "lm head chunk fwd"),
    ]
    for M, N, K, a_mn, b_mn, label in shapes:
        A = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
        B = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_ms(lambda: cu.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=C))
        At = A.t() if a_mn else A
        Bt = B if b_mn else B.t()
        ms_lib = time_ms(lambda: torch.matmul(At, Bt, out=C))
        tf = 2.0 * M * N * K / ms / 1e9
        out.append({"kernel": "gemm_tcgen05", "case": label, "M": M, "N": N, "K": K, "ms": ms, "tflops": tf,
                    "frac_of_" + pk["kind"]: tf / pk["bf16_tflops"], "cublas_ms": ms_lib,
                    "cublas_tflops": 2.0 * M * N * K / ms_lib / 1e9})
        cu.check_errors()
    return out


def bench_grouped() -> List[dict]:
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import extra
    pk = peaks()
    T, k, E, H, Fh = 16384, 4, 16, 4096, 896
    ids = torch.randint(0, E, (T * k,), device="cuda")
    counts = torch.bincount(ids, minlength=E)
    x = torch.randn(T * k, H, device="cuda").bfloat16()
    w1 = (torch.randn(E, 2 * Fh, H, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(E, H, Fh, device="cuda") * 0.02).bfloat16()
    with torch.no_grad():
        ms = time_ms(lambda: extra.moe_experts(x, w1, w2, counts))
    cu.check_errors()
    flops = 2.0 * T * k * H * Fh * 3
    return [{"kernel": "moe_experts fwd (pad + grouped fc1 + swiglu + grouped fc2 + unpad)", "tokens": T, "topk": k,
             "ms": ms, "tflops": flops / ms / 1e9, "frac_of_" + pk["kind"]: flops / ms / 1e9 / pk["bf16_tflops"]}]


def bench_rmsnorm() -> List[dict]:
    from cppmega_b200.ops import cuda as cu
    pk = peaks()
    rows, H = 65536, 4096
    x = torch.randn(rows, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    with torch.no_grad():
        ms = time_ms(lambda: cu.rmsnorm(x, w, 1e-5))
    gbs = 2 * rows * H * 2 / ms / 1e6
    return [{"kernel": "rmsnorm_fwd", "rows": rows, "H": H, "ms": ms, "GB/s": gbs,
             "frac_of_" + pk["kind"]: gbs / pk["hbm_gbs"]}]


def bench_ce() -> List[dict]:
    from cppmega_b200.ops.cuda import extra
    pk = peaks()
    T, H, V = 16384, 4096, 131072
    h = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16().requires_grad_()
    lab = torch.randint(0, V, (T,), device="cuda")
    rw = torch.full((T,), 1.0 / T, device="cuda")
    ms = time_ms(lambda: extra.linear_cross_entropy_weighted(h, w, lab, rw, -100), iters=3, warmup=1)
    flops = 2.0 * T * H * V * 3
    return [{"kernel": "linear_ce fwd+bwd (3 GEMMs + softmax)", "T": T, "V": V, "ms": ms, "tflops": flops / ms / 1e9,
             "frac_of_" + pk["kind"]: flops / ms / 1e9 / pk["bf16_tflops"]}]


CASES = {"gemm": bench_gemm, "grouped": bench_grouped, "rmsnorm": bench_rmsnorm, "ce": bench_ce}


def register(name: str, fn: Callable[[], List[dict]]) -> None:
    CASES[name] = fn


def bench_glue() -> List[dict]:
    """The small fused operators against the library ops they replace, same inputs, same harness: depthwise causal
    conv1d + SiLU of the M2RNN mixer, the per-head 64 x 64 maps of the absorbed sparse-attention path (32 heads), the
    word-embedding gather / scatter-add into an fp32 gradient buffer (vocabulary 131,072); forward + backward."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops import reference as ref
    pk = peaks()
    out = []
    dev = "cuda"
    B, S = 4, 4096

    def fwd_bwd(fn, inputs, g):
        def run():
            for t in inputs:
                t.grad = None
            fn().backward(g)
        return run

    # conv1d + SiLU, read in place from a wider projection (the M2RNN mixer of the NAM56R recipe: q + k + v channels)
    from cppmega_b200.config.model import nam56r_full
    mc = nam56r_full()
    r = mc.m2rnn
    C, k = (r.num_q_heads + r.num_k_heads) * r.k_head_dim + r.heads(mc.hidden_size) * r.v_head_dim, r.conv_kernel
    proj = torch.randn(B, S, (2 * C + 63) // 8 * 8, device=dev).bfloat16()
    x = proj[..., :C].detach().requires_grad_()
    w = (torch.randn(C, 1, k, device=dev) * 0.5).bfloat16().requires_grad_()
    b = torch.zeros(C, device=dev).bfloat16().requires_grad_()
    g = torch.randn(B, S, C, device=dev).bfloat16()
    ours = time_ms(fwd_bwd(lambda: F_.causal_conv1d_silu(x, w, b), (x, w, b), g))
    lib = time_ms(fwd_bwd(lambda: ref.causal_conv1d_silu(x, w.squeeze(1), b), (x, w, b), g))
    byts = B * S * C * 2 * 7.0              # x, y, dy, g (write + k-fold cached read), dx: about seven passes
    out.append({"kernel": "causal_conv1d_silu fwd+bwd", "B": B, "S": S, "C": C, "k": k, "ms": ours, "library_ms": lib,
                "speedup": lib / ours, "frac_of_" + pk["kind"] + "_hbm": byts / ours / 1e6 / pk["hbm_gbs"]})
    # per-head maps
    H = 32
    xh = torch.randn(B, S, H, 64, device=dev).bfloat16().requires_grad_()
    wh = (torch.randn(H, 64, 64, device=dev) * 0.1).bfloat16().requires_grad_()
    gh = torch.randn(B, S, H, 64, device=dev).bfloat16()
    ours = time_ms(fwd_bwd(lambda: F_.head_linear(xh, wh), (xh, wh), gh))
    lib = time_ms(fwd_bwd(lambda: torch.einsum("bshi,hoi->bsho", xh, wh), (xh, wh), gh))
    byts = B * S * H * 64 * 2 * 6.0         # x, y | dy, dx | dy, x again for the weight gradient
    out.append({"kernel": "head_linear fwd+bwd", "tokens": B * S, "heads": H, "ms": ours, "library_ms": lib,
                "speedup": lib / ours, "frac_of_" + pk["kind"] + "_hbm": byts / ours / 1e6 / pk["hbm_gbs"]})
    # word embedding: gather + gradient rows added into the fp32 flat gradient buffer
    V, Hd = 131072, 4096
    we = torch.nn.Parameter((torch.randn(V, Hd, device=dev) * 0.02).bfloat16())
    ids = torch.randint(0, V, (B, S), device=dev)
    ge = torch.randn(B, S, Hd, device=dev).bfloat16()
    main = torch.zeros(V, Hd, device=dev, dtype=torch.float32)

    def lib_embed():
        we.grad = None
        torch.nn.functional.embedding(ids, we).backward(ge)
        main.add_(we.grad)

    def our_embed():
        we.grad = None
        F_.embedding(ids, we).backward(ge)

    lib = time_ms(lib_embed)
    we.main_grad, we.fuse_wgrad_accumulation = main, True
    ours = time_ms(our_embed)
    out.append({"kernel": "embedding fwd + bwd into the fp32 gradient buffer", "tokens": B * S, "vocab": V, "hidden": Hd, "ms": ours,
                "library_ms": lib, "speedup": lib / ours})
    cu.check_errors()
    assert not F_.fallback_counts(), F_.fallback_counts()
    return out


CASES["glue"] = bench_glue


def bench_fp8_activations() -> List[dict]:
    """Training step of the four-layer production-width slice (one Mamba3, one DSA, one MoE, one M2RNN layer; hidden 1024)
    with and without FP8 storage of the saved activations: step time and peak allocator memory."""
    from cppmega_b200.config.model import nam56r_slice
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches
    from cppmega_b200.utils import fp8_activations as fa
    out = []
    mb, seq = 4, 4096
    for mode in ("off", "mxfp8", "tensor"):
        cfg = nam56r_slice(seq_length=seq)
        tc = TrainConfig(micro_batch_size=mb, seq_length=seq, dtype="bf16", fp8_activations=mode, fp8_activations_bf16_first=0,
                         fp8_activations_bf16_last=0, log_interval=0, optimizer=OptimizerConfig(lr=1e-4, weight_decay=0.0))
        tr = Trainer(cfg, tc, device=torch.device("cuda", 0))
        stream = synthetic_batches(cfg.vocab_size, mb, seq, seed=0)
        batches = [next(stream) for _ in range(2)]
        for i in range(3):
            loss = tr.train_step(batches[i % 2])["loss"]
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        resident = torch.cuda.memory_allocated()           # parameters, optimizer state, buffers: everything but activations
        fa.reset_stats()
        ms = time_ms(lambda: tr.train_step(batches[0]), iters=5, warmup=1)
        out.append({"case": "nam56r_slice train step", "fp8_activations": mode, "ms_per_step": ms,
                    "activation_peak_gb": (torch.cuda.max_memory_allocated() - resident) / 2**30,
                    "resident_gb": resident / 2**30, "loss": float(loss),
                    "packed_tensors_per_step": fa.STATS["packed"] / 6, "saved_gb_per_step":
                    (fa.STATS["bytes_in"] - fa.STATS["bytes_out"]) / 6 / 2**30})
        tr.close()
        del tr, stream, batches
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    return out


CASES["fp8_activations"] = bench_fp8_activations


def main(argv: List[str]) -> int:
    out_path = None
    names = []
    it = iter(argv)
    for a in it:
        if a == "--out":
            out_path = next(it)
        else:
            names.append(a)
    try:
        from . import kernel_bench_extra  # noqa: F401  (registers more cases)
    except ImportError:
        pass
    names = names or list(CASES)
    results = []
    for n in names:
        for rec in CASES[n]():
            print(json.dumps(rec))
            results.append(rec)
    if out_path:
        with open(out_path, "w") as f:
            json.dump({"peaks": peaks(), "results": results}, f, indent=1)
    return 0


def bench_scan() -> List[dict]:
    """Mamba3 MIMO scan forward at the NAM56R layer shape (B4 S4096 H128 G8 N128 P64 R4)."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels3
    pk = peaks()
    B, S, H, G, N, P, R = 4, 4096, 128, 8, 128, 64, 4
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
    ms = time_ms(lambda: kernels3.mimo_fwd_raw(Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D), iters=5)
    cu.check_errors()
    chunks = B * H * (S // 32)
    flops = chunks * (2.0 * 128 * 128 * 128 + 3 * 2.0 * 128 * 64 * 128)
    return [{"kernel": "mimo_scan_fwd (local_state + state_scan + chunk_out)", "B": B, "S": S, "H": H, "ms": ms,
             "tflops": flops / ms / 1e9, "frac_of_" + pk["kind"]: flops / ms / 1e9 / pk["bf16_tflops"],
             "tokens_per_s": B * S / ms * 1e3}]


CASES["scan"] = bench_scan


def bench_scan_bar() -> List[dict]:
    """The shape at which the reference publishes TileLang-on-B200 timings of the Mamba3 MIMO kernels
    (B2 S256 H8 G1 N64 P64 R4, chunk 16, bf16: forward 54 us, backward 72 + 179 us;
    docs/modal_b200_cutile_variant_sweep_2026_04_11.md:13-18).  Here the state dimension 64 runs zero-padded on the
    128-wide kernels; the padding copies are inside the timed region."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels3
    B, S, H, G, N, P, R = 2, 256, 8, 1, 64, 64, 4
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    Q = (rn(B, S, R, G, N) * 0.5).bfloat16().requires_grad_()
    K = (rn(B, S, R, G, N) * 0.5).bfloat16().requires_grad_()
    V, Z = rn(B, S, H, P).bfloat16().requires_grad_(), rn(B, S, H, P).bfloat16().requires_grad_()
    DT = torch.rand(B, H, S, device=dev, generator=g) * 0.1
    ADT = (-DT * torch.rand(B, H, S, device=dev, generator=g)).requires_grad_()
    DT.requires_grad_()
    Trap = rn(B, H, S).requires_grad_()
    Qb, Kb = rn(H, R, N).requires_grad_(), rn(H, R, N).requires_grad_()
    Psi, Zeta, Phi = (rn(H, R, P).requires_grad_() for _ in range(3))
    ang = rn(B, S, H, N // 4).requires_grad_()
    D = rn(H).requires_grad_()
    args = (Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z)
    with torch.no_grad():
        ms_f = time_ms(lambda: kernels3.mimo_scan(*args, 4, 16), iters=20, warmup=5)
    y = kernels3.mimo_scan(*args, 4, 16)
    dy = torch.randn_like(y)
    ms_b = time_ms(lambda: torch.autograd.grad(y, args, dy, retain_graph=True), iters=20, warmup=5)
    cu.check_errors()
    row = {"kernel": "mimo_scan at the reference's published shape", "B": B, "S": S, "H": H, "G": G, "N": N, "P": P, "R": R,
           "fwd_us": ms_f * 1e3, "bwd_us": ms_b * 1e3, "reference_tilelang_b200_fwd_us": 54.0,
           "reference_tilelang_b200_bwd_us": 72.0 + 179.0,
           "note": "includes the zero-padding of the state dimension 64 -> 128 and, in backward, the head->group reductions"}
    # At this size (128 chunks) the ~30 launches of a call cost more on the host than on the device: the same calls
    # replayed from a CUDA graph, which is how the trainer runs launch-bound layers (TrainConfig.cuda_graph_scope).
    try:
        def capture(fn):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            return graph

        def fwd_only():
            with torch.no_grad():
                kernels3.mimo_scan(*args, 4, 16)

        def fwd_bwd():                      # gradients land in .grad tensors that the capture itself allocates
            for t in args:
                t.grad = None
            kernels3.mimo_scan(*args, 4, 16).backward(dy)

        del y                                   # no autograd graph from before the capture may stay alive
        g_f, g_fb = capture(fwd_only), capture(fwd_bwd)
        us_f = time_ms(g_f.replay, iters=20, warmup=5) * 1e3
        us_fb = time_ms(g_fb.replay, iters=20, warmup=5) * 1e3
        cu.check_errors()
        row.update(graph_fwd_us=us_f, graph_fwd_bwd_us=us_fb, graph_bwd_us=us_fb - us_f)
    except Exception as e:                                   # keep the eager numbers if the capture is refused
        row["graph_error"] = f"{type(e).__name__}: {str(e)[:160]}"
    return [row]


CASES["scan_bar"] = bench_scan_bar


def bench_mxfp8_gemm() -> List[dict]:
    """Block-scaled MXFP8 GEMM (operands already quantised; the swizzle of the scales is outside the timed region)."""
    import ctypes
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import mxfp8
    pk = peaks()
    out = []
    for M, N, K, label in [(16384, 24960, 4096, "mamba in_proj fwd"), (16384, 4096, 8192, "mamba out_proj fwd"),
                           (8192, 8192, 8192, "square 8192"), (24960, 4096, 16384, "mamba in_proj wgrad (TN of transposes)")]:
        a = mxfp8.quantize_rowwise(torch.randn(M, K, device="cuda").bfloat16())
        b = mxfp8.quantize_rowwise(torch.randn(N, K, device="cuda").bfloat16())
        sfa, sfb = mxfp8.swizzle_scales(a.scales), mxfp8.swizzle_scales(b.scales)
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        L, err = mxfp8._lib(), cu.err_word(C.device)

        def run():
            rc = L.cm_mxfp8_gemm(a.payload.data_ptr(), sfa.data_ptr(), b.payload.data_ptr(), sfb.data_ptr(), C.data_ptr(), M, N, K,
                                 K, K, N, 0, 0, err.data_ptr(), cu.stream_ptr())
            assert rc == 0, rc
        ms = time_ms(run)
        cu.check_errors()
        tf = 2.0 * M * N * K / ms / 1e9
        out.append({"kernel": "mxfp8_gemm_kernel", "case": label, "M": M, "N": N, "K": K, "ms": ms, "tflops": tf,
                    "x_of_" + pk["kind"] + "_bf16": tf / pk["bf16_tflops"], "frac_of_nominal_fp8_4500": tf / 4500.0})
    return out


CASES["mxfp8_gemm"] = bench_mxfp8_gemm


def bench_longctx() -> List[dict]:
    """Single-layer long-context sweep at hidden 4096, batch 1: MIMO scan fwd / bwd (128 heads) and the DSA path
    (indexer top-256 + sparse MLA fwd / bwd, 32 heads) at seq 4096 .. 32768."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels3, kernels4
    from cppmega_b200.ops.cuda.mimo_bwd import mimo_bwd
    pk = peaks()
    out = []
    dev = "cuda"
    for S in (4096, 8192, 16384, 32768):
        B, H, G, N, P, R = 1, 128, 8, 128, 64, 4
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
        args = (Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D)
        ms_f = time_ms(lambda: kernels3.mimo_fwd_raw(*args), iters=5)
        y, states, tot = kernels3.mimo_fwd_raw(*args)
        saved = [Qn.permute(0, 1, 3, 2, 4), Kn.permute(0, 1, 3, 2, 4), V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z]
        dy = torch.randn_like(y)
        ms_b = time_ms(lambda: mimo_bwd(saved, dy, states, tot), iters=5)
        cu.check_errors()
        chunks = B * H * (S // 32)
        flops = chunks * (2.0 * 128 * 128 * 128 + 3 * 2.0 * 128 * 64 * 128)
        out.append({"kernel": "mimo_scan", "S": S, "fwd_ms": ms_f, "bwd_ms": ms_b, "fwd_tflops": flops / ms_f / 1e9,
                    "fwd_frac_of_" + pk["kind"]: flops / ms_f / 1e9 / pk["bf16_tflops"], "tokens_per_s_fwd_bwd": S / (ms_f + ms_b) * 1e3})
        del y, states, tot, saved, dy, args
        qi = torch.randn(B, S, 32, 64, device=dev).bfloat16()
        ki = torch.randn(B, S, 64, device=dev).bfloat16()
        wi = torch.rand(B, S, 32, device=dev)
        ms_i = time_ms(lambda: kernels4.indexer_topk(qi, ki, wi, 256), iters=5)
        idx = kernels4.indexer_topk(qi, ki, wi, 256)
        q = (torch.randn(B, S, 32, 128, device=dev) * 0.3).bfloat16().requires_grad_()
        kv = (torch.randn(B, S, 128, device=dev) * 0.3).bfloat16().requires_grad_()
        ms_sf = time_ms(lambda: kernels4.sparse_mla_fwd_raw(q.detach(), kv.detach(), idx, 128 ** -0.5, 64), iters=5)
        o = kernels4.SparseMLAFn.apply(q, kv, idx, 128 ** -0.5, 64)
        g = torch.randn_like(o)
        ms_sb = time_ms(lambda: torch.autograd.grad(o, (q, kv), g, retain_graph=True), iters=5)
        cu.check_errors()
        idx_flops = 2.0 * B * S * (S / 2) * 32 * 64
        smla_flops = 2.0 * B * S * 32 * 256 * (128 + 64)
        out.append({"kernel": "dsa", "S": S, "indexer_topk_ms": ms_i, "indexer_tflops": idx_flops / ms_i / 1e9,
                    "sparse_mla_fwd_ms": ms_sf, "sparse_mla_fwd_tflops": smla_flops / ms_sf / 1e9, "sparse_mla_bwd_ms": ms_sb,
                    "indexer_frac_of_" + pk["kind"]: idx_flops / ms_i / 1e9 / pk["bf16_tflops"]})
        del qi, ki, wi, idx, q, kv, o, g
        torch.cuda.empty_cache()
    return out


CASES["longctx"] = bench_longctx


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
