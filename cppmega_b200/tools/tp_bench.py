"""Isolated tensor-parallel linear benchmark: all-gather -> GEMM and GEMM -> reduce-scatter, fused vs NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \\
        -m cppmega_b200.tools.tp_bench [--batch 4] [--seq 4096] [--iters 10]

TP = N with sequence parallelism, the projection shapes of one NAM56R layer (hidden 4096): the Mamba3 in-projection
(column parallel, all-gather -> GEMM) and out-projection (row parallel, GEMM -> reduce-scatter), and two projections
of the MLA width (hidden -> heads x (qk + v), heads x v -> hidden).  Three implementations of each, timed on the device with CUDA events, max over ranks, with
an L2 flush between iterations:

* ``staged``  every shard is pushed once into the consumers' memory by a copy kernel on a second stream (one flag per
              source) while the tcgen05 GEMM of the local shard runs; remote shards are multiplied as their flags
              arrive.  GEMM -> reduce-scatter: one GEMM per destination shard whose epilogue stores into the owner's
              staging slot, then a flag barrier and one summation pass (``parallel/fused_tp.py``);
* ``direct``  one GEMM whose TMA producer reads every row block of the gathered operand from the peer that holds it;
* ``nccl``    ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` around the same tcgen05 GEMM.

The roofline per operation is the slower of its FLOPs at the measured bf16 GEMM peak and the bytes that must cross
NVLink per GPU and direction ((N-1)/N of the gathered or scattered activation) at the measured 770 GB/s.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _shapes():
    """(name, kind, K, N): full (unsharded) weight shapes of the TP linears of the NAM56R layers."""
    from cppmega_b200.config.model import nam56r_full
    c = nam56r_full()
    h = c.hidden_size
    return [
        ("mamba_in_proj", "ag_gemm", h, sum(c.mamba3.in_proj_sizes(h, 1))),
        ("mamba_out_proj", "gemm_rs", c.mamba3.d_inner(h), h),
        ("mla_kv_up", "ag_gemm", h, c.mla.num_heads * (c.mla.qk_head_dim + c.mla.v_head_dim)),
        ("mla_out_proj", "gemm_rs", c.mla.num_heads * c.mla.v_head_dim, h),
    ]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true", help="compare the three implementations' results once")
    ns = ap.parse_args(argv)
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.parallel import state as pstate
    from cppmega_b200.parallel.fused_tp import FusedTP
    from cppmega_b200.parallel.state import ParallelConfig
    from cppmega_b200.tools.kernel_bench import peaks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        print(json.dumps({"tool": "tp_bench", "unavailable": "needs 2 or more ranks"}))
        return 0
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pc = pstate.initialize(ParallelConfig(tp=world, sequence_parallel=True))
    rank = dist.get_rank()
    B, S = ns.batch, ns.seq
    Sl = S // world
    shapes = _shapes()
    width = max(k if kind == "ag_gemm" else n for _, kind, k, n in shapes)
    tp = FusedTP(pc, dev, B * Sl, width)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    pk = peaks()
    torch.manual_seed(1234 + rank)
    results = []

    def timed(fn):
        for _ in range(ns.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ms = []
        for _ in range(ns.iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        ms.sort()
        t = torch.tensor([ms[len(ms) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        cu.check_errors(dev)
        return float(t.item())

    for name, kind, K, N in shapes:
        if kind == "ag_gemm":
            Nl = N // world // 8 * 8
            x = torch.randn(B, Sl, K, device=dev, dtype=torch.bfloat16)
            w = torch.randn(Nl, K, device=dev, dtype=torch.bfloat16) * 0.02
            gathered = torch.empty(world, B, Sl, K, device=dev, dtype=torch.bfloat16)

            def nccl():
                dist.all_gather_into_tensor(gathered, x, group=pc.tp_group)
                out = torch.empty(B, S, Nl, device=dev, dtype=torch.bfloat16)
                for p in range(world):
                    for b in range(B):
                        cu.gemm(gathered[p, b], w, out=out[b, p * Sl:(p + 1) * Sl])
                return out

            def fused():
                return tp.ag_gemm(x, w, b_mn=False)

            flops = 2.0 * B * S * K * Nl
            link_bytes = (world - 1) * B * Sl * K * 2
        else:
            Kl = K // world // 8 * 8
            x = torch.randn(B, S, Kl, device=dev, dtype=torch.bfloat16)
            w = torch.randn(N, Kl, device=dev, dtype=torch.bfloat16) * 0.02

            def nccl():
                full = cu.gemm(x.view(B * S, Kl), w).view(B, world, Sl, N).transpose(0, 1).contiguous()
                out = torch.empty(B, Sl, N, device=dev, dtype=torch.bfloat16)
                dist.reduce_scatter_tensor(out, full, group=pc.tp_group)
                return out

            def fused():
                return tp.gemm_rs(x, w, b_mn=False)

            flops = 2.0 * B * S * Kl * N
            link_bytes = (world - 1) * B * Sl * N * 2
        row = {"name": name, "kind": kind, "tp": world, "tokens": B * S, "K": K, "N": N}
        if ns.check:
            ref = nccl().float()
            for mode in ("staged", "direct"):
                tp.mode = mode
                got = fused().float()
                err = (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
                row[f"{mode}_rel_err"] = err
        row["nccl_ms"] = timed(nccl)
        for mode in ("staged", "direct"):
            tp.mode = mode
            row[f"{mode}_ms"] = timed(fused)
        t_roof = max(flops / (pk["bf16_tflops"] * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        row["roofline_ms"] = t_roof
        row["bound"] = "gemm" if flops / (pk["bf16_tflops"] * 1e12) >= link_bytes / (NVLINK_GBS * 1e9) else "nvlink"
        for mode in ("staged", "direct", "nccl"):
            row[f"{mode}_frac_of_roofline"] = t_roof / row[f"{mode}_ms"]
        results.append(row)
    if rank == 0:
        print(json.dumps({"tool": "tp_bench", "results": results, "peaks": pk, "nvlink_gbs": NVLINK_GBS}))
    tp.heap.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
