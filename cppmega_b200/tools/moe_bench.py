"""Isolated MoE-layer benchmark: fused dispatch -> grouped GEMM -> combine, forward + backward, against the NCCL path.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \\
        -m cppmega_b200.tools.moe_bench [--tokens 16384] [--skew zipf] [--precision mxfp8] [--iters 10]

One MoE layer of the NAM56R recipe (hidden 4096, 16 experts top-4 + shared expert, SwiGLU expert FFN 896), EP = N,
16384 tokens per rank.  The router weight is replaced by fixed logits: N(0,1) (near-uniform load) or N(0,1) + log of a
Zipf(1.2) popularity (``--skew zipf``).  Timed on the device with CUDA events, max over ranks:

* ``fused``  peer-memory dispatch / combine kernels around the grouped tcgen05 GEMMs (``parallel/fused_moe.py``), two token
             chunks pipelined over two streams (``fused_one_chunk_ms``: the same without the pipeline);
* ``nccl``   the same layer through ``AllToAllDispatcher`` (NCCL all-to-all + permute) and the same grouped GEMMs.

The roofline is the slower of the expert + shared GEMM FLOPs at the measured bf16 peak and the bytes that must cross
NVLink (4 transfers of tokens x top-k x hidden x 2 bytes x (N-1)/N per direction for forward + backward) at the
measured 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


class _OneLayer(torch.nn.Module):
    def __init__(self, cfg, layer):
        super().__init__()
        self.cfg, self.layer = cfg, layer

    def moe_layers(self):
        return [self.layer]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--skew", default="none", choices=["none", "zipf"])
    ap.add_argument("--precision", default="bf16", choices=["bf16", "mxfp8"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--capacity-factor", type=float, default=None)
    ap.add_argument("--sweep-transport", action="store_true", help="also time the pipelined path with 8 / 4 / 2 / 1 transport blocks per SM")
    ap.add_argument("--no-overlap-shared", action="store_true", help="keep the shared expert on the main stream (default: second stream beside the routed path)")
    ns = ap.parse_args(argv)
    from cppmega_b200.config.model import nam56r_full
    from cppmega_b200.models.moe import MoELayer
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.parallel import fused_moe
    from cppmega_b200.parallel import state as pstate
    from cppmega_b200.parallel.state import ParallelConfig
    from cppmega_b200.tools.kernel_bench import peaks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pc = pstate.initialize(ParallelConfig(ep=world))
    import dataclasses
    mcfg = nam56r_full()
    mcfg = dataclasses.replace(mcfg, moe=dataclasses.replace(mcfg.moe, aux_loss_coeff=0.0))      # the layer alone, no auxiliary loss
    H, E, topk = mcfg.hidden_size, mcfg.moe.num_experts, mcfg.moe.topk
    F_.set_precision_recipe(ns.precision)
    layer = MoELayer(H, mcfg.moe, pc, "bench.layer", init_std=0.02, out_std=0.02, dtype=torch.bfloat16, seed=1).to(dev)
    T = ns.tokens
    gen = torch.Generator(device="cpu").manual_seed(1234 + pc.rank)
    x = (torch.randn(1, T, H, generator=gen) * 0.5).bfloat16().to(dev).requires_grad_()
    logits = torch.randn(T, E, generator=gen)
    if ns.skew == "zipf":
        logits = logits + torch.log(1.0 / torch.arange(1, E + 1).float() ** 1.2)[None, :] * 2.0
    logits = logits.to(dev)

    class FixedRouter(torch.nn.Module):
        def forward(self, flat):
            probs, ids, scores = F_.router_topk(logits, topk, mcfg.moe.score_function, None, mcfg.moe.norm_topk_prob)
            return probs.to(flat.dtype), ids, scores

    layer.router = FixedRouter()
    overlap_shared = not ns.no_overlap_shared
    ids = layer.router(x.reshape(T, H))[1]
    load = torch.bincount(ids.reshape(-1), minlength=E).float()
    per_rank = load.view(world, -1).sum(1)
    worst = float(per_rank.max() / per_rank.mean()) if world > 1 else 1.0
    dist_worst = torch.tensor([worst], device=dev)
    if world > 1:
        dist.all_reduce(dist_worst, op=dist.ReduceOp.MAX)
    cap = ns.capacity_factor or max(2.0, float(dist_worst) * 1.25)
    g = torch.randn(1, T, H, device=dev, dtype=torch.bfloat16)

    def run():
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        layer(x).backward(g)

    def timed():
        for _ in range(ns.warmup):
            run()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(ns.iters):
            run()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / ns.iters], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        cu.check_errors()
        return float(t)

    res = {"tokens_per_rank": T, "ep": world, "skew": ns.skew, "precision": ns.precision, "overlap_shared": overlap_shared,
           "max_rank_load_over_mean": float(dist_worst), "capacity_factor": cap}
    layer.fused_dispatcher = None
    res["nccl_ms"] = timed() if world > 1 else None
    bufs = fused_moe.attach(_OneLayer(mcfg, layer), pc, dev, tokens_per_rank=T, capacity_factor=cap, overlap_shared_expert=overlap_shared)
    res["fused_ms"] = timed() if bufs is not None else None
    if bufs is not None and world > 1:
        res["chunks"] = bufs.chunks_for(T, topk)
        res["transport_blocks_per_sm"] = fused_moe.set_transport_blocks_per_sm(8)
        fused_moe.set_transport_blocks_per_sm(res["transport_blocks_per_sm"])
        if ns.sweep_transport:
            res["fused_ms_by_transport_blocks_per_sm"] = {}
            for n in (8, 4, 2, 1):
                fused_moe.set_transport_blocks_per_sm(n)
                res["fused_ms_by_transport_blocks_per_sm"][str(n)] = timed()
            fused_moe.set_transport_blocks_per_sm(res["transport_blocks_per_sm"])
        bufs.chunks = 1                                   # the same kernels without the two-chunk / two-stream pipeline
        fused_moe.set_transport_blocks_per_sm(8)
        res["fused_one_chunk_ms"] = timed()
    Fe, Fs = mcfg.moe.expert_ffn, mcfg.moe.shared_expert_ffn
    flops = 3 * 2.0 * T * (topk * 3 * H * Fe + 3 * H * Fs)                 # fwd + dgrad + wgrad, SwiGLU = 3 matrices
    pk = peaks()
    t_compute = flops / (pk["bf16_tflops"] * 1e9)
    t_link = 4 * T * topk * H * 2.0 * (world - 1) / world / 770e6 if world > 1 else 0.0
    res["roofline_ms"] = max(t_compute, t_link)
    res["roofline_bound"] = "nvlink" if t_link > t_compute else "tensor"
    if res["fused_ms"]:
        res["fused_frac_of_roofline"] = res["roofline_ms"] / res["fused_ms"]
        if res["nccl_ms"]:
            res["fused_over_nccl"] = res["nccl_ms"] / res["fused_ms"]
    if pc.rank == 0:
        print(json.dumps(res))
    pstate.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
