#!/usr/bin/env python
"""Headline benchmark: NAM56R training tokens/sec at seq 4096 on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Weak scaling: micro-batch 4 x seq 4096 per GPU, expert-parallel over all N ranks
(EP = DP = N), ZeRO-1 distributed optimizer, bf16 compute, synthetic uniform tokens,
random-init weights.  Rank 0 prints one JSON line.

Two timed regions, both bracketed by barrier + synchronize, timed with CUDA events, max
over ranks:
  * ``value``: K optimizer steps on batches already resident on the device;
  * ``e2e``: K steps through ``Trainer.train_step`` fed from pinned host memory, with the
    loss read back to the host every step.
Extra keys that explain the headline (short runs, a few steps each):
  * ``like_for_like``: the same step with the SAME per-GPU memory policy at every N (every layer recomputed, nothing
    kept), so that values at different N can be divided by each other;
  * ``nccl_path`` (N >= 2): the same step with the library collectives (NCCL reduce-scatter / all-gather / all-to-all)
    instead of the peer-memory kernels (``--no-fused-collectives`` runs only that arm as the main measurement).
``--impl reference`` reports why the reference stack cannot run on this machine.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")   # 140+ GB resident: avoid fragmentation

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "NAM56R train tokens/sec/box @seq4096"
PUBLISHED_TOK_S_BOX = 74000.0      # reference bf16 record, 8xH200 (docs/production_status.md:48-53)


class ClockSampler(threading.Thread):
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        super().__init__(daemon=True)
        self.gpu_index = gpu_index
        self.samples = []
        self._stop_evt = threading.Event()

    def run(self):
        while not self._stop_evt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu_index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 8:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop_evt.wait(0.2)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=6)

    def summary(self) -> dict:
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "", 1).isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "", 1).isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for name, val in zip(names, s[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


def reference_arm(args) -> int:
    """The reference needs its Megatron-LM fork, TransformerEngine fork, mamba_ssm and TileLang
    (STACK.lock); none of them is installed or installable offline here."""
    why = None
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    sys.path.insert(0, ref_dir)
    missing = []
    for mod in ("megatron.core", "transformer_engine", "mamba_ssm", "tilelang"):
        try:
            __import__(mod)
        except Exception:
            missing.append(mod)
    if missing:
        why = ("reference training entry point needs " + ", ".join(missing) +
               " (pinned forks in STACK.lock), which are not in the image or the offline wheelhouse")
    else:
        why = "reference dependencies import, but its launcher needs a tokenised corpus and the pinned forks"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="nam56r")
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--depth", type=int, default=0, help="debug: truncate the stack (result is then not the headline config)")
    ap.add_argument("--recompute", default="auto", choices=["auto", "none", "selective", "full"])
    ap.add_argument("--keep-last", type=int, default=-1,
                    help="layers at the end of the stack whose activations are kept instead of recomputed "
                         "(-1: 6 on one GPU in the headline config, else 0)")
    ap.add_argument("--no-fused-collectives", action="store_true",
                    help="main measurement on the NCCL collectives instead of the peer-memory kernels")
    ap.add_argument("--no-extras", action="store_true", help="skip the like_for_like and nccl_path side measurements")
    ap.add_argument("--extra-steps", type=int, default=3, help="timed steps of each side measurement")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "mxfp8", "tensorwise"],
                    help="mxfp8 / tensorwise: FP8 linears and expert GEMMs (an extra measurement; the headline number is bf16)")
    ap.add_argument("--fp8-modules", nargs="*", default=[], help="restrict --precision to these module patterns (moe, mamba_proj, globs)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (with sequence parallelism); data parallel = gpus / tp")
    ap.add_argument("--ep", type=int, default=0, help="expert-parallel size (default: the data-parallel size)")
    ap.add_argument("--fp8-activations", default="off", choices=["off", "mxfp8", "tensor"],
                    help="FP8-compress the activations kept for backward (first and last layer stay bf16)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--profile-dir", default=None, help="after timing, capture one step with the torch profiler here")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from cppmega_b200.config.model import get_preset
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.parallel import state as pstate
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.parallel.state import ParallelConfig
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py: --gpus {args.gpus} needs torch.distributed.run with {args.gpus} ranks", file=sys.stderr)
            return 2
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)

    overrides = {}
    if args.depth:
        overrides["depth"] = args.depth
    if args.seq != 4096:
        overrides["seq_length"] = args.seq
    mcfg = get_preset(args.model, **overrides)
    tp = max(args.tp, 1)
    if world % tp:
        print(f"bench.py: --tp {tp} does not divide {world} GPUs", file=sys.stderr)
        return 2
    dp = world // tp
    ep = args.ep if args.ep > 0 else (dp if mcfg.moe.num_experts % dp == 0 else 1)
    pcfg = ParallelConfig(tp=tp, pp=1, ep=ep, sequence_parallel=tp > 1, distributed_optimizer=True,
                          fused_collectives=not args.no_fused_collectives)
    pc = pstate.initialize(pcfg)
    recompute = args.recompute
    if recompute == "auto":
        # one GPU holds all 16 experts and the whole optimizer state (~16 bytes/param): only
        # per-layer recomputation leaves room for activations.  With experts and optimizer
        # state sharded over >= 4 ranks the activations fit without recomputation.
        recompute = "full" if world < 4 else "selective"
    keep_last = args.keep_last
    if keep_last < 0:
        # spare memory on a single GPU (180 GB minus parameters, optimizer state and the scan stash) pays for keeping the
        # activations of the last 6 layers (161.7 GB peak with every layer recomputed, +1.8 GB per kept layer); a fixed
        # number: if the device does not have that much free the run fails instead of measuring another configuration
        keep_last = 6 if (world == 1 and recompute == "full" and not args.depth and args.seq == 4096
                          and args.micro_batch == 4 and args.precision == "bf16") else 0
    grad_dtype = "bf16" if world < 4 else "fp32"

    def make_trainer(pctx, rc, kl):
        tcfg = TrainConfig(micro_batch_size=args.micro_batch, seq_length=args.seq, dtype="bf16", recompute=rc,
                           recompute_keep_last=kl, precision_recipe=args.precision, precision_modules=tuple(args.fp8_modules),
                           fp8_activations=args.fp8_activations,
                           optimizer=OptimizerConfig(lr=1e-5, weight_decay=0.1, grad_dtype=grad_dtype), log_interval=0)
        return Trainer(mcfg, tcfg, pctx, device=device)

    trainer = make_trainer(pc, recompute, keep_last)
    n_params = sum(p.numel() for p in trainer.model.parameters())
    holder = {"trainer": trainer}

    host_batches = synthetic_batches(mcfg.vocab_size, args.micro_batch, args.seq, seed=1234, rank=pc.dp_rank)   # one stream per data-parallel rank
    dev_pool = []
    for _ in range(2):
        mb = next(host_batches)
        dev_pool.append([{k: v.to(device) for k, v in m.items()} for m in mb])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def step_device(i):
        holder["trainer"].train_step(dev_pool[i % len(dev_pool)])

    last_loss = []

    def step_e2e(i):
        res = holder["trainer"].train_step(next(host_batches))
        last_loss.append(float(res["loss"].item()))       # device -> host read of the step's result

    for i in range(args.warmup):
        step_device(i)
    torch.cuda.synchronize()
    from cppmega_b200.ops import cuda as cu
    cu.check_errors()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    F_.reset_counters()
    ms_dev = timed(step_device, args.steps)
    launches = sum(F_.launch_counts().values())
    fallbacks = F_.fallback_counts()
    e2e = None
    if not args.no_e2e:
        ms_e2e = timed(step_e2e, args.steps)
    if rank == 0:
        sampler.stop()
    cu.check_errors()

    tokens_per_step = args.micro_batch * args.seq * dp
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    fused_paths = dict(trainer.fused)

    # ---- side measurements ------------------------------------------------------------------------------------------
    def short_run(tag):
        for i in range(2):
            step_device(i)
        torch.cuda.synchronize()
        cu.check_errors()
        ms = timed(step_device, args.extra_steps) / args.extra_steps
        return {"ms_per_step": ms, "tokens_per_s": tokens_per_step / (ms / 1e3), "steps": args.extra_steps, "warmup": 2}

    like, nccl = None, None
    if args.profile_dir:
        args.no_extras = True                       # the profiled step must be the main configuration
    if not args.no_extras:
        # (1) every layer recomputed and nothing kept, at every N: the only memory policy that fits one GPU, so the one
        # under which values at different N are comparable.  Same trainer: the policy is a property of the layer loop.
        try:
            m = trainer.model
            old_policy = (m.recompute, m.recompute_keep_last)
            m.recompute, m.recompute_keep_last = "full", 0
            if old_policy == ("full", 0):           # the headline already is that configuration
                like = {"ms_per_step": ms_dev / args.steps, "tokens_per_s": value, "steps": args.steps, "warmup": args.warmup}
            else:
                like = short_run("like_for_like")
            like.update(recompute="full", recompute_keep_last=0, grad_dtype=grad_dtype,
                        note="same memory policy at every N; the gradient buffers are bf16 below 4 GPUs (fp32 does not fit one GPU) and fp32 from 4 GPUs")
            m.recompute, m.recompute_keep_last = old_policy
        except Exception as e:                                   # never lose the headline over a side measurement
            like = {"failed": f"{type(e).__name__}: {str(e)[:200]}"}
        # (2) the same step on the library collectives.  Needs its own trainer (other buffers), so the first one goes.
        if world > 1 and pcfg.fused_collectives:
            try:
                import dataclasses
                import gc
                holder["trainer"] = None
                trainer.close()
                trainer = m = None
                gc.collect()
                torch.cuda.empty_cache()
                barrier()
                # The second trainer needs the memory of the first: go on only if EVERY rank got (nearly) all of it back,
                # so that no rank can run out of memory alone and leave the others waiting in a collective.
                free_b, total_b = torch.cuda.mem_get_info()
                enough = torch.tensor([1 if free_b >= 0.9 * total_b else 0], device=device, dtype=torch.int32)
                dist.all_reduce(enough, op=dist.ReduceOp.MIN)
                if int(enough.item()) == 0:
                    nccl = {"skipped": f"only {free_b / 2**30:.0f} of {total_b / 2**30:.0f} GiB free after closing the fused trainer"}
                else:
                    pc_nccl = dataclasses.replace(pc, config=dataclasses.replace(pc.config, fused_collectives=False))
                    holder["trainer"] = make_trainer(pc_nccl, recompute, keep_last)
                    nccl = short_run("nccl_path")
                    nccl["fused_paths"] = dict(holder["trainer"].fused)
                    nccl["fused_over_nccl"] = nccl["ms_per_step"] / (ms_dev / args.steps)
            except Exception as e:
                nccl = {"failed": f"{type(e).__name__}: {str(e)[:200]}"}
    # FLOPs the GPU actually executes: a recomputed layer runs its forward twice (the scan and sparse-attention kernels
    # reuse their stashed outputs; their share is left in, so this is an upper bound by a few per cent)
    kinds = mcfg.layer_kinds()
    n_re = (len(kinds) - keep_last if recompute == "full" else
            sum(k in ("mamba3", "m2rnn") for k in kinds[:len(kinds) - keep_last]) if recompute == "selective" else 0)
    hw_factor = 1.0 + (n_re / max(len(kinds), 1)) / 3.0
    if not args.no_e2e:
        h2d = 2 * args.micro_batch * args.seq * 8             # input_ids + labels, int64, per rank
        e2e = {"value": tokens_per_step * args.steps / (ms_e2e / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": 4 * world,      # every rank copies its (TP-replicated) batch
               "ms_per_step": ms_e2e / args.steps, "last_loss": last_loss[-1] if last_loss else None}
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / PUBLISHED_TOK_S_BOX, "dtype": "bf16" if args.precision == "bf16" else f"{args.precision} fp8 linears ({' '.join(args.fp8_modules) or 'all'}), bf16 elsewhere", "data": "synthetic uniform tokens, random-init weights",
            "impl": "ours",
            "config": {"model": f"{mcfg.name} {n_params / 1e9:.2f}B params on rank 0 ({mcfg.param_count()['total'] / 1e9:.2f}B total), "
                                f"{mcfg.depth} layers {mcfg.pattern}, hidden {mcfg.hidden_size}, vocab {mcfg.vocab_size}, MTP {mcfg.mtp.num_layers}",
                       "global_batch": args.micro_batch * dp, "micro_batch": args.micro_batch, "seq_len": args.seq,
                       "parallelism": (f"tp{tp}ep{ep}dp{dp} (sequence parallel)" if tp > 1 else f"ep{ep}dp{world}") if world > 1 else "single GPU (16 local experts)",
                       "distributed_optimizer": True, "recompute": recompute, "recompute_keep_last": keep_last,
                       "grad_dtype": grad_dtype, "fp8_activations": args.fp8_activations, "collectives": "peer-memory kernels" if pcfg.fused_collectives else "nccl",
                       "l2": "weights + activations per step are far larger than the 126 MB L2",
                       "headline_config": not args.depth and args.seq == 4096 and args.micro_batch == 4 and args.precision == "bf16" and tp == 1
                                          and args.fp8_activations == "off"},
            "clocks": sampler.summary() if rank == 0 else None,
            "e2e": e2e, "gpu_launches": launches, "fallback_ops": fallbacks, "fused_paths": fused_paths,
            "like_for_like": like, "nccl_path": nccl,
            "model_tflops_per_gpu": mcfg.flops_per_token(args.seq) * value / world / 1e12,
            "hw_tflops_per_gpu": mcfg.flops_per_token(args.seq) * value / world / 1e12 * hw_factor,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
        }
        print(json.dumps(out))
    if args.profile_dir:
        # every rank runs the profiled step (it contains collectives); rank 0 keeps the tables
        from cppmega_b200.utils.profiling import profile_steps
        pdir = args.profile_dir if rank == 0 else os.path.join(args.profile_dir, f"rank{rank}")
        if holder["trainer"] is None:
            raise SystemExit("--profile-dir needs --no-extras (the side measurements replace the trainer)")
        table = profile_steps(step_device, 1, pdir)
        if rank == 0:
            print(table[:200], file=sys.stderr)
    if world > 1:
        dist.barrier()
        pstate.destroy()
    return 0


if __name__ == "__main__":
    t0 = time.time()
    sys.exit(main())
