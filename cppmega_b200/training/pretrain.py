"""Pre-training entry point.

    python -m cppmega_b200.training.pretrain <Megatron-style args>
    python -m torch.distributed.run --nproc-per-node 8 -m cppmega_b200.training.pretrain <args>

One process per GPU.  Counterpart of the reference's wrapped ``pretrain_mamba.py`` launch
(scripts/remote_smoke_h200_dsa_9_4_m.sh:467-478,691-740): parse arguments, build groups / model / optimizer, resume
from ``--load``, train for ``--train-iters`` with logging of loss, grad-norm, tokens/s and model TFLOP/s/GPU
(``--log-throughput``), save every ``--save-interval``.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Dict, Iterator, List, Optional, Sequence

import torch

from ..checkpoint import sharded
from ..parallel import state as pstate
from ..utils.memory_debug import peak_memory_report
from ..utils.monitor import MetricsServer
from ..utils.profiling import cuda_profiler_window, install_layer_nvtx
from ..utils.watchdog import StepWatchdog
from .arguments import parse_args
from .trainer import Trainer, synthetic_batches


def _data_iterator(extras: Dict, mcfg, tcfg, pc, num_microbatches: int,
                   consumed_steps: int = 0) -> Iterator[List[Dict[str, torch.Tensor]]]:
    """Batches for this data-parallel rank.  ``consumed_steps`` optimizer steps of data were used by the run being
    resumed: the stream starts after them, so a resumed run sees the samples the uninterrupted run would have seen
    (Megatron keeps ``consumed_train_samples`` for the same purpose)."""
    if extras["data_path"] and not extras["mock_data"]:
        from ..data.indexed import TokenStream
        stream = TokenStream(extras["data_path"], tcfg.seq_length, tcfg.micro_batch_size, rank=pc.dp_rank, world=pc.dp,
                             seed=tcfg.seed)
        stream.skip(consumed_steps * num_microbatches)

        def gen():
            while True:
                yield [next(stream) for _ in range(num_microbatches)]
        return gen()
    if not extras["mock_data"]:
        raise SystemExit("no --data-path given: pass --mock-data to train on synthetic uniform tokens "
                         "(throughput measured that way is not a real-data number)")
    return synthetic_batches(mcfg.vocab_size, tcfg.micro_batch_size, tcfg.seq_length, num_microbatches,
                             seed=tcfg.seed, rank=pc.dp_rank, skip=consumed_steps)


def _rng_state() -> Dict:
    st = {"torch_cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["torch_cuda"] = torch.cuda.get_rng_state()
    return st


def _restore_rng(st: Optional[Dict]) -> None:
    if not st:
        return
    if "torch_cpu" in st:
        torch.set_rng_state(st["torch_cpu"].cpu().to(torch.uint8))
    if "torch_cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["torch_cuda"].cpu().to(torch.uint8))


def main(argv: Optional[Sequence[str]] = None) -> int:
    mcfg, pcfg, tcfg, extras = parse_args(argv)
    pc = pstate.initialize(pcfg)
    device = (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    trainer = Trainer(mcfg, tcfg, pc, device=device)
    log = (lambda rec: print(json.dumps(rec), flush=True)) if pc.rank == 0 else (lambda rec: None)
    if pc.rank == 0:
        counts = mcfg.param_count()
        print(f"[cppmega_b200] {mcfg.name}: {counts['total'] / 1e9:.2f}B params ({counts['active'] / 1e9:.2f}B active), "
              f"pattern {mcfg.plan().full_pattern[:64]}..., world {pc.world_size} ({pcfg.describe(pc.world_size)}), "
              f"paths {trainer.describe_paths()}", flush=True)
    start_iter = 0
    consumed_steps = 0
    if extras["load"]:
        it = sharded.latest_iteration(extras["load"])
        if it is not None:
            info = sharded.load_checkpoint(extras["load"], trainer.model, pc, trainer.optimizer,
                                           allow_optimizer_reset=extras.get("no_load_optim", False))
            start_iter = info["iteration"]
            trainer.step = start_iter
            trainer.tokens_seen = info["extra"].get("tokens_seen", 0)
            consumed_steps = info["extra"].get("consumed_steps", start_iter)
            _restore_rng(info.get("rank_extra", {}).get("rng"))
            if info.get("optimizer_reset") and pc.rank == 0:
                print("[cppmega_b200] WARNING: " + info["optimizer_reset"], flush=True)
    if extras["profile"]:
        install_layer_nvtx(trainer.model)
    server = MetricsServer(extras["monitor_port"]).start() if (extras["monitor_port"] and pc.rank == 0) else None
    if extras["step_timeout_s"] > 0:
        trainer.watchdog = StepWatchdog(extras["step_timeout_s"], rank=pc.rank).start()
    batches = _data_iterator(extras, mcfg, tcfg, pc, trainer.num_microbatches, consumed_steps)
    flops_tok = mcfg.flops_per_token(tcfg.seq_length)
    t_last = time.perf_counter()
    try:
        for it in range(start_iter, extras["train_iters"]):
            prof = extras["profile"] and extras["profile_step_start"] <= it < extras["profile_step_end"]
            with cuda_profiler_window(prof):
                res = trainer.train_step(next(batches))
            if tcfg.log_interval and (it + 1) % tcfg.log_interval == 0:
                rec = trainer.reduce_loss_for_logging(res)
                if device.type == "cuda":
                    from ..ops import cuda as cu
                    cu.check_errors(device)
                now = time.perf_counter()
                dt = (now - t_last) / tcfg.log_interval
                t_last = now
                toks = trainer.global_batch_size * tcfg.seq_length
                rec.update(iteration=it + 1, lr=res["lr"], elapsed_ms=dt * 1e3, tokens_per_s=toks / dt)
                if extras["log_throughput"]:
                    rec["tflops_per_gpu"] = flops_tok * toks / dt / 1e12 / pc.world_size
                log(rec)
                if server is not None:
                    server.publish(rec)
            if extras["save"] and extras["save_interval"] and (it + 1) % extras["save_interval"] == 0:
                if device.type == "cuda":
                    from ..ops import cuda as cu
                    cu.check_errors(device)       # a step whose kernels gave up must not be written out as a good state
                sharded.save_checkpoint(extras["save"], it + 1, trainer.model, pc, trainer.optimizer,
                                        extra={"tokens_seen": trainer.tokens_seen, "consumed_steps": it + 1},
                                        rank_extra={"rng": _rng_state()})
            if (extras.get("inject_failure_at_iteration") and it + 1 == extras["inject_failure_at_iteration"]
                    and start_iter == 0 and pc.rank == pc.world_size - 1):
                raise RuntimeError(f"injected failure on rank {pc.rank} after iteration {it + 1}")     # host-side fault injection
    finally:
        if trainer.watchdog is not None:
            trainer.watchdog.stop()
        if server is not None:
            server.stop()
    if pc.rank == 0:
        print(peak_memory_report(), flush=True)
    pstate.destroy()
    return 0


if __name__ == "__main__":
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    sys.exit(main())
