"""Worker for the multi-GPU tests: trains the tiny model for a few steps with either the plain
NCCL collectives or the fused peer-memory kernels and prints the loss curve on rank 0."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from cppmega_b200.config.model import nam56r_tiny  # noqa: E402
from cppmega_b200.ops import cuda as cu  # noqa: E402
from cppmega_b200.ops import functional as F_  # noqa: E402
from cppmega_b200.parallel import state as pstate  # noqa: E402
from cppmega_b200.parallel.dist_optimizer import OptimizerConfig  # noqa: E402
from cppmega_b200.parallel.state import ParallelConfig  # noqa: E402
from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches  # noqa: E402


def main():
    mode, steps = sys.argv[1], int(sys.argv[2])
    recompute = sys.argv[3] if len(sys.argv) > 3 else "none"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    tp_mode = mode.startswith("tp_")
    tpdp_mode = mode.startswith("tpdp_")                # TP 2 x DP (world / 2), EP = DP
    pp_mode = mode in ("pp", "pp_vpp2", "dualpipev", "single4")
    seq = 256 if (tp_mode or tpdp_mode) else 128                      # fused TP wants (seq / tp) % 128 == 0
    schedule = {"pp_vpp2": "interleaved", "dualpipev": "dualpipev"}.get(mode, "1f1b")
    n_mb = 4 if pp_mode else world
    if tp_mode:
        pc = pstate.initialize(ParallelConfig(tp=world, sequence_parallel=True, fused_collectives=(mode == "tp_fused")))
    elif tpdp_mode:
        pc = pstate.initialize(ParallelConfig(tp=2, ep=world // 2, sequence_parallel=True,
                                              fused_collectives=(mode == "tpdp_fused")))
    elif pp_mode:
        cfgs = {"pp": ParallelConfig(pp=world), "pp_vpp2": ParallelConfig(pp=world, vpp=2), "dualpipev": ParallelConfig(pp=world),
                "single4": ParallelConfig()}
        pc = pstate.initialize(cfgs[mode])
    else:
        ep = min(world, nam56r_tiny().moe.num_experts)
        pc = pstate.initialize(ParallelConfig(ep=ep, fused_collectives=(mode == "fused")))
    mcfg = nam56r_tiny(seq_length=seq)
    from cppmega_b200.parallel import fused_moe  # noqa: E402
    fused_moe.MIN_CHUNK_COPIES = 64              # the tiny model routes 512 copies per call: still take the two-chunk pipeline
    tcfg = TrainConfig(micro_batch_size=2, global_batch_size=2 * n_mb if pp_mode else None, seq_length=seq, dtype="bf16",
                       recompute=recompute, optimizer=OptimizerConfig(lr=1e-3, weight_decay=0.0), log_interval=0,
                       pipeline_schedule=schedule)
    trainer = Trainer(mcfg, tcfg, pc, device=torch.device("cuda", local_rank))
    stream = synthetic_batches(mcfg.vocab_size, 2, seq, num_microbatches=n_mb, seed=0, pin=False, rank=0)
    F_.reset_counters()
    losses = []
    for _ in range(steps):
        mbs = next(stream)
        if pp_mode:
            res = trainer.train_step(mbs)
            has_loss = pc.is_first_pp if mode == "dualpipev" else pc.is_last_pp
            rec = (trainer.reduce_loss_for_logging(res) if has_loss
                   else {"loss": 0.0, "lm_loss": 0.0, "grad_norm": float(res["grad_norm"])})
        else:
            res = trainer.train_step([mbs[pc.dp_rank]])
            rec = trainer.reduce_loss_for_logging(res)
        losses.append([rec["loss"], rec["lm_loss"], rec["grad_norm"]])
    torch.cuda.synchronize()
    cu.check_errors()
    report = 0
    if mode in ("pp", "pp_vpp2"):
        report = world - 1
    if pc.rank == report:
        print("RESULT " + json.dumps({"mode": mode, "losses": losses, "fused": trainer.fused,
                                      "launches": F_.launch_counts()}), flush=True)
    pstate.destroy()


if __name__ == "__main__":
    main()
