"""Worker launched by the multi-process CPU tests (gloo).  Prints one JSON line on rank 0."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from cppmega_b200.config.model import nam56r_tiny  # noqa: E402
from cppmega_b200.parallel import state as pstate  # noqa: E402
from cppmega_b200.parallel.dist_optimizer import OptimizerConfig  # noqa: E402
from cppmega_b200.parallel.state import ParallelConfig  # noqa: E402
from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches  # noqa: E402


def main():
    mode = sys.argv[1]
    steps = int(sys.argv[2])
    torch.manual_seed(0)
    torch.set_num_threads(2)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfgs = {
        "ep": ParallelConfig(ep=world), "dp": ParallelConfig(), "tp": ParallelConfig(tp=world),
        "tp_sp": ParallelConfig(tp=world, sequence_parallel=True),
        "pp": ParallelConfig(pp=world), "ep_nodistopt": ParallelConfig(ep=world, distributed_optimizer=False),
        "pp_vpp2": ParallelConfig(pp=world, vpp=2), "dualpipev": ParallelConfig(pp=world),
        "dp_muon": ParallelConfig(), "ep_muon": ParallelConfig(ep=world),
    }
    schedule = {"pp_vpp2": "interleaved", "dualpipev": "dualpipev"}.get(mode, "1f1b")
    n_mb = 4 if schedule != "1f1b" else 2
    pc = pstate.initialize(cfgs[mode], backend="gloo")
    mcfg = nam56r_tiny(seq_length=64)
    seq, mb = 64, 2
    dp = pc.dp
    if len(sys.argv) > 3:
        n_mb = int(sys.argv[3])
    tcfg = TrainConfig(micro_batch_size=mb, global_batch_size=n_mb * mb, seq_length=seq, dtype="fp32",
                       optimizer=(OptimizerConfig(optimizer="muon", lr=1e-3, weight_decay=0.01, bucket_mb=1)
                                  if mode.endswith("_muon") else OptimizerConfig(lr=1e-3, weight_decay=0.0)),
                       log_interval=0, pipeline_schedule=schedule)
    trainer = Trainer(mcfg, tcfg, pc, device=torch.device("cpu"))
    # the global batch is always the same 2 micro-batches; each DP rank takes its slice
    stream = synthetic_batches(mcfg.vocab_size, mb, seq, num_microbatches=n_mb, seed=0, pin=False, rank=0)
    losses = []
    for _ in range(steps):
        global_mbs = next(stream)
        per_rank = len(global_mbs) // dp
        mine = global_mbs[pc.dp_rank * per_rank:(pc.dp_rank + 1) * per_rank]
        res = trainer.train_step(mine)
        has_loss = pc.is_first_pp if mode == "dualpipev" else pc.is_last_pp
        rec = trainer.reduce_loss_for_logging(res) if has_loss else {"loss": 0.0, "lm_loss": 0.0, "grad_norm": float(res["grad_norm"])}
        losses.append([rec["loss"], rec["lm_loss"], rec["grad_norm"]])
    out = {"mode": mode, "world": world, "losses": losses}
    if mode.endswith("_muon"):
        st = trainer.optimizer.state
        out["muon_whole"] = sum(len(x["muon"]) for x in st)
        out["muon_cut"] = sum(len(x["muon_cross"]) for x in st)
    report_rank = (world - 1 if mode in ("pp", "pp_vpp2") else 0)
    if mode == "dualpipev":
        report_rank = 0                      # the V turns back: the last chunk lives on the first rank
    if pc.rank == report_rank:
        print("RESULT " + json.dumps(out), flush=True)
    pstate.destroy()


if __name__ == "__main__":
    main()
