"""CUDA-graph capture of static layers: a captured run follows the eager loss curve."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(scope, steps=3):
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.parallel import state as pstate
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.parallel.state import ParallelConfig
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches
    pc = pstate.initialize(ParallelConfig())
    try:
        mcfg = nam56r_tiny(seq_length=128)
        tcfg = TrainConfig(micro_batch_size=2, seq_length=128, dtype="bf16", cuda_graph_scope=scope,
                           optimizer=OptimizerConfig(lr=1e-3, weight_decay=0.0), log_interval=0)
        trainer = Trainer(mcfg, tcfg, pc, device=torch.device("cuda", 0))
        stream = synthetic_batches(mcfg.vocab_size, 2, 128, num_microbatches=1, seed=0, pin=False, rank=0)
        losses = []
        for _ in range(steps):
            res = trainer.train_step(next(stream))
            losses.append(trainer.reduce_loss_for_logging(res)["loss"])
        torch.cuda.synchronize()
        cu.check_errors()
        replays = sum(getattr(l, "replays", 0) for l in trainer.model.decoder.layers.values())
        return losses, trainer.graphed_layers, replays
    finally:
        pstate.destroy()


def test_graphed_mamba_and_attention_layers_match_eager():
    eager, n0, _ = _run(())
    graphed, n, replays = _run(("mamba", "attn"))
    assert n0 == 0 and n > 0 and replays == n * len(graphed)
    for a, b in zip(eager, graphed):
        assert abs(a - b) < 3e-2 * max(1.0, abs(a)), (eager, graphed)
