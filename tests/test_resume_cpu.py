"""Resume: data position, optimizer-state rules and per-rank random state."""
import numpy as np
import pytest
import torch

from cppmega_b200.checkpoint import sharded
from cppmega_b200.config.model import nam56r_tiny
from cppmega_b200.data.indexed import TokenStream, write_indexed_dataset
from cppmega_b200.models import build_model
from cppmega_b200.parallel.dist_optimizer import DistributedOptimizer, OptimizerConfig
from cppmega_b200.parallel.state import ParallelConfig, ParallelContext
from cppmega_b200.training.trainer import synthetic_batches


def test_synthetic_stream_skip_equals_consuming():
    a = synthetic_batches(1000, 2, 16, num_microbatches=2, seed=3, pin=False, rank=1)
    for _ in range(5):
        next(a)
    b = synthetic_batches(1000, 2, 16, num_microbatches=2, seed=3, pin=False, rank=1, skip=5)
    for _ in range(3):
        xa, xb = next(a), next(b)
        for ma, mb in zip(xa, xb):
            assert torch.equal(ma["input_ids"], mb["input_ids"]) and torch.equal(ma["labels"], mb["labels"])


def test_token_stream_skip_equals_consuming(tmp_path):
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 500, size=int(n)).tolist() for n in rng.integers(20, 90, size=40)]
    prefix = str(tmp_path / "toy")
    write_indexed_dataset(prefix, docs)
    kw = dict(seq_len=16, micro_batch=3, rank=1, world=2, seed=11, pin=False, native=False)
    a, b = TokenStream(prefix, **kw), TokenStream(prefix, **kw)
    n = a.num_samples // (3 * 2) + 4           # crosses an epoch boundary
    for _ in range(n):
        next(a)
    b.skip(n)
    for _ in range(5):
        assert torch.equal(next(a)["input_ids"], next(b)["input_ids"])


def test_optimizer_state_is_not_dropped_silently(tmp_path):
    pc = ParallelContext(config=ParallelConfig())
    cfg = nam56r_tiny(depth=2, pattern="ME")
    model = build_model(cfg, pc)
    opt = DistributedOptimizer(model, OptimizerConfig(), pc)
    d = sharded.save_checkpoint(str(tmp_path), 3, model, pc, opt, extra={"consumed_steps": 3},
                                rank_extra={"rng": {"torch_cpu": torch.get_rng_state()}})
    info = sharded.load_checkpoint(str(tmp_path), model, pc, opt, allow_optimizer_reset=False)
    assert info["optimizer_reset"] is None and info["extra"]["consumed_steps"] == 3
    assert torch.equal(info["rank_extra"]["rng"]["torch_cpu"], torch.get_rng_state())
    (tmp_path / "iter_0000003" / "optim_rank00000.pt").unlink()
    with pytest.raises(ValueError, match="cannot restore the optimizer state"):
        sharded.load_checkpoint(str(tmp_path), model, pc, opt, allow_optimizer_reset=False)
    with pytest.warns(UserWarning, match="optimizer state NOT restored"):
        info = sharded.load_checkpoint(str(tmp_path), model, pc, opt, allow_optimizer_reset=True)
    assert "moments zeroed" in info["optimizer_reset"]
    _ = d


def test_a_closed_trainer_is_released():
    """The gradient hooks sit in the tensors' autograd metadata (a cycle the garbage collector cannot see): ``close()``
    removes them, after which dropping the trainer frees model, flat buffers and optimizer state."""
    import gc
    import weakref
    import torch
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches
    cfg = nam56r_tiny(seq_length=32)
    tr = Trainer(cfg, TrainConfig(micro_batch_size=1, seq_length=32, dtype="fp32", log_interval=0,
                                  optimizer=OptimizerConfig(lr=1e-3)), device=torch.device("cpu"))
    stream = synthetic_batches(cfg.vocab_size, 1, 32, seed=0, pin=False)
    float(tr.train_step(next(stream))["loss"])
    wm, wo = weakref.ref(tr.model), weakref.ref(tr.optimizer)
    tr.close()
    del tr, stream
    gc.collect()
    assert wm() is None and wo() is None
