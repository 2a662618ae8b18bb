"""Device-side failure detection without a GPU fault: a bounded wait on a flag that nobody sets runs out, the kernel
returns, the error word names the cause, and the kernels behind it on the stream leave the optimizer state alone."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _heap():
    from cppmega_b200.parallel.symm_mem import SymmetricHeap
    return SymmetricHeap(None, [0], 1 << 20, torch.device("cuda", 0))


def test_wait_on_a_flag_nobody_sets_returns_with_an_error_status():
    from cppmega_b200.ops import cuda as cu
    torch.cuda.set_device(0)
    cu.check_errors()
    heap = _heap()
    try:
        t0 = time.perf_counter()
        heap.wait(7, 1, timeout_ns=1_000_000)            # 1 ms: flag word 7 stays 0
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 5.0, "the wait did not return promptly"
        with pytest.raises(cu.KernelError, match="peer flag never set"):
            cu.check_errors()
        cu.check_errors()                                 # the word was cleared by the failed check
        # the context is still usable, and a flag that IS set passes
        heap.signal(7, 1)
        heap.wait(7, 1, timeout_ns=1_000_000)
        x = torch.arange(8, device="cuda").float().sum()
        torch.cuda.synchronize()
        cu.check_errors()
        assert float(x) == 28.0
    finally:
        heap.close()


def test_update_is_skipped_on_the_device_after_a_timed_out_wait():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.optim.adamw import adamw_shard_update
    torch.cuda.set_device(0)
    cu.check_errors()
    heap = _heap()
    try:
        n = 4096 + 3
        g = torch.Generator(device="cuda").manual_seed(0)
        master = torch.randn(n, device="cuda", generator=g)
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        grad = torch.randn(n, device="cuda", generator=g)
        out = master.to(torch.bfloat16)
        wd = torch.ones(n, dtype=torch.bool, device="cuda")
        clip = torch.ones((), device="cuda")
        before = (master.clone(), m.clone(), v.clone(), out.clone())
        gate = cu.err_word(master.device)
        heap.wait(9, 1, timeout_ns=1_000_000)            # runs out: error word set, stream carries on
        adamw_shard_update(master, m, v, grad, out, wd, clip, 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, gate=gate)
        torch.cuda.synchronize()
        for a, b in zip(before, (master, m, v, out)):
            assert torch.equal(a, b), "the gated update touched optimizer state after a failed wait"
        with pytest.raises(cu.KernelError):
            cu.check_errors()
        # with the word clear the same call updates
        adamw_shard_update(master, m, v, grad, out, wd, clip, 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, gate=gate)
        torch.cuda.synchronize()
        cu.check_errors()
        assert not torch.equal(before[0], master) and m.abs().sum() > 0
    finally:
        heap.close()
