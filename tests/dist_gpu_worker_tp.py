"""Worker for the fused tensor-parallel test: a column-parallel + row-parallel linear pair under sequence
parallelism, once over NCCL and once with the collectives fused into the GEMMs; prints outputs' checksums."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from cppmega_b200.ops import cuda as cu  # noqa: E402
from cppmega_b200.ops import functional as F_  # noqa: E402
from cppmega_b200.parallel import fused_tp  # noqa: E402
from cppmega_b200.parallel import state as pstate  # noqa: E402
from cppmega_b200.parallel.state import ParallelConfig  # noqa: E402
from cppmega_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear  # noqa: E402


def main():
    world = int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pc = pstate.initialize(ParallelConfig(tp=world, sequence_parallel=True))
    B, S, H, F = 2, 256 * world, 512, 1536
    col = ColumnParallelLinear(H, F, pc, std=0.05, seed=1, dtype=torch.bfloat16, name="col").to(dev)
    row = RowParallelLinear(F, H, pc, std=0.05, seed=2, dtype=torch.bfloat16, name="row").to(dev)
    gen = torch.Generator(device="cpu").manual_seed(7)
    x_full = (torch.randn(B, S, H, generator=gen) * 0.5).bfloat16()
    g_full = (torch.randn(B, S, H, generator=gen) * 0.5).bfloat16()
    Sl = S // world
    sl = slice(pc.tp_rank * Sl, (pc.tp_rank + 1) * Sl)

    def run(fused, mode="staged"):
        if fused:
            tp = fused_tp.install(pc, dev, B * Sl, max(H, F))
            assert tp is not None
            tp.mode = mode
        else:
            fused_tp.uninstall()
        for p in list(col.parameters()) + list(row.parameters()):
            p.grad = None
        x = x_full[:, sl].to(dev).requires_grad_()
        F_.reset_counters()
        y = row(torch.nn.functional.gelu(col(x)))
        y.backward(g_full[:, sl].to(dev))
        torch.cuda.synchronize()
        cu.check_errors()
        return y.detach().float(), x.grad.float(), col.weight.grad.float(), row.weight.grad.float(), F_.launch_counts()

    base = run(False)
    rel = lambda a, b: ((a - b).norm() / b.norm().clamp_min(1e-12)).item()
    res = {"rank": pc.rank, "base_launches": base[4], "modes": {}}
    for mode in ("staged", "direct", "staged"):          # the second staged pass reuses slots that peers have read
        fused = run(True, mode)
        res["modes"][mode] = {"rel": [rel(f, b) for f, b in zip(fused[:4], base[:4])], "launches": fused[4]}
    outs = [None] * world
    torch.distributed.all_gather_object(outs, res)
    if pc.rank == 0:
        print("RESULT " + json.dumps(outs), flush=True)
    pstate.destroy()


if __name__ == "__main__":
    main()
