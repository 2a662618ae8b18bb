"""Worker of the context-parallel DSA test (gloo): every rank runs one sparse-attention layer on its chunk of the
sequence with the keys gathered over the group; rank 0 prints the distance to the single-process result."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from cppmega_b200.config.model import nam56r_tiny  # noqa: E402
from cppmega_b200.models.attention import MLAttention  # noqa: E402
from cppmega_b200.parallel.context_parallel import ContextGroup  # noqa: E402
from cppmega_b200.parallel.state import single_process_context  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    cfg = nam56r_tiny()
    pc = single_process_context()
    layer = MLAttention(cfg.hidden_size, cfg.mla, pc, "decoder.layers.4", dsa=cfg.dsa, dsa_rank=0, dtype=torch.float32, seed=7)
    B, S = 2, 96
    x = torch.randn(B, S, cfg.hidden_size)
    g = torch.randn(B, S, cfg.hidden_size)
    # single process, whole sequence
    xf = x.clone().requires_grad_()
    yf = layer(xf)
    (yf * g).sum().backward()
    ref_grads = {n: p.grad.clone() for n, p in layer.named_parameters() if p.grad is not None}
    ref_dx = xf.grad.clone()
    layer.zero_grad()
    # split sequence
    n = S // world
    layer.context_group = ContextGroup(dist.group.WORLD, world, rank)
    xc = x[:, rank * n:(rank + 1) * n].clone().requires_grad_()
    yc = layer(xc)
    (yc * g[:, rank * n:(rank + 1) * n]).sum().backward()
    rel = lambda a, b: float((a - b).norm() / b.norm().clamp_min(1e-12))
    out = {"y": rel(yc, yf[:, rank * n:(rank + 1) * n].detach()), "dx": rel(xc.grad, ref_dx[:, rank * n:(rank + 1) * n])}
    worst = 0.0
    for name, p in layer.named_parameters():
        if name not in ref_grads:
            continue
        gsum = p.grad.clone() if p.grad is not None else torch.zeros_like(p)
        dist.all_reduce(gsum)
        worst = max(worst, rel(gsum, ref_grads[name]))
    out["param_grads"] = worst
    t = torch.tensor([out["y"], out["dx"]])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print("RESULT " + json.dumps({"y": float(t[0]), "dx": float(t[1]), "param_grads": worst}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
