"""Memory-bound kernels around the mixers and the permute-fused MoE path, against PyTorch definitions."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("B,S,H,A,transposed", [(2, 1300, 6, 32, True), (1, 512, 3, 8, False), (2, 96, 4, 32, True)])
def test_angle_cumsum(B, S, H, A, transposed):
    from cppmega_b200.ops import mimo_scan_ref as R
    from cppmega_b200.ops.cuda import kernels4
    torch.manual_seed(0)
    raw = torch.randn(B, S, A, device="cuda").bfloat16().requires_grad_()
    base = (torch.rand(B, S, H, device="cuda") * 0.1) if transposed else (torch.rand(B, H, S, device="cuda") * 0.1)
    base.requires_grad_()
    dt = base.transpose(1, 2) if transposed else base
    out = kernels4.angle_cumsum(raw, dt)
    g = torch.randn_like(out)
    out.backward(g)
    raw2 = raw.detach().clone().requires_grad_()
    base2 = base.detach().clone().requires_grad_()
    ref = R.angle_cumsum(raw2, base2.transpose(1, 2) if transposed else base2)
    ref.backward(g)
    assert _rel(out, ref) < 1e-4
    assert _rel(raw.grad, raw2.grad) < 1e-2          # bf16 gradient
    assert _rel(base.grad, base2.grad) < 1e-4


def test_local_fused_moe_matches_plain_dispatch():
    from cppmega_b200.config.model import MoEConfig
    from cppmega_b200.models.moe import MoELayer
    from cppmega_b200.parallel import fused_moe
    from cppmega_b200.parallel.state import single_process_context
    from cppmega_b200.ops import cuda as cu
    pc = single_process_context()
    cfg = MoEConfig(num_experts=8, topk=2, expert_ffn=64, shared_expert_ffn=0)
    hidden = 128
    layer = MoELayer(hidden, cfg, pc, "decoder.layers.0", dtype=torch.bfloat16, seed=3).cuda()
    layer.train()
    x = (torch.randn(2, 200, hidden, device="cuda") * 0.5).bfloat16()
    g = torch.randn_like(x)

    def run(fused):
        layer.zero_grad(set_to_none=True)
        layer.fused_dispatcher = (fused_moe.FusedMoEDispatcher(fused_moe.LocalMoEBuffers(pc, hidden, cfg.num_experts, x.device), 0)
                                  if fused else None)
        xi = x.clone().requires_grad_()
        y = layer(xi)
        y.backward(g)
        torch.cuda.synchronize()
        cu.check_errors()
        return y, xi.grad, {n: p.grad.clone() for n, p in layer.named_parameters() if p.grad is not None}

    y0, dx0, g0 = run(False)
    y1, dx1, g1 = run(True)
    assert _rel(y1, y0) < 2e-2
    assert _rel(dx1, dx0) < 3e-2
    assert set(g0) == set(g1)
    for n in g0:
        assert _rel(g1[n], g0[n]) < 4e-2, n
