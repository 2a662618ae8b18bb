"""Bandwidth-bound kernels and the fused cross-entropy against fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("rows,H", [(37, 64), (1000, 128), (513, 256), (300, 1024), (257, 4096), (64, 8192)])
def test_rmsnorm(rows, H):
    from cppmega_b200.ops import cuda as cu, reference as ref
    torch.manual_seed(rows)
    x = torch.randn(rows, H, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    y = cu.rmsnorm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rmsnorm(xr, wr, 1e-5)
    yr.backward(g.float())
    assert _rel(y, yr) < 6e-3
    assert _rel(x.grad, xr.grad) < 8e-3
    assert _rel(w.grad, wr.grad) < 8e-3


def test_swiglu():
    from cppmega_b200.ops import cuda as cu, reference as ref
    torch.manual_seed(0)
    x = torch.randn(777, 2 * 896, device="cuda").bfloat16().requires_grad_()
    y = cu.swiglu(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = ref.swiglu(xr)
    yr.backward(g.float())
    assert _rel(y, yr) < 6e-3
    assert _rel(x.grad, xr.grad) < 8e-3


@pytest.mark.parametrize("gdt", [torch.float32, torch.bfloat16])
def test_adamw(gdt):
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.optim.adamw import adamw_reference
    torch.manual_seed(0)
    n = 100_003
    master = torch.randn(n, device="cuda")
    m = torch.randn(n, device="cuda") * 0.1
    v = torch.rand(n, device="cuda") * 0.01
    g = torch.randn(n, device="cuda").to(gdt)
    wd = torch.rand(n, device="cuda") > 0.5
    clip = torch.tensor(0.7, device="cuda")
    ref_state = [t.clone() for t in (master, m, v)]
    out_ref = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    adamw_reference(*ref_state, g, out_ref, wd, clip, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05)
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    cu.adamw_shard(master, m, v, g, out, wd, clip, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05)
    for a, b in zip((master, m, v), ref_state):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
    assert torch.allclose(out.float(), out_ref.float(), rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("T,H,V", [(300, 256, 4096), (5000, 128, 1024)])
def test_linear_ce_weighted(T, H, V):
    from cppmega_b200.ops import cuda as cu, reference as ref
    from cppmega_b200.ops.cuda import extra
    torch.manual_seed(0)
    h = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.1).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    rw = torch.rand(T, device="cuda") / T
    total, per = extra.linear_cross_entropy_weighted(h, w, labels, rw, -100)
    (total * 0.5).backward()
    cu.check_errors()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    pr = ref.linear_cross_entropy(hr, wr, labels, -100, "none")
    tr = (pr * rw).sum()
    (tr * 0.5).backward()
    assert torch.allclose(per, pr, rtol=2e-2, atol=2e-2)
    assert abs(total.item() - tr.item()) < 2e-2 * abs(tr.item()) + 1e-3
    assert _rel(h.grad, hr.grad) < 3e-2
    assert _rel(w.grad, wr.grad) < 3e-2
