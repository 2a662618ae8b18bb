"""Fused Mamba3 MIMO scan kernels against the fp32 PyTorch definition."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _inputs(B, S, H, G, N=128, P=64, R=4, seed=0):
    torch.manual_seed(seed)
    dev = "cuda"
    Qn = (torch.randn(B, S, G, R, N, device=dev) * 0.5).bfloat16()
    Kn = (torch.randn(B, S, G, R, N, device=dev) * 0.5).bfloat16()
    V = torch.randn(B, S, H, P, device=dev).bfloat16()
    Z = torch.randn(B, S, H, P, device=dev).bfloat16()
    DT = torch.rand(B, H, S, device=dev) * 0.1 + 0.001
    ADT = -DT * (torch.rand(B, H, S, device=dev) * 4 + 0.1)
    Trap = torch.randn(B, H, S, device=dev)
    Qb = torch.randn(H, R, N, device=dev) * 0.3
    Kb = torch.randn(H, R, N, device=dev) * 0.3
    Psi, Zeta, Phi = (torch.randn(H, R, P, device=dev) * 0.5 for _ in range(3))
    ang = (torch.randn(B, S, H, N // 4, device=dev) * 0.2).cumsum(1)
    D = torch.randn(H, device=dev)
    return Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D


@pytest.mark.parametrize("B,S,H,G", [(1, 32, 2, 1), (2, 128, 4, 2), (1, 256, 16, 1)])
def test_mimo_scan_forward(B, S, H, G):
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import mimo_scan_ref as R
    from cppmega_b200.ops.cuda import kernels3
    Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _inputs(B, S, H, G)
    y, states, tot, final = kernels3.mimo_fwd_raw(Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D,
                                                   want_state=True)
    torch.cuda.synchronize()
    cu.check_errors()
    Q5, K5 = Qn.permute(0, 1, 3, 2, 4), Kn.permute(0, 1, 3, 2, 4)
    yr, sr = R.mimo_scan_chunked(Q5.float(), K5.float(), V.float(), ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D,
                                 Z.float(), 4, 16, return_state=True)
    assert _rel(final, sr) < 2e-2
    assert _rel(y, yr) < 2e-2


def test_mimo_scan_autograd_runs():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import mimo_scan_ref as R
    from cppmega_b200.ops.cuda import kernels3
    Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _inputs(1, 64, 4, 2, seed=1)
    Q5, K5 = Qn.permute(0, 1, 3, 2, 4), Kn.permute(0, 1, 3, 2, 4)
    args = [Q5, K5, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z]
    a1 = [t.detach().clone().requires_grad_() for t in args]
    a2 = [t.detach().float().clone().requires_grad_() for t in args]
    y1 = kernels3.mimo_scan(*a1, 4, 16)
    y2 = R.mimo_scan_sequential(*a2, 4)
    g = torch.randn_like(y2)
    y1.backward(g.to(y1.dtype))
    y2.backward(g)
    cu.check_errors()
    assert _rel(y1, y2) < 2e-2
    names = "Q K V ADT DT Trap Qb Kb Psi Zeta Phi angles D Z".split()
    for n, x, r in zip(names, a1, a2):
        assert _rel(x.grad, r.grad) < 6e-2, n


@pytest.mark.parametrize("B,S,H,G", [(2, 512, 16, 2), (1, 1024, 8, 8)])
def test_mimo_scan_backward_many_chunks(B, S, H, G):
    """All 14 gradients against autograd through the fp32 chunked definition: 16 / 32 chunks of the kernels' 32-token
    tile (the reverse inter-chunk recurrence runs many steps), batch stride B > 1, one head per group (G == H) and
    several heads per group (G < H)."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import mimo_scan_ref as R
    from cppmega_b200.ops.cuda import kernels3
    Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _inputs(B, S, H, G, seed=2)
    Q5, K5 = Qn.permute(0, 1, 3, 2, 4), Kn.permute(0, 1, 3, 2, 4)
    args = [Q5, K5, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z]
    a1 = [t.detach().clone().requires_grad_() for t in args]
    a2 = [t.detach().float().clone().requires_grad_() for t in args]
    y1 = kernels3.mimo_scan(*a1, 4, 16)
    y2 = R.mimo_scan_chunked(*a2, 4, 16)
    g = torch.randn_like(y2)
    y1.backward(g.to(y1.dtype))
    y2.backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    assert _rel(y1, y2) < 2e-2
    names = "Q K V ADT DT Trap Qb Kb Psi Zeta Phi angles D Z".split()
    for n, x, r in zip(names, a1, a2):
        assert x.grad is not None and torch.isfinite(x.grad.float()).all(), n
        assert _rel(x.grad, r.grad) < 6e-2, (n, _rel(x.grad, r.grad))


@pytest.mark.parametrize("N,B,S,H,G", [(64, 2, 256, 8, 1), (32, 2, 64, 4, 2)])
def test_mimo_scan_smaller_state_dims(N, B, S, H, G):
    """State dimension 64 (the shape of the reference's published kernel timings: B2 S256 H8 G1 N64 P64 R4) and 32
    (the CPU plumbing configuration) run on the kernels through zero padding; forward and all gradients against the
    fp32 definition at the ORIGINAL state dimension."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops import mimo_scan_ref as R
    from cppmega_b200.ops.cuda import kernels3
    Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _inputs(B, S, H, G, N=N, seed=3)
    Q5, K5 = Qn.permute(0, 1, 3, 2, 4), Kn.permute(0, 1, 3, 2, 4)
    args = [Q5, K5, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z]
    a1 = [t.detach().clone().requires_grad_() for t in args]
    a2 = [t.detach().float().clone().requires_grad_() for t in args]
    F_.reset_counters()
    y1 = kernels3.mimo_scan(*a1, 4, 16)
    assert F_.launch_counts().get("mimo_scan_fwd", 0) == 3 and not F_.fallback_counts()
    y2 = R.mimo_scan_chunked(*a2, 4, 16)
    g = torch.randn_like(y2)
    y1.backward(g.to(y1.dtype))
    y2.backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    assert _rel(y1, y2) < 2e-2
    names = "Q K V ADT DT Trap Qb Kb Psi Zeta Phi angles D Z".split()
    for n, x, r in zip(names, a1, a2):
        assert x.grad.shape == r.grad.shape, n
        assert _rel(x.grad, r.grad) < 6e-2, (n, _rel(x.grad, r.grad))


@pytest.mark.gpu
@pytest.mark.parametrize("n", [64, 32])
def test_state_dim_padding_kernel_matches_the_concatenations(n):
    """One launch widens Q / K / biases (split halves) and the angles (zero-extended); its adjoint narrows the gradients."""
    from cppmega_b200.ops.cuda import kernels3
    torch.manual_seed(n)
    dev = "cuda"
    Q = torch.randn(2, 64, 4, 2, n, device=dev).bfloat16().requires_grad_()
    K = torch.randn(2, 64, 4, 2, n, device=dev).bfloat16().permute(0, 1, 2, 3, 4).requires_grad_()
    Qb, Kb = torch.randn(8, 4, n, device=dev).requires_grad_(), torch.randn(8, 4, n, device=dev).requires_grad_()
    ang = torch.randn(2, 64, 8, n // 4, device=dev).requires_grad_()
    outs = kernels3.PadStateFn.apply(Q, K, Qb, Kb, ang)
    refs = [kernels3._pad_state_dim(t, n) for t in (Q, K, Qb, Kb)] + [
        torch.cat([ang, ang.new_zeros(*ang.shape[:-1], 32 - ang.shape[-1])], dim=-1)]
    gs = [torch.randn_like(o) for o in outs]
    got = torch.autograd.grad(outs, (Q, K, Qb, Kb, ang), gs)
    want = torch.autograd.grad(refs, (Q, K, Qb, Kb, ang), gs)
    for o, r in zip(outs, refs):
        assert o.shape == r.shape and torch.equal(o, r)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
