"""Activation recomputation with the operator stash: gradients equal plain autograd, stashed ops run once."""
import torch

from cppmega_b200.utils import recompute as rc


class _TanhFromSaved(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y):
        ctx.save_for_backward(y)
        return y.clone()

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        return g * (1 - y * y), None


def _layer(lin, calls):
    def expensive(x):
        def compute():
            calls["n"] += 1
            return (torch.tanh(x.detach()),)
        return rc.stashed_call("tanh", compute, lambda res: _TanhFromSaved.apply(x, res[0]))

    def layer(x, unused):
        return lin(expensive(lin(x))) + expensive(x)
    return layer


def test_checkpoint_matches_autograd_and_stash_skips_replay():
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 8)
    calls = {"n": 0}
    layer = _layer(lin, calls)
    x = torch.randn(4, 8, requires_grad=True)
    rc.checkpoint(layer, x, None).sum().backward()
    g1, w1 = x.grad.clone(), lin.weight.grad.clone()
    assert calls["n"] == 2                      # two stashed ops, each computed once (not again in the replay)
    x.grad = None
    lin.zero_grad()
    (lin(torch.tanh(lin(x))) + torch.tanh(x)).sum().backward()
    torch.testing.assert_close(g1, x.grad)
    torch.testing.assert_close(w1, lin.weight.grad)


def test_stash_can_be_disabled_and_is_released():
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 8)
    calls = {"n": 0}
    layer = _layer(lin, calls)
    x = torch.randn(4, 8, requires_grad=True)
    rc.STASH_ENABLED = False
    try:
        rc.checkpoint(layer, x, None).sum().backward()
    finally:
        rc.STASH_ENABLED = True
    assert calls["n"] == 4                      # without the stash both passes compute
    assert rc.current_stash() is None           # nothing leaks out of a finished checkpoint
    with torch.no_grad():
        assert rc.checkpoint(layer, x, None).shape == (4, 8)


def test_model_gradients_identical_with_and_without_recompute():
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.models.nam56r import build_model
    cfg = nam56r_tiny(seq_length=32)
    ids = torch.randint(0, cfg.vocab_size, (2, 32))
    grads = []
    for mode in ("none", "full"):
        torch.manual_seed(0)
        m = build_model(cfg, recompute=mode)
        m.train()
        m(ids, ids)["loss"].backward()
        grads.append({n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None})
    assert grads[0].keys() == grads[1].keys()
    for n in grads[0]:         # same mathematics, different fp32 accumulation order
        a, b = grads[0][n], grads[1][n]
        assert ((a - b).norm() / (a.norm() + 1e-12)).item() < 2e-3, n


def test_m2rnn_chunked_reference_matches_stepwise_definition():
    import torch
    from cppmega_b200.ops import reference as ref
    from cppmega_b200.ops.m2rnn_chunk_ref import m2rnn_scan_chunked
    torch.manual_seed(0)
    B, S, H, K, V = 2, 37, 3, 8, 4
    mk = lambda *s: torch.randn(*s, dtype=torch.float64).mul(0.5).requires_grad_()
    q, k, v = mk(B, S, 1, K), mk(B, S, 1, K), mk(B, S, H, V)
    W = (torch.eye(V, dtype=torch.float64).repeat(H, 1, 1) + 0.1 * torch.randn(H, V, V, dtype=torch.float64)).requires_grad_()
    f = torch.rand(B, S, H, dtype=torch.float64).requires_grad_()
    h0 = mk(B, H, K, V)
    gy, gh = torch.randn(B, S, H, V, dtype=torch.float64), torch.randn(B, H, K, V, dtype=torch.float64)

    def run(fn, with_h0):
        ins = [t.detach().clone().requires_grad_() for t in (q, k, v, W, f)] + ([h0.detach().clone().requires_grad_()] if with_h0 else [])
        y, h = fn(*ins)
        ((y.double() * gy).sum() + (h.double() * gh).sum()).backward()
        return y, h, [t.grad for t in ins]

    for with_h0 in (False, True):
        y1, h1, g1 = run(ref.m2rnn_scan, with_h0)
        y2, h2, g2 = run(lambda *a: m2rnn_scan_chunked(*a, chunk=8), with_h0)
        assert torch.allclose(y1.double(), y2.double(), atol=1e-5) and torch.allclose(h1.double(), h2.double(), atol=1e-5)
        for a, b in zip(g1, g2):
            assert torch.allclose(a.double(), b.double(), atol=1e-4), (a - b).abs().max()
