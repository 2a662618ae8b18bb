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
