"""FP8 compression of saved activations (counterpart of cppmega/megatron/fp8_activations.py:598-878)."""
import pytest
import torch

from cppmega_b200.utils import fp8_activations as fa


def _mlp(seed=0, width=256):
    g = torch.Generator().manual_seed(seed)
    w1 = (torch.randn(4 * width, width, generator=g) * 0.05).bfloat16().requires_grad_()
    w2 = (torch.randn(width, 4 * width, generator=g) * 0.05).bfloat16().requires_grad_()
    x = torch.randn(128, width, generator=g).bfloat16().requires_grad_()
    return x, w1, w2


def _run(x, w1, w2, ctx):
    for t in (x, w1, w2):
        t.grad = None
    with ctx:
        h = torch.nn.functional.silu(x @ w1.t())
        y = h @ w2.t()
    y.float().square().mean().backward()
    return [t.grad.float().clone() for t in (x, w1, w2)]


@pytest.mark.parametrize("recipe", ["mxfp8", "tensor"])
def test_saved_activations_are_packed_and_gradients_stay_close(recipe):
    x, w1, w2 = _mlp()
    base = _run(x, w1, w2, fa.fp8_activation_context(enabled=False))
    fa.reset_stats()
    got = _run(x, w1, w2, fa.fp8_activation_context(recipe=recipe, min_elements=1024))
    assert fa.STATS["packed"] >= 1                                  # the hidden activation (x and the weights are leaves)
    assert fa.STATS["bytes_out"] < 0.54 * fa.STATS["bytes_in"]      # 1 byte + 1/32 scale byte per 2-byte value
    for b, g in zip(base, got):
        rel = (b - g).norm() / b.norm()
        assert 0 < rel < 0.08, rel                                  # compressed (not identical) but close


def test_small_tensors_parameters_and_other_dtypes_pass_through():
    p = fa.Fp8ActivationPacker(min_elements=64)
    small = torch.randn(8, 4).bfloat16()
    assert p.pack(small) is small
    f32 = torch.randn(64, 64)
    assert p.pack(f32) is f32
    idx = torch.arange(4096)
    assert p.pack(idx) is idx
    par = torch.nn.Parameter(torch.randn(64, 64).bfloat16())
    assert p.pack(par) is par
    odd = torch.randn(33, 5).bfloat16()                             # 165 values: not a multiple of 32
    assert p.pack(odd) is odd
    assert p.pack(None) is None and p.pack(3) == 3
    big = torch.randn(4, 16, 48).bfloat16()                         # last dim 48: packed as rows of 32
    q = p.pack(big)
    assert isinstance(q, fa.PackedActivation) and q.shape == (4, 16, 48)
    back = p.unpack(q)
    assert back.shape == big.shape and back.dtype == torch.bfloat16
    assert (back.float() - big.float()).abs().max() <= 0.07 * big.float().abs().max()


def test_opt_out_context_and_decorator():
    p = fa.Fp8ActivationPacker(min_elements=64)
    t = torch.randn(64, 64).bfloat16()
    with fa.fp8_quantize_disabled():
        with fa.fp8_quantize_disabled():
            assert p.pack(t) is t
        assert p.pack(t) is t
    assert isinstance(p.pack(t), fa.PackedActivation)

    @fa.no_fp8_quantize
    def f():
        return p.pack(t)

    assert f() is t


def test_first_and_last_layers_stay_bf16():
    assert fa.is_bf16_layer(0, 8, 1, 1) and fa.is_bf16_layer(7, 8, 1, 1)
    assert not fa.is_bf16_layer(1, 8, 1, 1) and not fa.is_bf16_layer(6, 8, 1, 1)
    assert fa.is_bf16_layer(1, 8, 2, 0) and not fa.is_bf16_layer(7, 8, 2, 0)
    assert not fa.is_bf16_layer(-1, 8, 1, 1)                        # outside the stack: compress
    p = fa.LayerAwareFp8Packer(4, 1, 1, min_elements=64)
    t = torch.randn(64, 64).bfloat16()
    try:
        for idx, packed in ((0, False), (1, True), (2, True), (3, False)):
            fa.set_current_layer_idx(idx)
            assert isinstance(p.pack(t), fa.PackedActivation) == packed
    finally:
        fa.set_current_layer_idx(-1)


def test_tensor_recipe_clamp_saturates_outliers():
    t = torch.randn(64, 64).bfloat16()
    t[0, 0] = 30000.0
    plain = fa.Fp8ActivationPacker("tensor", min_elements=64)
    clamp = fa.Fp8ActivationPacker("tensor", clamp=True, min_elements=64)
    a, b = plain.unpack(plain.pack(t)).float(), clamp.unpack(clamp.pack(t)).float()
    assert a[0, 0] > 20000 and b[0, 0] <= 448.0                     # the outlier survives / saturates
    rest = torch.ones_like(t, dtype=torch.bool)
    rest[0, 0] = False
    err_plain = (a - t.float())[rest].abs().mean()
    err_clamp = (b - t.float())[rest].abs().mean()
    assert err_clamp < 0.5 * err_plain                              # the bulk keeps its precision under the clamp


def test_training_with_compressed_activations_follows_the_bf16_loss_curve():
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches
    curves = {}
    for mode in ("off", "mxfp8"):
        cfg = nam56r_tiny(seq_length=64)
        tc = TrainConfig(micro_batch_size=2, seq_length=64, dtype="bf16", fp8_activations=mode, log_interval=0,
                         optimizer=OptimizerConfig(lr=1e-3, weight_decay=0.0))
        tr = Trainer(cfg, tc, device=torch.device("cpu"))
        stream = synthetic_batches(cfg.vocab_size, 2, 64, seed=0, pin=False)
        fa.reset_stats()
        curves[mode] = [float(tr.train_step(next(stream))["loss"]) for _ in range(3)]
        if mode == "mxfp8":
            assert fa.STATS["packed"] > 0
        else:
            assert fa.STATS["packed"] == 0
    for a, b in zip(curves["off"], curves["mxfp8"]):
        assert abs(a - b) < 0.05 * abs(a), curves


@pytest.mark.gpu
@pytest.mark.parametrize("recipe", ["mxfp8", "tensor"])
def test_pack_unpack_kernels_match_the_definition(recipe):
    from cppmega_b200.ops import functional as F_
    dev = torch.device("cuda")
    t = (torch.randn(2, 512, 384, device=dev) * 3).bfloat16()
    p = fa.Fp8ActivationPacker(recipe)
    F_.reset_counters()
    q = p.pack(t)
    assert isinstance(q, fa.PackedActivation) and q.payload.dtype == torch.uint8
    out = p.unpack(q)
    assert F_.launch_counts().get("mxfp8_quantize", 0) == 1 and F_.launch_counts().get("mxfp8_dequantize", 0) == 1
    ref = p.unpack(p.pack(t.cpu()))                                 # the PyTorch definition of the same recipe
    assert out.shape == t.shape and out.dtype == torch.bfloat16
    assert torch.equal(out.cpu(), ref)


def test_a_tensor_saved_by_several_consumers_is_packed_once():
    x = torch.randn(128, 256).bfloat16().requires_grad_()
    w = [(torch.randn(64, 256) * 0.05).bfloat16().requires_grad_() for _ in range(3)]
    fa.reset_stats()
    with fa.fp8_activation_context(recipe="mxfp8", min_elements=1024):
        h = torch.nn.functional.silu(x)                     # saved by silu's backward? no: silu saves its input x
        ys = [h @ wi.t() for wi in w]                       # h is saved three times, once per product
    assert fa.STATS["shared"] == 2 and fa.STATS["packed"] == 1, fa.STATS       # h once; x and the weights are leaves
    sum(y.float().square().mean() for y in ys).backward()
    assert x.grad is not None and all(wi.grad is not None for wi in w)
