"""Sequence-mixer kernels against the fp32 PyTorch definitions."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("B,S,H,KD,shared", [(2, 77, 3, 64, True), (1, 130, 5, 16, True), (2, 64, 4, 32, False)])
def test_m2rnn_scan(B, S, H, KD, shared):
    from cppmega_b200.ops import reference as ref
    from cppmega_b200.ops.cuda import kernels2
    torch.manual_seed(0)
    Hq = 1 if shared else H
    dev = "cuda"
    q = (torch.randn(B, S, Hq, KD, device=dev) * 0.5).bfloat16().requires_grad_()
    k = (torch.randn(B, S, Hq, KD, device=dev) * 0.5).bfloat16().requires_grad_()
    v = (torch.randn(B, S, H, 16, device=dev) * 0.5).bfloat16().requires_grad_()
    W = (torch.eye(16, device=dev).repeat(H, 1, 1) + 0.1 * torch.randn(H, 16, 16, device=dev)).bfloat16().requires_grad_()
    f = torch.rand(B, S, H, device=dev).requires_grad_()
    y = kernels2.m2rnn_scan(q, k, v, W, f)
    g = torch.randn_like(y)
    y.backward(g)
    refs = [t.detach().float().requires_grad_() for t in (q, k, v, W, f)]
    yr, _ = ref.m2rnn_scan(*refs)
    yr.backward(g.float())
    assert _rel(y, yr) < 2e-2
    for name, a, b in zip("q k v W f".split(), (q, k, v, W, f), refs):
        assert _rel(a.grad, b.grad) < 4e-2, name


def test_mimo_scan_lean_matches_sequential():
    from cppmega_b200.ops import mimo_scan_ref as R
    from cppmega_b200.ops.mimo_scan_lean import mimo_scan_lean
    torch.manual_seed(0)
    dev = "cuda"
    B, S, Rk, G, N, H, P = 2, 96, 4, 2, 32, 4, 16
    Q = torch.randn(B, S, Rk, G, N, device=dev)
    K = torch.randn(B, S, Rk, G, N, device=dev)
    V = torch.randn(B, S, H, P, device=dev)
    Z = torch.randn(B, S, H, P, device=dev)
    DT = torch.rand(B, H, S, device=dev) * 0.1
    ADT = -DT * torch.rand(B, H, S, device=dev) * 3
    Trap = torch.randn(B, H, S, device=dev)
    Qb, Kb = torch.randn(H, Rk, N, device=dev), torch.randn(H, Rk, N, device=dev)
    Psi, Zeta, Phi = (torch.randn(H, Rk, P, device=dev) for _ in range(3))
    ang = torch.randn(B, S, H, N // 4, device=dev).cumsum(1) * 0.1
    D = torch.randn(H, device=dev)
    args = [Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z]
    a1 = [t.clone().requires_grad_() for t in args]
    a2 = [t.clone().requires_grad_() for t in args]
    y1 = R.mimo_scan_sequential(*a1, 4)
    y2 = mimo_scan_lean(*a2, 4, 32)
    g = torch.randn_like(y1)
    y1.backward(g)
    y2.backward(g)
    assert _rel(y2, y1) < 2e-2
    for i, (x, r) in enumerate(zip(a2, a1)):
        assert _rel(x.grad, r.grad) < 5e-2, i


def _attn_ref(q, k, v, scale):
    """fp32 causal attention, [B,S,H,D] layout."""
    B, S, H, _ = q.shape
    s = torch.einsum("bihd,bjhd->bhij", q.float(), k.float()) * scale
    s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return torch.einsum("bhij,bjhd->bihd", torch.softmax(s, dim=-1), v.float())


@pytest.mark.parametrize("B,S,H", [(1, 128, 2), (2, 512, 4), (1, 1024, 3)])
def test_dense_causal_attention_kernels(B, S, H):
    """Forward and the three gradients of the tcgen05 attention kernels against the fp32 definition: one key tile, several
    key tiles (online softmax, the state gradients kept in TMEM over the query loop), batch and head strides."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    torch.manual_seed(S)
    q = (torch.randn(B, S, H, 128, device="cuda") * 0.7).bfloat16().requires_grad_()
    k = (torch.randn(B, S, H, 128, device="cuda") * 0.7).bfloat16().requires_grad_()
    v = torch.randn(B, S, H, 64, device="cuda").bfloat16().requires_grad_()
    scale = 128 ** -0.5
    F_.reset_counters()
    o = F_.causal_attention(q, k, v, scale)
    assert F_.launch_counts().get("causal_attention", 0) == 1 and not F_.fallback_counts()
    g = torch.randn_like(o)
    o.backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = _attn_ref(qr, kr, vr, scale)
    orf.backward(g.float())
    assert _rel(o, orf) < 1.5e-2
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        assert torch.isfinite(a.float()).all(), name
        assert _rel(a, b) < 2.5e-2, (name, _rel(a, b))


@pytest.mark.parametrize("T,H,sliced", [(256, 32, True), (200, 5, False), (1024, 32, False)])
def test_head_linear_kernels(T, H, sliced):
    """Per-head 64 x 64 maps (the absorbed MLA up-projections): output, input gradient and weight gradient against fp32,
    on an operand that is a column slice of a wider tensor (read in place), on a token count that is not a multiple of
    the tile, and on an odd head count (the last head pair of the weight-gradient kernel is half empty)."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    torch.manual_seed(T + H)
    base = torch.randn(2, T // 2, H, 128 if sliced else 64, device="cuda").bfloat16()
    x = (base[..., :64] if sliced else base).detach().requires_grad_()
    w = (torch.randn(H, 64, 64, device="cuda") * 0.2).bfloat16().requires_grad_()
    F_.reset_counters()
    y = F_.head_linear(x, w)
    assert F_.launch_counts().get("head_linear", 0) == 1 and not F_.fallback_counts()
    g = torch.randn_like(y)
    y.backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = torch.einsum("bshi,hoi->bsho", xr, wr)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    # the transposed-weight view used by the model (q . W_uk with W_uk stored [H, in, out])
    wt = (torch.randn(H, 64, 64, device="cuda") * 0.2).bfloat16()
    y2 = F_.head_linear(x.detach(), wt.transpose(1, 2))
    assert _rel(y2, torch.einsum("bshi,hio->bsho", x.detach().float(), wt.float())) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("B,S,C,k,sliced", [(2, 200, 136, 4, True), (1, 64, 64, 2, False), (3, 130, 72, 3, True)])
def test_causal_conv1d_silu_kernels(B, S, C, k, sliced):
    """Depthwise causal conv + SiLU, channels-last, read in place from a wider projection: output, input gradient, weight
    and bias gradients against the fp32 definition (segments of 64 tokens: S = 200 / 130 cross segment boundaries)."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops import reference as ref
    torch.manual_seed(S + C)
    base = torch.randn(B, S, C + 40 if sliced else C, device="cuda").bfloat16()
    x = (base[..., :C] if sliced else base).detach().requires_grad_()
    w = (torch.randn(C, 1, k, device="cuda") * 0.5).bfloat16().requires_grad_()
    b = (torch.randn(C, device="cuda") * 0.1).bfloat16().requires_grad_()
    F_.reset_counters()
    y = F_.causal_conv1d_silu(x, w, b)
    assert F_.launch_counts().get("causal_conv1d_silu", 0) == 1 and not F_.fallback_counts()
    g = torch.randn_like(y)
    y.backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = ref.causal_conv1d_silu(xr, wr.squeeze(1), br)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1.5e-2
    assert _rel(w.grad, wr.grad) < 1.5e-2
    assert _rel(b.grad, br.grad) < 1.5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["ssd", "noconv_ssd"])
def test_ssd_variant_mixers_on_gpu_match_the_cpu_fp32_module(variant):
    """The alternative SSM mixers (Mamba2-style SSD with the fused causal conv + SiLU kernel, and the no-conv variant with
    QK-norm / biases / data-dependent A / trapezoid / rotary state) in bf16 on the GPU against the same module in fp32 on
    the CPU: output and input gradient."""
    import copy
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.models.mamba_variants import build_variant_mixer
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.parallel.state import single_process_context
    cfg = nam56r_tiny(seq_length=128, mamba_variant=variant)
    pc = single_process_context()
    ref_mod = build_variant_mixer(cfg, pc, 1, dtype=torch.float32, seed=3, out_std=0.02)
    gpu_mod = copy.deepcopy(ref_mod).to("cuda").to(torch.bfloat16)
    for n, p in gpu_mod.named_parameters():                       # per-head fp32 parameters stay fp32, as in the model
        if p.dim() <= 1 and "norm" not in n and "conv" not in n:
            p.data = p.data.float()
    torch.manual_seed(5)
    x = torch.randn(2, 128, cfg.hidden_size) * 0.5
    g = torch.randn(2, 128, cfg.hidden_size) * 0.1
    xr = x.clone().requires_grad_()
    yr = ref_mod(xr)
    yr.backward(g)
    xg = x.cuda().bfloat16().requires_grad_()
    F_.reset_counters()
    yg = gpu_mod(xg)
    yg.backward(g.cuda().bfloat16())
    torch.cuda.synchronize()
    cu.check_errors()
    if variant == "ssd":
        assert F_.launch_counts().get("causal_conv1d_silu", 0) == 1
    assert _rel(yg.cpu(), yr) < 4e-2
    assert _rel(xg.grad.cpu(), xr.grad) < 6e-2
