"""tcgen05 GEMM family against fp32 PyTorch matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.fixture(scope="module")
def cu():
    from cppmega_b200.ops import cuda
    return cuda


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 776, 520), (4096, 4096, 1024),
                                   (8, 16, 8), (304, 24960, 256)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(cu, M, N, K, a_mn, b_mn):
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(N, K, device="cuda").bfloat16()
    ref = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = cu.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    cu.check_errors()
    assert out.shape == (M, N)
    assert _rel(out, ref) < 6e-3


def test_gemm_fp32_accumulate(cu):
    torch.manual_seed(1)
    A = torch.randn(512, 320, device="cuda").bfloat16()
    B = torch.randn(384, 320, device="cuda").bfloat16()
    C0 = torch.randn(512, 384, device="cuda")
    out = C0.clone()
    cu.gemm(A, B, out=out, accumulate=True)
    cu.check_errors()
    ref = C0 + A.float() @ B.float().t()
    assert _rel(out, ref) < 1e-4
    out2 = torch.empty(512, 384, device="cuda")
    cu.gemm(A, B, out=out2)
    assert _rel(out2, A.float() @ B.float().t()) < 1e-4


def test_linear_autograd(cu):
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = cu.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    cu.check_errors()
    assert _rel(y, yr) < 6e-3
    assert _rel(x.grad, xr.grad) < 6e-3
    assert _rel(w.grad, wr.grad) < 6e-3


@pytest.mark.parametrize("counts", [[128, 0, 300, 5], [1, 1, 1, 1], [0, 0, 0, 700], [257, 129, 64, 63]])
def test_grouped_experts(cu, counts):
    from cppmega_b200.ops.cuda import extra
    from cppmega_b200.ops import reference as ref
    torch.manual_seed(3)
    E, H, Fh = len(counts), 256, 192
    T = sum(counts)
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w1 = (torch.randn(E, 2 * Fh, H, device="cuda") * 0.05).bfloat16().requires_grad_()
    w2 = (torch.randn(E, H, Fh, device="cuda") * 0.05).bfloat16().requires_grad_()
    cnt = torch.tensor(counts, device="cuda")
    y = extra.moe_experts(x, w1, w2, cnt)
    g = torch.randn_like(y)
    y.backward(g)
    cu.check_errors()
    xr, w1r, w2r = (t.detach().float().requires_grad_() for t in (x, w1, w2))
    h = ref.grouped_gemm(xr, w1r.transpose(1, 2), counts)
    h = ref.swiglu(h)
    yr = ref.grouped_gemm(h, w2r.transpose(1, 2), counts)
    yr.backward(g.float())
    assert _rel(y, yr) < 1.5e-2
    assert _rel(x.grad, xr.grad) < 1.5e-2
    assert _rel(w1.grad, w1r.grad) < 1.5e-2
    assert _rel(w2.grad, w2r.grad) < 1.5e-2


def test_linear_fp32out_router_shape():
    from cppmega_b200.ops import cuda as cu
    torch.manual_seed(0)
    x = (torch.randn(3000, 512, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(16, 512, device="cuda") * 0.05).requires_grad_()
    y = cu.linear_fp32out(x, w)
    assert y.dtype == torch.float32
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().clone().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(y, yr) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    assert rel(w.grad, wr.grad) < 2e-2
    assert w.grad.dtype == torch.float32
