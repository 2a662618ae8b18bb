"""The allocation-free MIMO scan entry point (`cm_mimo_scan_fwd_static`), called through its exported C symbol.

Collected last on purpose: it must give the same answer alone and after every other GPU test has used the library.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = -20


def _symbol():
    from cppmega_b200.ops import cuda as cu
    fn = cu.lib().cm_mimo_scan_fwd_static
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp] * 16 + [i32] * 5 + [vp, vp]
    fn.restype = i32
    return fn


def _inputs(B, S, H, G, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    N, P, R = 128, 64, 4
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    Qn = (rn(B, S, G, R, N) * 0.5).bfloat16()
    Kn = (rn(B, S, G, R, N) * 0.5).bfloat16()
    V, Z = rn(B, S, H, P).bfloat16(), rn(B, S, H, P).bfloat16()
    DT = torch.rand(B, H, S, device="cuda", generator=g) * 0.1
    ADT = -DT * torch.rand(B, H, S, device="cuda", generator=g)
    Trap = rn(B, H, S)
    Qb, Kb = rn(H, R, N) * 0.1, rn(H, R, N) * 0.1
    Psi, Zeta, Phi = rn(H, R, P), rn(H, R, P), rn(H, R, P)
    ang = rn(B, S, H, N // 4)
    D = rn(H)
    return [Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D]


def _call_static(fn, args, B, S, H, G):
    from cppmega_b200.ops import cuda as cu
    y = torch.empty(B, S, H, 64, dtype=torch.bfloat16, device="cuda")
    final = torch.empty(B, H, 128, 64, dtype=torch.float32, device="cuda")
    rc = fn(*[t.data_ptr() for t in args], final.data_ptr(), y.data_ptr(), B, S, H, G, 128,
            cu.err_word(y.device).data_ptr(), cu.stream_ptr())
    return rc, y, final


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_static_scratch_matches_regular_entry_point_twice():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels3
    fn = _symbol()
    B, S, H, G = 1, 1024, 4, 2                      # 128 chunks of the 256 the fixed array holds
    for seed in (11, 12):                           # two calls in a row, different data: stale contents must not leak
        args = _inputs(B, S, H, G, seed)
        y_ref, _, _, f_ref = kernels3.mimo_fwd_raw(*args, want_state=True)
        rc, y, final = _call_static(fn, args, B, S, H, G)
        assert rc == 0
        torch.cuda.synchronize()
        cu.check_errors()
        assert torch.isfinite(y.float()).all()
        # both entry points run the same kernels on the same inputs: bit-for-bit, so a stale word of the shared array
        # leaking into a result of any size shows up
        assert torch.equal(y, y_ref)
        assert torch.equal(final, f_ref)


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_static_scratch_rejects_oversize_and_full_size_fits():
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels3
    fn = _symbol()
    args = _inputs(1, 4096, 4, 2, 5)                # 512 chunks > 256: refused before any launch
    rc, _, _ = _call_static(fn, args, 1, 4096, 4, 2)
    assert rc == TOO_LARGE
    args = _inputs(2, 1024, 4, 4, 6)                # exactly 256 chunks
    y_ref, _, _ = kernels3.mimo_fwd_raw(*args)
    rc, y, _ = _call_static(fn, args, 2, 1024, 4, 4)
    assert rc == 0
    torch.cuda.synchronize()
    cu.check_errors()
    assert torch.equal(y, y_ref)
