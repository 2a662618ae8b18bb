"""Muon: q8 momentum arithmetic, normalisation plan, Newton-Schulz, and the optimizer path."""
import math

import pytest
import torch

from cppmega_b200.optim import muon
from cppmega_b200.ops import reference as ref


def test_q8_update_matches_dequant_math():
    torch.manual_seed(0)
    shape = (24, 100)                                    # 2400 values: last block is partial
    st = muon.QuantizedMomentum.zeros(shape, "cpu")
    m_ref = torch.zeros(shape)
    for step in range(4):
        g = torch.randn(shape)
        work = g.clone()
        ss = muon.qmuon_update_(st, work, beta=0.9)
        m_ref = 0.9 * m_ref + 0.1 * g
        # quantisation error: half a step of absmax/127 per block, compounding slowly
        assert (st.dequantize() - m_ref).abs().max() < 0.03 * m_ref.abs().max() * (step + 1)
        assert abs(ss.sum().item() - (m_ref ** 2).sum().item()) < 0.05 * (m_ref ** 2).sum().item()
        assert abs(work.norm().item() - 1.0) < 1e-3       # scaled to unit Frobenius norm
        m_ref = st.dequantize()                           # follow the quantised trajectory


def test_norm_plan_groups_fused_rows():
    plan = muon.build_norm_plan((12, 256), row_splits=(4, 4, 4))
    assert plan.num_groups == 3 and plan.block_group.tolist() == [0] * 4 + [1] * 4 + [2] * 4
    with pytest.raises(ValueError):
        muon.build_norm_plan((3, 100), row_splits=(1, 2))        # second segment starts mid-block
    st = muon.QuantizedMomentum.zeros((12, 256), "cpu")
    g = torch.randn(12, 256)
    g[4:8] *= 100.0
    work = g.clone()
    muon.qmuon_update_(st, work, beta=0.0, plan=plan)
    for lo in (0, 4, 8):                                           # every segment is normalised on its own
        assert abs(work[lo:lo + 4].norm().item() - 1.0) < 1e-3


def test_newton_schulz_orthogonalises():
    torch.manual_seed(1)
    G = torch.randn(64, 32)
    U = muon.newton_schulz(G, 6)
    sv = torch.linalg.svdvals(U.float())
    assert sv.max() < 1.3 and sv.min() > 0.5


def test_carrier_emission_roundtrip():
    torch.manual_seed(2)
    st = muon.QuantizedMomentum.zeros((8, 256), "cpu")
    muon.qmuon_update_(st, torch.randn(8, 256), beta=0.0)
    payload, scales = muon.emit_mxfp8_carrier(st)
    deq = ref.mxfp8_dequantize(payload.view(torch.float8_e4m3fn).view(8, 256), scales.view(8, 8))
    assert (deq - st.dequantize()).abs().max() < 0.07 * st.dequantize().abs().max()


@pytest.mark.parametrize("quantized", [False, True])
def test_muon_optimizer_trains_tiny_model(quantized):
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.parallel.state import single_process_context
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches
    mcfg = nam56r_tiny(seq_length=32)
    tcfg = TrainConfig(micro_batch_size=2, seq_length=32, dtype="fp32", log_interval=0,
                       optimizer=OptimizerConfig(optimizer="muon", lr=2e-3, weight_decay=0.0,
                                                 muon_quantized_momentum=quantized))
    tr = Trainer(mcfg, tcfg, single_process_context(), device=torch.device("cpu"))
    assert any(st["muon"] for st in tr.optimizer.state)
    batch = next(synthetic_batches(mcfg.vocab_size, 2, 32, 1, seed=0, pin=False))
    losses = [float(tr.train_step(batch)["loss"]) for _ in range(6)]
    assert all(math.isfinite(l) for l in losses) and losses[-1] < losses[0]


@pytest.mark.gpu
def test_q8_cuda_kernels_match_reference():
    torch.manual_seed(3)
    n_shape = (40, 200)
    for dtype in (torch.float32, torch.bfloat16):
        st_c = muon.QuantizedMomentum.zeros(n_shape, "cuda")
        st_r = muon.QuantizedMomentum.zeros(n_shape, "cpu")
        plan = muon.build_norm_plan(n_shape, device="cuda")
        for _ in range(3):
            g = torch.randn(n_shape).to(dtype)
            wc, wr = g.cuda().clone(), g.float().clone()
            ss_c = muon.qmuon_update_(st_c, wc, 0.95, plan)
            ss_r = muon.qmuon_update_(st_r, wr, 0.95)
            assert (st_c.data.cpu().int() - st_r.data.int()).abs().max() <= 1
            torch.testing.assert_close(st_c.absmax.cpu(), st_r.absmax, rtol=1e-2, atol=1e-6)
            torch.testing.assert_close(ss_c.cpu(), ss_r, rtol=2e-2, atol=1e-6)
            torch.testing.assert_close(wc.float().cpu(), wr, rtol=3e-2, atol=3e-3)
            st_r.data.copy_(st_c.data.cpu())
            st_r.absmax.copy_(st_c.absmax.cpu())
    payload, scales = muon.emit_mxfp8_carrier(muon.QuantizedMomentum(st_c.data[:8000 // 32 * 32], st_c.absmax, (8000,)))
    ref_p, ref_s = muon.emit_mxfp8_carrier(muon.QuantizedMomentum(st_c.data[:8000].cpu(), st_c.absmax.cpu(), (8000,)))
    assert (scales.cpu().int() - ref_s.int()).abs().max() == 0
    assert (payload.cpu() != ref_p).float().mean() < 0.01


def test_adam8bit_tracks_fp32_adamw():
    """8-bit state: the parameter trajectory stays close to fp32 AdamW, the state is 2 bytes per value, and elements
    masked out by ``active`` are left alone."""
    from cppmega_b200.optim.adam8bit import Adam8bitState, adam8bit_update
    from cppmega_b200.optim.adamw import adamw_reference
    torch.manual_seed(0)
    n = 1000                                              # last block is partial
    p8, p32 = torch.randn(n), None
    p32 = p8.clone()
    st = Adam8bitState.zeros(n, "cpu")
    m, v = torch.zeros(n), torch.zeros(n)
    out8, out32 = torch.zeros(n), torch.zeros(n)
    wd = torch.ones(n, dtype=torch.bool)
    active = torch.ones(n, dtype=torch.bool)
    active[100:200] = False
    frozen = p8[100:200].clone()
    for step in range(1, 21):
        g = torch.randn(n) * (0.1 + (torch.arange(n) % 7).float())
        bc1, bc2 = 1 - 0.9 ** step, 1 - 0.95 ** step
        adam8bit_update(p8, st, g, out8, wd, torch.ones(()), 1e-2, 0.9, 0.95, 1e-8, 0.01, bc1, bc2, active=active)
        adamw_reference(p32, m, v, g, out32, wd, torch.ones(()), 1e-2, 0.9, 0.95, 1e-8, 0.01, bc1, bc2)
    assert torch.equal(p8[100:200], frozen)
    keep = active
    assert (p8[keep] - p32[keep]).abs().max() < 0.03      # 20 steps of lr 1e-2: well inside one step's size
    m8, v8 = st.moments()
    assert ((m8 - m)[keep].abs() <= 0.02 * m.abs().max() + 1e-6).all()
    assert st.nbytes() < 2.1 * n


def test_muon_with_adam8bit_scalars_trains_tiny_model():
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.parallel.state import single_process_context
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches
    mcfg = nam56r_tiny(seq_length=32)
    tcfg = TrainConfig(micro_batch_size=2, seq_length=32, dtype="fp32", log_interval=0,
                       optimizer=OptimizerConfig(optimizer="muon", lr=2e-3, weight_decay=0.0, muon_scalar_optimizer="adam8bit",
                                                 muon_quantized_momentum=True))
    tr = Trainer(mcfg, tcfg, single_process_context(), device=torch.device("cpu"))
    assert all(st["a8"] is not None and st["v"] is None for st in tr.optimizer.state)
    batch = next(synthetic_batches(mcfg.vocab_size, 2, 32, 1, seed=0, pin=False))
    losses = [float(tr.train_step(batch)["loss"]) for _ in range(6)]
    assert all(math.isfinite(l) for l in losses) and losses[-1] < losses[0]
    sd = tr.optimizer.state_dict()
    tr.optimizer.load_state_dict(sd)                      # the 8-bit state round-trips through a checkpoint


@pytest.mark.gpu
def test_adam8bit_cuda_kernel_matches_definition():
    from cppmega_b200.optim.adam8bit import Adam8bitState, adam8bit_reference, adam8bit_update
    torch.manual_seed(1)
    n = 5000
    for gdt, odt in ((torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)):
        pc = torch.randn(n, device="cuda")
        pr = pc.cpu().clone()
        sc, sr = Adam8bitState.zeros(n, "cuda"), Adam8bitState.zeros(n, "cpu")
        oc, orf = torch.zeros(n, device="cuda", dtype=odt), torch.zeros(n, dtype=odt)
        wd = torch.rand(n) > 0.5
        act = torch.rand(n) > 0.1
        for step in range(1, 5):
            g = torch.randn(n).to(gdt)
            bc1, bc2 = 1 - 0.9 ** step, 1 - 0.95 ** step
            adam8bit_update(pc, sc, g.cuda(), oc, wd.cuda(), torch.full((), 0.5, device="cuda"), 1e-2, 0.9, 0.95, 1e-8, 0.1, bc1, bc2,
                            active=act.cuda())
            adam8bit_reference(pr, sr, g, orf, wd, torch.full((), 0.5), 1e-2, 0.9, 0.95, 1e-8, 0.1, bc1, bc2, active=act)
            assert (sc.m8.cpu().int() - sr.m8.int()).abs().max() <= 1
            assert (sc.v8.cpu().int() - sr.v8.int()).abs().max() <= 1
            torch.testing.assert_close(pc.cpu(), pr, rtol=1e-4, atol=1e-4)
            sr.m8.copy_(sc.m8.cpu()); sr.v8.copy_(sc.v8.cpu()); sr.am_m.copy_(sc.am_m.cpu()); sr.am_v.copy_(sc.am_v.cpu())
            pr.copy_(pc.cpu())
        # the low-precision copy is written for the active elements only
        torch.testing.assert_close(oc.float().cpu()[act], pc.to(odt).float().cpu()[act], rtol=0, atol=0)
        assert (oc.float().cpu()[~act] == 0).all()
