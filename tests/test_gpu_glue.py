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


@pytest.mark.parametrize("B,S,Skv", [(1, 300, 300), (2, 520, 520)])
def test_sparse_mla_kernels(B, S, Skv):
    from cppmega_b200.ops import reference as ref
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels4
    torch.manual_seed(0)
    Hq, D, TK, DV = 32, 128, 256, 64
    q = (torch.randn(B, S, Hq, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    kv = (torch.randn(B, Skv, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    # causal random selections: query s may pick keys <= s; the first positions see fewer than TK keys (-1 padding)
    idx = torch.full((B, S, TK), -1, dtype=torch.int32, device="cuda")
    for b in range(B):
        for s in range(S):
            n = min(TK, s + 1)
            perm = torch.randperm(s + 1, device="cuda")[:n]
            idx[b, s, :n] = perm.to(torch.int32)
    scale = D ** -0.5
    out = kernels4.sparse_mla(q, kv, idx, scale, DV)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    cu.check_errors()
    q2 = q.detach().float().requires_grad_()
    kv2 = kv.detach().float().requires_grad_()
    ref_out, _ = ref.sparse_mla(q2, kv2, idx, scale, DV)
    ref_out.backward(g.float())
    assert torch.isfinite(out.float()).all()
    assert _rel(out, ref_out) < 2e-2
    assert _rel(q.grad, q2.grad) < 3e-2
    assert _rel(kv.grad, kv2.grad) < 3e-2


def test_mimo_scan_reads_column_slices_in_place():
    """V and Z given as column slices of one wide projection output give the same result as packed copies."""
    from cppmega_b200.ops.cuda import kernels3
    from cppmega_b200.tools.ncu_cases import _scan_inputs
    B, S, H, G = 2, 128, 4, 2
    Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _scan_inputs(B, S, H, G)
    wide = torch.zeros(B, S, 2 * H * 64 + 72, dtype=torch.bfloat16, device="cuda")
    wide[..., :H * 64] = Z.reshape(B, S, -1)
    wide[..., H * 64:2 * H * 64] = V.reshape(B, S, -1)
    Zs = wide[..., :H * 64].view(B, S, H, 64)
    Vs = wide[..., H * 64:2 * H * 64].view(B, S, H, 64)
    assert not Vs.is_contiguous() and kernels3.token_strided(Vs)[1] == wide.shape[-1]
    y0, _, _ = kernels3.mimo_fwd_raw(Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D)
    y1, _, _ = kernels3.mimo_fwd_raw(Qn, Kn, Vs, Zs, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D)
    torch.cuda.synchronize()
    assert torch.equal(y0, y1)


@pytest.mark.parametrize("B,S,topk", [(2, 512, 256), (1, 1100, 256), (1, 8448, 256)])   # the last one: 512-thread select
def test_indexer_topk_kernels(B, S, topk):
    from cppmega_b200.ops import reference as ref
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops.cuda import kernels4
    torch.manual_seed(0)
    q = torch.randn(B, S, 32, 64, device="cuda").bfloat16()
    k = torch.randn(B, S, 64, device="cuda").bfloat16()
    w = torch.randn(B, S, 32, device="cuda") * 0.1
    idx = kernels4.indexer_topk(q, k, w, topk)
    torch.cuda.synchronize()
    cu.check_errors()
    sc = ref.indexer_scores(q, k, w)
    causal = torch.ones(S, S, dtype=torch.bool, device="cuda").tril()
    sc = sc.masked_fill(~causal, float("-inf"))
    ref_idx = ref.indexer_topk(q, k, w, topk)
    for b in range(B):
        for i in (0, 1, topk - 2, topk - 1, topk, topk + 1, S // 2, S - 1):
            got = idx[b, i]
            got_valid = got[got >= 0]
            n = min(i + 1, topk)
            assert got_valid.numel() == n and got_valid.unique().numel() == n and int(got_valid.max()) <= i
            # same selection up to ties: the smallest selected score is not below the largest rejected one
            sel = sc[b, i, got_valid.long()]
            want = sc[b, i, ref_idx[b, i][ref_idx[b, i] >= 0].long()]
            assert abs(sel.min().item() - want.min().item()) <= 2e-2 * max(1.0, abs(want.min().item()))
            assert abs(sel.sum().item() - want.sum().item()) <= 2e-2 * max(1.0, abs(want.sum().item()))


def test_mxfp8_quantize_kernels_match_reference():
    from cppmega_b200.ops import reference as ref
    from cppmega_b200.ops.cuda import mxfp8
    torch.manual_seed(0)
    x = (torch.randn(96, 256, device="cuda") * torch.logspace(-3, 2, 256, device="cuda")).bfloat16()
    x[5, 32:64] = 0                                             # an all-zero block takes the neutral scale
    r = mxfp8.quantize_rowwise(x)
    pay_ref, sc_ref = ref.mxfp8_quantize(x, axis=-1)
    assert torch.equal(r.scales, sc_ref)
    assert torch.equal(r.payload, pay_ref.view(torch.uint8))
    c = mxfp8.quantize_colwise(x)
    pay_c, sc_c = ref.mxfp8_quantize(x, axis=0)                 # blocks along rows, [rows, cols] / [rows/32, cols]
    assert torch.equal(c.scales, sc_c.t().contiguous())
    assert torch.equal(c.payload, pay_c.view(torch.uint8).t().contiguous())
    deq = mxfp8.dequantize(r)
    torch.testing.assert_close(deq.float(), ref.mxfp8_dequantize(pay_ref, sc_ref).bfloat16().float(), rtol=0, atol=0)
    assert ((deq.float() - x.float()).abs() <= 0.07 * x.float().abs() + 1e-6).all()       # 3 mantissa bits
    sw = mxfp8.swizzle_scales(r.scales)
    assert torch.equal(sw, ref.swizzle_scales_128x4(r.scales))
    both_r, both_c = mxfp8.quantize_both(x)
    assert torch.equal(both_r.payload, r.payload) and torch.equal(both_r.scales, r.scales)
    assert torch.equal(both_c.payload, c.payload) and torch.equal(both_c.scales, c.scales)
    assert torch.equal(both_r.swizzled(), sw) and torch.equal(both_c.swizzled(), ref.swizzle_scales_128x4(c.scales))
    wide = (torch.randn(64, 544, device="cuda") * 3).bfloat16()          # 2 full column tiles + a 32-wide tail
    wr, wc = mxfp8.quantize_both(wide)
    assert torch.equal(wr.payload, mxfp8.quantize_rowwise(wide).payload) and torch.equal(wc.payload, mxfp8.quantize_colwise(wide).payload)
    assert torch.equal(wc.scales, mxfp8.quantize_colwise(wide).scales)
    # the quantise kernels can write the tile order themselves
    assert torch.equal(mxfp8.quantize_rowwise(x, True).swizzled(), sw)
    assert torch.equal(mxfp8.quantize_colwise(x, True).swizzled(), ref.swizzle_scales_128x4(c.scales))


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (300, 200, 160), (128, 256, 4096), (1024, 768, 1024)])
def test_mxfp8_block_scaled_gemm(M, N, K):
    """tcgen05 block-scaled product against the fp32 product of the dequantised operands."""
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops.cuda import mxfp8
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 1, K, device="cuda")).bfloat16()
    b = (torch.randn(N, K, device="cuda") * torch.logspace(1, -2, N, device="cuda")[:, None]).bfloat16()
    aq, bq = mxfp8.quantize_rowwise(a), mxfp8.quantize_rowwise(b)
    want = mxfp8.dequantize(aq).float() @ mxfp8.dequantize(bq).float().t()
    before = F_.launch_counts().get("mxfp8_gemm", 0)
    got = mxfp8.gemm_mxfp8(aq, bq)
    assert F_.launch_counts().get("mxfp8_gemm", 0) == before + 1
    assert got.dtype == torch.bfloat16 and _rel(got, want) < 5e-3
    acc = torch.randn(M, N, device="cuda")
    got32 = mxfp8.gemm_mxfp8(aq, bq, out=acc.clone(), accumulate=True)
    assert _rel(got32, want + acc) < 1e-5
    acc16 = torch.randn(M, N, device="cuda").bfloat16()
    got16 = mxfp8.gemm_mxfp8(aq, bq, out=acc16.clone(), accumulate=True)
    assert _rel(got16, want + acc16.float()) < 5e-3
    torch.testing.assert_close(mxfp8.gemm_mxfp8(aq, bq, out_dtype=torch.float32), want, rtol=1e-4, atol=1e-3 * want.abs().max().item())


def test_mxfp8_linear_matches_quantised_reference():
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops import reference as ref
    torch.manual_seed(1)
    x = (torch.randn(4, 64, 256, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(128, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    F_.set_precision_recipe("mxfp8")
    try:
        y = F_.linear(x, w)
        g = torch.randn_like(y)
        y.backward(g)
    finally:
        F_.set_precision_recipe("bf16")
    q = lambda t, ax: ref.mxfp8_dequantize(*ref.mxfp8_quantize(t, axis=ax), axis=ax)
    x2, g2 = x.detach().reshape(-1, 256), g.reshape(-1, 128)
    y_ref = q(x2, -1) @ q(w.detach(), -1).t()
    dx_ref = q(g2, -1) @ q(w.detach(), 0)
    dw_ref = q(g2, 0).t() @ q(x2, 0)
    assert _rel(y.reshape(-1, 128), y_ref) < 1e-2
    assert _rel(x.grad.reshape(-1, 256), dx_ref) < 1e-2
    assert _rel(w.grad, dw_ref) < 1e-2
    # and it stays close to the unquantised product
    assert _rel(y.reshape(-1, 128), x2.float() @ w.detach().float().t()) < 6e-2


@pytest.mark.parametrize("score_fn,norm", [("sigmoid", True), ("softmax", True), ("softmax", False)])
def test_router_topk_kernel(score_fn, norm):
    from cppmega_b200.ops import reference as ref
    from cppmega_b200.ops.cuda import kernels4
    torch.manual_seed(0)
    T, E, K = 777, 16, 4
    logits = torch.randn(T, E, device="cuda").requires_grad_()
    bias = torch.randn(E, device="cuda") * 0.1
    probs, ids, scores = kernels4.router_topk(logits, K, score_fn, bias, norm)
    gp, gs = torch.randn_like(probs), torch.randn_like(scores) * 0.1
    (probs * gp).sum().add((scores * gs).sum()).backward()
    l2 = logits.detach().clone().requires_grad_()
    p2, i2, s2 = ref.router_topk(l2, K, score_fn, bias, norm)
    (p2 * gp).sum().add((s2 * gs).sum()).backward()
    assert torch.equal(ids.sort(-1).values, i2.sort(-1).values)
    torch.testing.assert_close(scores, s2, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(probs.sort(-1).values, p2.sort(-1).values, rtol=1e-4, atol=1e-6)
    assert _rel(logits.grad, l2.grad) < 1e-3


def test_ngram_hash_embed_kernel():
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.models.embedding import NgramHashEmbedding
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops import reference as ref
    cfg = nam56r_tiny()
    torch.manual_seed(0)
    emb = NgramHashEmbedding(cfg.hidden_size, cfg.ngram_hash, dtype=torch.bfloat16).cuda()
    ids = torch.randint(0, cfg.vocab_size, (3, 50), device="cuda")
    args = (emb.hash_mults, emb.hash_bias, emb.table_sizes_t, emb.table_offsets, emb.order_for_table)
    table = emb.unified_table.weight
    out = F_.ngram_hash_embed(ids, table, *args)
    want = ref.ngram_hash_embed(ids, table, *args)
    assert torch.equal(out, want)
    g = torch.randn_like(out)
    (gk,) = torch.autograd.grad(out, table, g)
    (gr,) = torch.autograd.grad(want, table, g)
    assert _rel(gk, gr) < 1e-2


def test_rope_kernel_on_slices():
    from cppmega_b200.ops import reference as ref
    from cppmega_b200.ops.cuda import kernels4
    torch.manual_seed(0)
    B, S, H, D = 2, 70, 4, 64
    wide = torch.randn(B, S, H, 2 * D, device="cuda").bfloat16().requires_grad_()
    cos, sin = ref.rope_tables(S, D, 5e5, device="cuda")
    x = wide[..., D:]                                   # column slice: rotated in place of a copy
    y = kernels4.apply_rope(x, cos, sin)
    g = torch.randn_like(y)
    (gw,) = torch.autograd.grad(y, wide, g)
    w2 = wide.detach().clone().requires_grad_()
    y2 = ref.apply_rope(w2[..., D:], cos, sin)
    (gw2,) = torch.autograd.grad(y2, w2, g)
    assert _rel(y, y2) < 1e-2 and _rel(gw, gw2) < 1e-2
    k = torch.randn(B, S, D, device="cuda").bfloat16()
    assert _rel(kernels4.apply_rope(k, cos, sin), ref.apply_rope(k, cos, sin)) < 1e-2


def test_fast_strided_copy_and_cat_split_helpers():
    from cppmega_b200.models.common import cat_last_dim, split_last_dim
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops.cuda import fast_contiguous, fast_copy_
    torch.manual_seed(0)
    packed = torch.randn(3, 130, 24960, device="cuda").bfloat16()
    view = packed[..., 8192:8192 + 4096].reshape(3, 130, 8, 4, 128).permute(0, 1, 3, 2, 4)        # 5-D, 256-byte runs
    n0 = F_.launch_counts().get("strided_copy", 0)
    assert torch.equal(fast_contiguous(view), view.contiguous())
    dst = torch.zeros(3, 130, 24960, device="cuda", dtype=torch.bfloat16)
    src = torch.randn(3, 130, 64, device="cuda").bfloat16()
    fast_copy_(dst[..., 128:192], src)
    assert torch.equal(dst[..., 128:192], src) and dst[..., :128].abs().sum() == 0 and dst[..., 192:].abs().sum() == 0
    exp = torch.randn(3, 130, 1, 64, device="cuda").bfloat16().expand(3, 130, 32, 64)             # stride-0 source
    assert torch.equal(fast_contiguous(exp), exp.contiguous())
    assert F_.launch_counts().get("strided_copy", 0) == n0 + 3
    wide = packed[..., 8192:8192 + 4096]                                                          # 8 KB runs: warp-strided variant
    assert torch.equal(fast_contiguous(wide), wide.contiguous())
    odd = torch.randn(5, 7, 9, device="cuda").bfloat16()[..., 1:6]                                # 10-byte runs: library path
    assert torch.equal(fast_contiguous(odd), odd.contiguous())
    # autograd of the helpers against torch.cat / slicing
    a = torch.randn(2, 50, 32, 64, device="cuda").bfloat16().requires_grad_()
    b = torch.randn(2, 50, 1, 64, device="cuda").bfloat16().requires_grad_()
    x = torch.randn(2, 50, 32, 192, device="cuda").bfloat16().requires_grad_()
    x1, x2 = split_last_dim(x, (128, 64))
    y = cat_last_dim([a, b.expand(2, 50, 32, 64), x2])
    g = torch.randn_like(y)
    (y * g).sum().add((x1 * x1).sum()).backward()
    a2, b2, xx = (t.detach().clone().requires_grad_() for t in (a, b, x))
    y2 = torch.cat([a2, b2.expand(2, 50, 32, 64), xx[..., 128:]], dim=-1)
    (y2 * g).sum().add((xx[..., :128] * xx[..., :128]).sum()).backward()
    assert torch.equal(y, y2)
    for p, q in ((a, a2), (b, b2), (x, xx)):
        torch.testing.assert_close(p.grad.float(), q.grad.float(), rtol=2e-2, atol=2e-2)


def test_mxfp8_grouped_expert_gemms():
    """Block-scaled grouped GEMMs (forward / dgrad / per-expert wgrad) against fp32 products of the dequantised operands."""
    from cppmega_b200.ops.cuda import mxfp8
    torch.manual_seed(3)
    E, N, K = 3, 384, 256
    tile_expert = torch.tensor([0, 0, 2, -1, 1, 2], dtype=torch.int32, device="cuda")      # 6 tiles of 128 rows, one unused
    rows = tile_expert.numel() * 128
    x = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(E, N, K, device="cuda") * 0.1).bfloat16()
    xq = mxfp8.quantize_rowwise(x, True)
    xd = mxfp8.dequantize(xq).float()
    te = tile_expert.repeat_interleave(128).long()
    live = te >= 0
    # forward: y[r] = x[r] . W[e(r)]^T
    wq = mxfp8.quantize_expert_weights(w, False)
    wd = mxfp8.dequantize(wq).float().view(E, N, K)
    y = mxfp8.grouped_rows_mxfp8(xq, wq, tile_expert, E, N, False)
    want = torch.einsum("rk,rnk->rn", xd[live], wd[te[live]])
    assert _rel(y[live], want) < 5e-3
    # dgrad: dx[r] = g[r] . W[e(r)]  (reduction over N)
    g = (torch.randn(rows, N, device="cuda") * 0.5).bfloat16()
    gq = mxfp8.quantize_rowwise(g, True)
    wtq = mxfp8.quantize_expert_weights(w, True)                                          # [K, E*N]
    wtd = mxfp8.dequantize(wtq).float().view(K, E, N).permute(1, 2, 0)                    # [E, N, K]
    dx = mxfp8.grouped_rows_mxfp8(gq, wtq, tile_expert, E, K, True)
    want = torch.einsum("rn,rnk->rk", mxfp8.dequantize(gq).float()[live], wtd[te[live]])
    assert _rel(dx[live], want) < 5e-3
    # wgrad: dW[e] = g_e^T x_e over expert e's rows; expert segments are contiguous in the sorted layout
    order = torch.tensor([0, 1, 4, 2, 5], device="cuda")                                   # tiles sorted by expert: 0,0,1,2,2
    xs = x.view(-1, 128, K)[order].reshape(-1, K).contiguous()
    gs = g.view(-1, 128, N)[order].reshape(-1, N).contiguous()
    seg = torch.tensor([0, 256, 384, 640], dtype=torch.int32, device="cuda")
    g_t, x_t = mxfp8.quantize_colwise(gs, True), mxfp8.quantize_colwise(xs, True)
    dw = mxfp8.grouped_wgrad_mxfp8(g_t, x_t, seg, E)
    gd, xdt = mxfp8.dequantize(g_t).float(), mxfp8.dequantize(x_t).float()                # [N, R], [K, R]
    for e in range(E):
        s0, s1 = int(seg[e]), int(seg[e + 1])
        assert _rel(dw[e], gd[:, s0:s1] @ xdt[:, s0:s1].t()) < 5e-3, e
    acc = torch.randn(E, N, K, device="cuda")
    dw32 = mxfp8.grouped_wgrad_mxfp8(g_t, x_t, seg, E, out=acc.clone(), accumulate=True)
    assert _rel(dw32 - acc, dw.float()) < 1e-2
    empty = torch.tensor([0, 256, 256, 640], dtype=torch.int32, device="cuda")             # expert 1 without tokens
    assert mxfp8.grouped_wgrad_mxfp8(g_t, x_t, empty, E)[1].abs().sum() == 0


@pytest.mark.parametrize("ep,ep_rank", [(1, 0), (4, 2)])
def test_moe_plan_kernels_match_library_ops(ep, ep_rank):
    from cppmega_b200.parallel.fused_moe import MoEPlan, TILE
    torch.manual_seed(ep)
    T, k, E = 3000, 4, 16
    ids = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)])          # distinct experts per token
    ids[:200, 0] = 5                                                                       # some skew
    others = torch.randint(0, 900, (ep, E), device="cuda")

    def gather(counts):
        allc = others.clone()
        allc[ep_rank] = counts
        return allc

    cap = ((T * k * 4 + 16 * TILE) // TILE) * TILE
    plans = []
    for flag in (False, True):
        MoEPlan.use_kernels = flag
        try:
            plans.append(MoEPlan(ids, E, ep, ep_rank, None, cap, gather if ep > 1 else None))
        finally:
            MoEPlan.use_kernels = True
    a, b = plans
    for name in ("dest_row", "dest_rank", "token_of_copy", "seg_start_local", "tot_local", "seg_offsets", "tile_expert", "counts_global"):
        assert torch.equal(getattr(a, name).long(), getattr(b, name).long()), name
    assert int(a.rows_used) == int(b.rows_used) and (a.T, a.k) == (b.T, b.k)


def test_moe_transport_skips_and_reports_rows_beyond_capacity():
    """Receive buffer smaller than the routing needs (EP 1, so the "peer" is this GPU): push drops the copies that do
    not fit, the pulls treat them as zero, no address beyond the buffer is formed, and the error word says so."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.parallel import fused_moe as fm
    cu.check_errors()
    torch.manual_seed(0)
    T, k, E, H = 512, 2, 4, 256
    ids = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)])
    cap = 4 * fm.TILE                                          # T*k = 1024 copies need >= 1024 rows
    plan = fm.MoEPlan(ids, E, 1, 0, None, cap, None)
    heap = fm._LocalHeap()
    x = torch.randn(T, H, device="cuda").bfloat16()
    guard = 64
    buf = torch.full((cap + guard, H), 7.0, device="cuda", dtype=torch.bfloat16)    # rows past `cap` must stay untouched
    dst = buf[:cap]
    fm._push(heap, x, plan, dst)
    torch.cuda.synchronize()
    assert (buf[cap:] == 7.0).all()
    with pytest.raises(cu.KernelError, match="bad argument"):
        cu.check_errors()
    w = torch.ones(T * k, device="cuda")
    y = fm._pull_combine(heap, dst, plan, w, H, torch.bfloat16)
    d = fm._pull_rowdot(heap, dst, plan, x)
    torch.cuda.synchronize()
    with pytest.raises(cu.KernelError, match="bad argument"):
        cu.check_errors()
    keep = (plan.dest_row < cap).view(T, k)
    expect = (x.float() * keep.sum(1, keepdim=True)).bfloat16()     # every kept copy returns the token itself
    assert _rel(y, expect) < 1e-2
    assert (d.view(T, k)[~keep] == 0).all()


def _tensorwise_q(t):
    """fp32 restatement of the tensorwise FP8 recipe: one power-of-two scale from the tensor's amax, E4M3 rounding."""
    from cppmega_b200.ops import reference as ref
    sb = ref.e8m0_from_amax(t.float().abs().max().reshape(1)).float()
    mult = torch.exp2(127.0 - sb)
    return (t.float() * mult).to(torch.float8_e4m3fn).float() / mult


def test_tensorwise_fp8_quantisers_and_linear():
    """The tensorwise recipe: every scale byte of a tensor is the same, the payload is the E4M3 rounding under that one
    scale, both orientations agree, and the linear's three products match the fp32 products of the rounded operands."""
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.ops.cuda import mxfp8
    torch.manual_seed(4)
    x = (torch.randn(96, 256, device="cuda") * 2.5).bfloat16()
    am = mxfp8.tensor_amax(x)
    assert float(am) == float(x.float().abs().max())
    r = mxfp8.quantize_rowwise(x, tensorwise=True)
    assert r.scales.unique().numel() == 1
    assert torch.equal(mxfp8.dequantize(r).float(), _tensorwise_q(x).bfloat16().float())
    br, bc = mxfp8.quantize_both(x, True, am)
    assert torch.equal(br.payload, r.payload) and bc.scales.unique().numel() == 1
    assert torch.equal(bc.payload, r.payload.t().contiguous())            # same scale: the transposed copy is a pure transpose
    c = mxfp8.quantize_colwise(x, tensorwise=am)
    assert torch.equal(c.payload, bc.payload) and torch.equal(c.scales, bc.scales)

    xx = (torch.randn(4, 64, 256, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(128, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    with F_.precision_scope("tensorwise"):
        y = F_.linear(xx, w)
    g = torch.randn_like(y)
    y.backward(g)                                                         # outside the scope: the op remembers its recipe
    assert F_.precision_recipe() == "bf16"
    x2, g2 = xx.detach().reshape(-1, 256), g.reshape(-1, 128)
    q = _tensorwise_q
    assert _rel(y.reshape(-1, 128), q(x2) @ q(w.detach()).t()) < 1e-2
    assert _rel(xx.grad.reshape(-1, 256), q(g2) @ q(w.detach())) < 1e-2
    assert _rel(w.grad, q(g2).t() @ q(x2)) < 1e-2
    assert _rel(y.reshape(-1, 128), x2.float() @ w.detach().float().t()) < 6e-2


@pytest.mark.gpu
@pytest.mark.parametrize("grad_dtype", [None, torch.float32, torch.bfloat16])
def test_embedding_kernels_gather_and_scatter_add(grad_dtype):
    """Row gather, and the backward that adds gradient rows with vector atomics: into a fresh tensor (``None``) or straight
    into the parameter's flat gradient buffer (fp32 / bf16), where a second use of the same table accumulates."""
    from cppmega_b200.ops import cuda as cu
    from cppmega_b200.ops import functional as F_
    torch.manual_seed(0)
    V, H = 1000, 256
    w = torch.nn.Parameter(torch.randn(V, H, device="cuda").bfloat16())
    ids = torch.randint(0, V, (3, 517), device="cuda")
    ids[0, :40] = 7                                            # repeated token: colliding atomics
    g = torch.randn(3, 517, H, device="cuda").bfloat16()
    if grad_dtype is not None:
        w.main_grad = torch.zeros(V, H, device="cuda", dtype=grad_dtype)
        w.fuse_wgrad_accumulation = True
    F_.reset_counters()
    y = F_.embedding(ids, w)
    assert torch.equal(y, torch.nn.functional.embedding(ids, w))
    (y * 1.0).backward(g)
    y2 = F_.embedding(ids[:1], w)                              # second use of the table in the same step
    y2.backward(g[:1])
    torch.cuda.synchronize()
    cu.check_errors()
    assert F_.launch_counts().get("embedding", 0) == 2 and F_.launch_counts().get("embedding_bwd", 0) == 2
    wr = w.detach().float().requires_grad_()
    (torch.nn.functional.embedding(ids, wr) * g.float()).sum().backward()
    (torch.nn.functional.embedding(ids[:1], wr) * g[:1].float()).sum().backward()
    if grad_dtype is None:
        got = w.grad.float()
    else:
        assert getattr(w, "grad_added_to_main_grad", False)
        got = w.main_grad.float()
    tol = 2e-2 if grad_dtype != torch.float32 else 1e-3
    assert (got - wr.grad).norm() / wr.grad.norm() < tol
