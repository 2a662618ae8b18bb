"""The PyTorch definitions that every kernel of this package is tested against, pinned to the reference project's own
pure-PyTorch oracles.  The reference package is imported unmodified from ``baseline/_ref`` (``pip install --target``
of the reference tree); the tests are skipped when it is not installed."""
import math
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "cppmega")), reason="reference package not installed")


def _ref(module: str):
    import importlib
    if REF not in sys.path:
        sys.path.insert(0, REF)
    return importlib.import_module(module)


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))


# ---- Mamba3 MIMO scan -------------------------------------------------------------------------------------------

def _mimo_inputs(B, S, H, G, N, P, R, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=dtype)
    Q, K = rn(B, S, R, G, N) * 0.5, rn(B, S, R, G, N) * 0.5
    V, Z = rn(B, S, H, P), rn(B, S, H, P)
    DT = torch.rand(B, H, S, generator=g, dtype=dtype) * 0.1 + 0.001
    ADT = -DT * (torch.rand(B, H, S, generator=g, dtype=dtype) * 4 + 0.1)
    Trap = rn(B, H, S)
    Qb, Kb = rn(H, R, N) * 0.3, rn(H, R, N) * 0.3
    Psi, Zeta, Phi = rn(H, R, P) * 0.5, rn(H, R, P) * 0.5, rn(H, R, P) * 0.5
    ang = (rn(B, S, H, N // 4) * 0.2).cumsum(1)
    D = rn(H)
    return Q, K, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D


def _prefix_sums(ADT, cs):
    """Per-chunk inclusive cumsum, sum after t, and segsum[i, j] = sum_{j < s <= i} ADT[s]."""
    B, H, S = ADT.shape
    a = ADT.view(B, H, S // cs, cs)
    cum = a.cumsum(-1)
    rev = cum[..., -1:] - cum
    seg = cum.unsqueeze(-1) - cum.unsqueeze(-2)
    return cum.reshape(B, H, S), rev.reshape(B, H, S), seg


def test_mimo_forward_matches_reference_within_a_chunk():
    """One chunk (S == chunk size): the output depends on everything except the carry into a later chunk."""
    fwd = _ref("cppmega.megatron.cute_dsl_mimo.cute_dsl_mimo_fwd").cute_dsl_mimo_fwd
    from cppmega_b200.ops import mimo_scan_ref as R
    B, S, H, G, N, P, Rk = 2, 16, 4, 2, 32, 16, 4
    Q, K, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _mimo_inputs(B, S, H, G, N, P, Rk, 0)
    cum, rev, seg = _prefix_sums(ADT, 16)
    y_ref, _, _ = fwd(Q, K, V, Qb, Kb, Psi, Phi, Z, D, Zeta, ang, cum, rev, DT, Trap, seg, 16, 4, torch.float32)
    y_seq = R.mimo_scan_sequential(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z, 4)
    y_chk = R.mimo_scan_chunked(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D, Z, 4, 16)
    assert _rel(y_seq, y_ref) < 1e-5 and _rel(y_chk, y_ref) < 1e-5
    # un-reduced output (Phi None) and no gate
    y_ref2, _, _ = fwd(Q, K, V, Qb, Kb, Psi, None, None, D, None, ang, cum, rev, DT, Trap, seg, 16, 4, torch.float32)
    y_seq2 = R.mimo_scan_sequential(Q, K, V, ADT, DT, Trap, Qb, Kb, Psi, None, None, ang, D, None, 4)
    assert y_seq2.shape == y_ref2.shape and _rel(y_seq2, y_ref2) < 1e-5


def test_mimo_backward_matches_reference_across_chunks():
    """Autograd through this package's definition against the reference's restatement of the backward kernel, two
    chunks, G < H.  The reference's backward carries the state gradient through the trapezoid-scaled K, i.e. the state
    update consumes the scaled K: the multi-chunk semantics this package implements in forward and backward."""
    bwd = _ref("cppmega.megatron.cute_dsl_mimo.full_bwd_bwd_epilogue").full_bwd_bwd_pytorch
    from cppmega_b200.ops import mimo_scan_ref as R
    B, S, H, G, N, P, Rk, cs = 1, 32, 4, 2, 32, 32, 4, 16          # the reference restatement needs N == P
    Q, K, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, ang, D = _mimo_inputs(B, S, H, G, N, P, Rk, 1)
    leaves = [t.clone().requires_grad_() for t in (Q, K, V, Psi, ang)]
    Ql, Kl, Vl, Psil, angl = leaves
    y = R.mimo_scan_sequential(Ql, Kl, Vl, ADT, DT, Trap, Qb, Kb, Psil, None, Phi, angl, D, None, 4)
    dout = torch.randn(y.shape, generator=torch.Generator().manual_seed(5))
    y.backward(dout)
    # inputs the reference's backward takes from its forward: chunk start states and the per-token q.k blocks
    q, k = R._prep(Q, K, V, Qb, Kb, ang, 4)                                   # [B,S,H,R,N] rotated
    q0 = Q.permute(0, 1, 3, 2, 4).repeat_interleave(H // G, dim=2) + Qb       # pre-rotary
    k0 = K.permute(0, 1, 3, 2, 4).repeat_interleave(H // G, dim=2) + Kb
    qk_dot = torch.einsum("bshrn,bshtn->bhsrt", q0, k0)
    # the state entering chunk c must use the trapezoid weight that looks one token ahead (DT/Trap of the first token
    # of chunk c), which a truncated sequence does not see: rebuild it from the full-sequence coefficients instead
    gamma, ts = R.trapezoid_coeffs(DT, Trap)
    psiv = V.unsqueeze(3) * Psi
    st = torch.zeros(B, H, N, P)
    states = []
    for t in range(S):
        if t % cs == 0:
            states.append(st.clone())
        st = st * torch.exp(ADT[:, :, t])[..., None, None] + ts[:, :, t, None, None] * torch.einsum("bhrn,bhrp->bhnp", k[:, t], psiv[:, t])
    states = torch.stack(states, dim=2)                                        # [B,H,nchunks,N,P]
    cum, rev, seg = _prefix_sums(ADT, cs)
    out = bwd(dout, Q, K, V, Qb, Kb, Psi, Phi, ang, cum, rev, DT, Trap, D, seg, states, qk_dot, chunk_size=cs, R=Rk,
              rotary_dim_divisor=4)
    hpg = H // G
    dQ_ref = out["DQ"].view(B, S, Rk, H, N).view(B, S, Rk, G, hpg, N).sum(4)   # heads of a group share Q
    dK_ref = out["DK"].view(B, S, Rk, H, N).view(B, S, Rk, G, hpg, N).sum(4)
    assert _rel(Ql.grad, dQ_ref) < 1e-4, _rel(Ql.grad, dQ_ref)
    assert _rel(Kl.grad, dK_ref) < 1e-4, _rel(Kl.grad, dK_ref)
    assert _rel(angl.grad, out["DANGLES"]) < 1e-4
    # dV: compared on the last chunk, where no state gradient flows in.  For earlier chunks the restatement multiplies K
    # by the TRANSPOSED state gradient (it only type-checks for N == P), which is not the adjoint of its own forward
    # `state += K^T PsiV`; dK, whose carry term needs exactly that transpose, agrees on every chunk.
    assert _rel(Vl.grad[:, S - cs:], out["DV"][:, S - cs:]) < 1e-4


# ---- M2RNN ------------------------------------------------------------------------------------------------------

def test_m2rnn_scan_matches_reference_chunked_form():
    ref_fn = _ref("cppmega.megatron.m2rnn_chunk").chunked_m2rnn_forward
    from cppmega_b200.ops import reference as ours
    g = torch.Generator().manual_seed(2)
    B, S, H, Kd, Vd = 2, 70, 3, 8, 4
    q, k = torch.randn(B, S, 1, Kd, generator=g), torch.randn(B, S, 1, Kd, generator=g)
    v = torch.randn(B, S, H, Vd, generator=g)
    W = torch.randn(H, Vd, Vd, generator=g) * 0.3
    f = torch.sigmoid(torch.randn(B, S, H, generator=g))
    y, h = ours.m2rnn_scan(q, k, v, W, f)
    y_ref, h_ref = ref_fn(q, k, v, W, f, chunk_size=16)
    assert y.shape == y_ref.shape and _rel(y, y_ref) < 1e-5 and _rel(h, h_ref) < 1e-5


# ---- DSA --------------------------------------------------------------------------------------------------------

def test_indexer_scores_match_reference():
    ref_fn = _ref("cppmega.megatron.dsa_indexer_fused_patch").compute_index_scores_fused_bf16
    from cppmega_b200.ops import reference as ours
    g = torch.Generator().manual_seed(3)
    B, S, Hh, Dd = 2, 40, 4, 16
    q, k, w = torch.randn(B, S, Hh, Dd, generator=g), torch.randn(B, S, Dd, generator=g), torch.randn(B, S, Hh, generator=g)
    sc = ours.indexer_scores(q, k, w)
    sc_ref = ref_fn(q.transpose(0, 1).contiguous(), w.transpose(0, 1).contiguous(), k.transpose(0, 1).contiguous())
    assert sc.shape == sc_ref.shape and _rel(sc, sc_ref) < 1e-5


def test_sparse_attention_matches_reference(monkeypatch):
    mod = _ref("cppmega.megatron.dsa_sparse_attention")
    from cppmega_b200.ops import reference as ours
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda *_a, **_k: (1 << 34, 1 << 34))     # the reference sizes its head chunks from free GPU memory
    g = torch.Generator().manual_seed(4)
    B, S, Hq, D, dv, topk = 2, 48, 4, 32, 16, 8
    q, kv = torch.randn(B, S, Hq, D, generator=g), torch.randn(B, S, D, generator=g)
    sc = torch.randn(B, S, S, generator=g).masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
    vals, idx = torch.topk(sc, topk, dim=-1)
    ours_idx = torch.where(torch.isinf(vals), torch.full_like(idx, -1), idx)
    scale = 1.0 / math.sqrt(D)
    out, _ = ours.sparse_mla(q, kv, ours_idx, scale, dv)
    # the reference masks by position (index > query position) instead of a sentinel: give the unseen slots a future index
    ref_idx = torch.where(ours_idx < 0, torch.full_like(idx, S - 1), idx)
    ref_idx[:, S - 1] = idx[:, S - 1]
    kq = kv.unsqueeze(2).expand(B, S, Hq, D)
    out_ref = mod.sparse_dsa_fn(q.transpose(0, 1).contiguous(), kq.transpose(0, 1).contiguous(),
                                kq[..., :dv].transpose(0, 1).contiguous(), ref_idx, scale)
    out_ref = out_ref.view(S, B, Hq, dv).transpose(0, 1)
    rows = slice(topk, S - 1)          # queries that see at least top-k keys and are not the last position
    assert _rel(out[:, rows], out_ref[:, rows]) < 1e-5


# ---- embeddings -------------------------------------------------------------------------------------------------

def test_ngram_hash_matches_reference_module():
    Ref = _ref("cppmega.features.engram.ngram_hash").CppMegaNgramHashEmbedding
    from cppmega_b200.ops import reference as ours
    torch.manual_seed(6)
    m = Ref(hidden_size=32, orders=(2, 3), num_heads=3, table_size=997, embed_dim=8)
    ids = torch.randint(0, 5000, (2, 37))
    idx_ref = m._hash_all(ids).permute(0, 2, 1)                                  # [B,S,T]
    idx = ours.ngram_hash_indices(ids, m.hash_mults, m.hash_bias, m.table_sizes_t, m.table_offsets, m.order_for_table)
    assert torch.equal(idx, idx_ref)
    emb = ours.ngram_hash_embed(ids, m.unified_table.weight, m.hash_mults, m.hash_bias, m.table_sizes_t, m.table_offsets,
                                m.order_for_table)
    torch.nn.init.normal_(m.out_proj.weight)
    assert _rel(torch.nn.functional.linear(emb, m.out_proj.weight), m(ids)) < 1e-6
