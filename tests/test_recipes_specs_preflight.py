"""Recipes, stack specs, launch preflight and the host-side failure detection."""
import threading
import time

import pytest
import torch

from cppmega_b200.config import recipes as R
from cppmega_b200.config.model import nam56r_full, nam56r_tiny
from cppmega_b200.models import specs as S
from cppmega_b200.utils import preflight as PF
from cppmega_b200.utils.deprecated import DeprecatedPathError
from cppmega_b200.utils.watchdog import DictStore, RankHeartbeat, StepWatchdog


def test_recipes_render_and_refuse_mock_data():
    r = R.get_recipe("native_pretrain")
    with pytest.raises(ValueError, match="refuses mock data"):
        r.to_args(mock_data=True, data_path=None)
    argv = r.to_args(data_path="/data/corpus")
    assert "--expert-model-parallel-size" in argv and argv[argv.index("--expert-model-parallel-size") + 1] == "8"
    assert "/data/corpus" in argv
    env = r.to_env_dict()
    assert env["NCCL_NVLS_ENABLE"] == "0"
    assert R.get_recipe("mamba3_native").to_env_dict()["CUDA_DEVICE_MAX_CONNECTIONS"] == "1"     # TP overlap ordering
    assert R.get_recipe("smoke_test").to_args()                                                   # synthetic data allowed
    assert "torch.distributed.run" in R.get_recipe("smoke_test").shell()
    with pytest.raises(DeprecatedPathError):
        R.get_recipe("mamba3_te")
    assert R.get_recipe("mamba3_te", ack=True).profile.model.mamba_variant == "ssd"
    with pytest.raises(KeyError):
        R.get_recipe("nope")


def test_recipe_argv_round_trips_through_the_parser():
    from cppmega_b200.training.arguments import parse_args
    r = R.get_recipe("noconv")
    mcfg, pcfg, tcfg, extras = parse_args(r.to_args(data_path="/d/x"))
    assert mcfg.mamba_variant == "noconv_ssd" and pcfg.ep == 8 and tcfg.micro_batch_size == 4
    assert extras["data_path"] == "/d/x" and not extras["mock_data"]


def test_moe_flag_validation():
    import dataclasses
    from cppmega_b200.parallel.state import ParallelConfig
    cfg = nam56r_full()
    bad = dataclasses.replace(cfg, moe=dataclasses.replace(cfg.moe, dispatcher="flex"))
    with pytest.raises(ValueError, match="expert parallelism"):
        R.validate_moe_flags(bad, ParallelConfig(ep=1))
    R.validate_moe_flags(bad, ParallelConfig(ep=8))


def test_stack_specs():
    cfg = nam56r_full()
    full = S.apply_spec(cfg, S.get_spec("nam56r_full"))
    idx = S.custom_layer_indices(full)
    assert len(idx["dsa"]) == 9 and len(idx["mla"]) == 4 and idx["m2rnn"] == [12, 24, 36, 48]
    lite = S.apply_spec(cfg, S.get_spec("nam56r_lite"))
    assert "dsa" not in S.custom_layer_indices(lite) and "m2rnn" not in S.custom_layer_indices(lite)
    local = S.apply_spec(cfg, S.get_spec("mamba_local"))
    kinds = set(local.layer_kinds())
    assert kinds == {"mla", "mlp", "mamba3"} and local.mtp.num_layers == 0 and local.mamba_variant == "ssd"
    desc = S.describe_stack(S.apply_spec(cfg, S.get_spec("nam56r_noconv")))
    assert any("SSDMixer[noconv_ssd]" in d[2] for d in desc) and len(desc) == 52
    with pytest.raises(KeyError):
        S.get_spec("x")


def test_every_spec_builds_and_runs_tiny():
    from cppmega_b200.models.nam56r import build_model
    for name in S.SPECS:
        cfg = S.apply_spec(nam56r_tiny(seq_length=32), S.get_spec(name))
        model = build_model(cfg)
        ids = torch.randint(0, cfg.vocab_size, (1, 32))
        out = model(ids, ids)
        assert torch.isfinite(out["loss"]), name


def test_preflight_parses_ptxas_and_flags_violations(tmp_path):
    text = """ptxas info    : Compiling entry function '_Z4kernA' for 'sm_100a'
ptxas info    : Function properties for _Z4kernA
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 96 registers, used 1 barriers, 1024 bytes smem
ptxas info    : Compiling entry function '_Z4kernB' for 'sm_100a'
ptxas info    : Function properties for _Z4kernB
    400 bytes stack frame, 380 bytes spill stores, 400 bytes spill loads
ptxas info    : Used 255 registers, used 1 barriers, 60000 bytes smem
"""
    ks = PF.parse_ptxas(text)
    assert [k.name for k in ks] == ["_Z4kernA", "_Z4kernB"] and ks[0].registers == 96 and ks[1].spill_stores == 380
    (tmp_path / "x.ptxas.txt").write_text(text)
    rep = PF.static_check(tmp_path)
    assert not rep.ok and any("static shared memory" in p for p in rep.problems)
    assert any("spills" in w for w in rep.warnings)
    src = tmp_path / "src"
    src.mkdir()
    (src / "k.cu").write_text("tmem_alloc(slot, 768);\n tmem_alloc(slot, 256);")
    rep2 = PF.source_check(src)
    assert len(rep2.problems) == 1 and "768" in rep2.problems[0]
    assert PF.source_check().ok and "preflight" in PF.run_all().render()


def test_step_watchdog_fires_only_without_progress():
    fired = []
    wd = StepWatchdog(0.3, rank=0, on_timeout=lambda idle, step: fired.append((idle, step)), poll_s=0.05).start()
    for s in range(5):
        time.sleep(0.1)
        wd.beat(s)
    assert not fired
    time.sleep(0.6)
    wd.stop()
    assert fired and fired[0][1] == 4 and wd.fired


def test_rank_heartbeat_reports_dead_and_lagging_ranks():
    store = DictStore()
    now = [100.0]
    hbs = [RankHeartbeat(store, r, 3, limit_s=5.0, clock=lambda: now[0]) for r in range(3)]
    for h in hbs:
        h.beat(10)
    assert hbs[0].dead_ranks() == []
    now[0] = 104.0
    hbs[0].beat(12)
    hbs[1].beat(12)                 # rank 2 stopped: raised, exited, or never joined this step
    now[0] = 107.0
    assert hbs[0].dead_ranks() == [2] and hbs[1].dead_ranks() == [2]
    assert hbs[0].lagging_ranks(max_lag_steps=1) == [2]
    fresh = RankHeartbeat(DictStore(), 0, 2, limit_s=1.0)
    fresh.beat(0)
    assert fresh.dead_ranks() == [1]          # a rank that never wrote a heartbeat counts as missing


def test_heartbeat_threads_share_a_store():
    store = DictStore()
    stop = threading.Event()

    def worker(rank):
        hb = RankHeartbeat(store, rank, 2, limit_s=0.5)
        step = 0
        while not stop.is_set() and step < 50:
            hb.beat(step)
            step += 1
            time.sleep(0.01)

    ts = [threading.Thread(target=worker, args=(r,)) for r in range(2)]
    for t in ts:
        t.start()
    time.sleep(0.1)
    assert RankHeartbeat(store, 0, 2, limit_s=0.5).dead_ranks() == []
    stop.set()
    for t in ts:
        t.join()


def test_cuda_graph_scope_parsing_and_argument_round_trip():
    from cppmega_b200.training.arguments import build_parser, configs_from_namespace
    from cppmega_b200.utils import cuda_graphs
    assert cuda_graphs.parse_scope(["mamba", "attn", "moe_router"]) == ("mamba3", "m2rnn", "mla")
    assert cuda_graphs.parse_scope([]) == ()
    with pytest.raises(ValueError):
        cuda_graphs.parse_scope(["everything"])
    with cuda_graphs.forbid_host_sync():          # no CUDA here: must be a no-op
        pass
    ns = build_parser().parse_args(["--cuda-graph-scope", "mamba", "mlp"])
    tcfg = configs_from_namespace(ns)[2]
    assert tcfg.cuda_graph_scope == ("mamba", "mlp")
    import torch.nn as nn
    assert cuda_graphs.capture_model_layers(nn.Linear(2, 2), ["mamba"], (1, 2, 2), None, "cpu") == 0


def test_moe_plan_invariants_on_cpu():
    """The library-op definition of the routing plan (the oracle of the plan kernels): destinations are unique, lie in
    their expert's padded segment on the owning rank, and the tile map agrees with the segments."""
    from cppmega_b200.parallel.fused_moe import MoEPlan, TILE
    torch.manual_seed(0)
    T, k, E, ep = 500, 4, 16, 4
    El = E // ep
    ids_by_rank = [torch.stack([torch.randperm(E)[:k] for _ in range(T)]) for _ in range(ep)]
    counts = torch.stack([torch.bincount(i.reshape(-1), minlength=E) for i in ids_by_rank])      # [ep, E]
    cap = ((T * k * ep + 16 * TILE) // TILE) * TILE
    plans = [MoEPlan(ids_by_rank[r], E, ep, r, None, cap, gather=lambda c, r=r: counts.clone()) for r in range(ep)]
    for owner in range(ep):
        rows = torch.cat([p.dest_row[p.dest_rank == owner] for p in plans])
        assert rows.unique().numel() == rows.numel()                                              # no two copies share a row
        po = plans[owner]
        tot = counts.sum(0)[owner * El:(owner + 1) * El]
        assert torch.equal(po.tot_local.long(), tot)
        seg = po.seg_offsets.long()
        assert (seg % TILE == 0).all() and int(po.rows_used) == int(seg[-1]) <= cap
        for r, p in enumerate(plans):
            sel = p.dest_rank == owner
            e_local = p_ids = ids_by_rank[r].reshape(-1)[sel] - owner * El
            assert ((p.dest_row[sel] >= seg[e_local]) & (p.dest_row[sel] < seg[e_local] + tot[e_local])).all()
        used_tiles = int(seg[-1]) // TILE
        te = po.tile_expert.long()
        assert (te[used_tiles:] == -1).all()
        for e in range(El):
            assert (te[int(seg[e]) // TILE:int(seg[e + 1]) // TILE] == e).all()


def test_moe_plan_overflow_is_clipped_to_the_buffer():
    """A skewed routing that needs more rows than the receive buffer holds: the receive layout (segments, tile map,
    reduction ranges) never reaches past the buffer, and the copies that do not fit are exactly those the transport
    kernels skip and report (row >= capacity)."""
    from cppmega_b200.parallel.fused_moe import MoEPlan, TILE
    torch.manual_seed(1)
    T, k, E, ep = 600, 2, 8, 2
    El = E // ep
    ids_by_rank = []
    for _ in range(ep):
        ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
        ids[: T * 3 // 4, 0] = 1                               # expert 1 (rank 0) takes three quarters of the tokens
        ids[: T * 3 // 4, 1] = 2
        ids_by_rank.append(ids)
    counts = torch.stack([torch.bincount(i.reshape(-1), minlength=E) for i in ids_by_rank])
    cap = 6 * TILE                                             # far below rank 0's load
    need0 = int(((counts.sum(0)[:El] + TILE - 1) // TILE * TILE).sum())
    assert need0 > cap
    plans = [MoEPlan(ids_by_rank[r], E, ep, r, None, cap, gather=lambda c: counts.clone()) for r in range(ep)]
    p0 = plans[0]
    assert int(p0.seg_offsets.max()) <= cap and int(p0.rows_used) <= cap
    assert ((p0.seg_start_local.long() + p0.tot_local.long()) <= cap).all()
    assert p0.tile_expert.numel() == cap // TILE
    dropped = sum(int(((p.dest_row >= cap) & (p.dest_rank == 0)).sum()) for p in plans)
    assert dropped > 0                                          # these are skipped + reported by push / pull
    kept = torch.cat([p.dest_row[(p.dest_rank == 0) & (p.dest_row < cap)] for p in plans])
    assert kept.unique().numel() == kept.numel() and int(kept.max()) < cap


def test_chunked_indexer_kl_loss_equals_dense_form():
    from cppmega_b200.ops import reference as ref
    torch.manual_seed(3)
    B, S, H, D, Hi, Di = 2, 70, 3, 8, 4, 6
    aq, ak = torch.randn(B, S, H, D), torch.randn(B, S, H, D)
    mk = lambda *s: torch.randn(*s, requires_grad=True)
    qi, ki, w = mk(B, S, Hi, Di), mk(B, S, Di), mk(B, S, Hi)
    dense = ref.indexer_kl_loss(aq, ak, 0.3, qi, ki, w, 0.7)
    g1 = torch.autograd.grad(dense, (qi, ki, w))
    chunked = ref.indexer_kl_loss_chunked(aq, ak, 0.3, qi, ki, w, 0.7, rows=16)
    g2 = torch.autograd.grad(chunked, (qi, ki, w))
    assert abs(float(dense) - float(chunked)) < 1e-5 * max(1.0, abs(float(dense)))
    for a, b in zip(g1, g2):
        assert (a - b).abs().max() < 1e-5


def test_dsa_warmup_pass_gives_dense_attention_and_the_indexer_kl_loss():
    """One chunked pass returns the dense causal attention output and the same KL loss as the separate definition; the loss
    sends gradients to the indexer operands only, the output to q / k / v."""
    import torch
    from cppmega_b200.ops import reference as ref
    torch.manual_seed(0)
    B, S, H, D, Dv, Hi, Di = 2, 48, 3, 16, 8, 2, 8
    q, k = torch.randn(B, S, H, D, requires_grad=True), torch.randn(B, S, H, D, requires_grad=True)
    v = torch.randn(B, S, H, Dv, requires_grad=True)
    qi, ki = torch.randn(B, S, Hi, Di, requires_grad=True), torch.randn(B, S, Di, requires_grad=True)
    w = torch.randn(B, S, Hi, requires_grad=True)
    out, loss = ref.dsa_warmup_attention_and_kl(q, k, v, D ** -0.5, qi, ki, w, coeff=0.5, rows=20)
    want_loss = ref.indexer_kl_loss(q.detach(), k.detach(), D ** -0.5, qi, ki, w, 0.5)
    want_out = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                is_causal=True, scale=D ** -0.5).transpose(1, 2)
    assert torch.allclose(loss, want_loss, atol=1e-5) and torch.allclose(out, want_out, atol=1e-5)
    gq, gqi = torch.autograd.grad(loss, (q, qi), allow_unused=True)
    assert gq is None and gqi is not None and gqi.abs().sum() > 0
    (gv,) = torch.autograd.grad(out.sum(), (v,), retain_graph=True)
    assert gv.abs().sum() > 0


def test_model_runs_the_dsa_warmup_mode():
    import dataclasses
    import torch
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.parallel.dist_optimizer import OptimizerConfig
    from cppmega_b200.training.trainer import TrainConfig, Trainer, synthetic_batches
    cfg = nam56r_tiny(seq_length=64)
    cfg = dataclasses.replace(cfg, dsa=dataclasses.replace(cfg.dsa, warmup_dense=True, indexer_loss_coeff=0.1))
    tr = Trainer(cfg, TrainConfig(micro_batch_size=2, seq_length=64, dtype="fp32", log_interval=0,
                                  optimizer=OptimizerConfig(lr=1e-3)), device=torch.device("cpu"))
    stream = synthetic_batches(cfg.vocab_size, 2, 64, seed=0, pin=False)
    losses = [float(tr.train_step(next(stream))["loss"]) for _ in range(2)]
    assert all(l == l and l < 20 for l in losses)
    dsa_layers = [l for l in tr.model.decoder.layers.values() if l.kind == "dsa"]
    assert dsa_layers and all(l.self_attention.last_indexer_loss is not None for l in dsa_layers)


def test_moe_chunk_selection_and_flag_layout():
    """Host-side bookkeeping of the two-chunk MoE pipeline: when a call is split, and that every (layer, chunk, purpose)
    gets its own flag word block inside the heap's flag area for a 64-layer model on 8 ranks."""
    import types
    from cppmega_b200.parallel import fused_moe as fm
    from cppmega_b200.parallel.symm_mem import FLAG_WORDS
    stub = types.SimpleNamespace(chunks=fm.MAX_CHUNKS)
    pick = lambda tokens, topk: fm.FusedMoEBuffers.chunks_for(stub, tokens, topk)
    assert pick(16384, 4) == 2                              # the benchmark shape: two chunks of 8192 tokens
    assert pick(16383, 4) == 1                              # odd token count: not split
    assert pick(2048, 4) == 1                               # 4096 copies per chunk: below the threshold
    stub.chunks = 1
    assert pick(16384, 4) == 1
    seen = set()
    for layer in range(64):
        for chunk in range(fm.MAX_CHUNKS):
            f0 = fm._flag0(layer, chunk)
            for purpose in range(fm.FLAGS_PER_CHUNK):
                idx = f0 + purpose
                assert idx not in seen and idx >= fm.FLAG_BASE
                seen.add(idx)
    assert (max(seen) + 1) * 8 <= FLAG_WORDS                # 8 ranks: one word per rank and flag
