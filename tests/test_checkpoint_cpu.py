"""sharded_state_dict layout, replica rules and save/load round trips on CPU."""
import json
import os

import pytest
import torch

from cppmega_b200.checkpoint import sharded
from cppmega_b200.config.model import nam56r_tiny
from cppmega_b200.models import build_model
from cppmega_b200.parallel.dist_optimizer import DistributedOptimizer, OptimizerConfig
from cppmega_b200.parallel.state import ParallelConfig, ParallelContext


def _pc(**kw):
    return ParallelContext(config=ParallelConfig(**{k: v for k, v in kw.items() if k in ("tp", "pp", "ep")}),
                           **{k: v for k, v in kw.items() if k not in ("tp", "pp", "ep")})


def test_keys_follow_reference_names():
    pc = _pc()
    model = build_model(nam56r_tiny(), pc)
    keys = {r.key for r in sharded.sharded_state_dict(model, pc)}
    for k in ["embedding.word_embeddings.weight", "embedding.cppmega_ngram_hash.unified_table.weight",
              "embedding.cppmega_ngram_hash.out_proj.weight", "decoder.layers.0.mixer.in_proj.weight",
              "decoder.layers.0.mixer.dt_bias", "decoder.layers.1.mlp.router.weight",
              "decoder.layers.1.mlp.experts.linear_fc1.weight0", "decoder.layers.1.mlp.experts.linear_fc2.weight3",
              "decoder.layers.1.mlp.shared_experts.linear_fc1.weight",
              "decoder.layers.4.self_attention.linear_q_down_proj.weight",
              "decoder.layers.4.self_attention.core_attention.indexer.linear_wk.weight", "decoder.final_norm.weight",
              "output_layer.weight", "mtp.layers.0.eh_proj.weight"]:
        assert k in keys, k


def test_packed_in_proj_emits_one_record_per_component():
    pc = _pc(tp=2, tp_rank=1, tp_ranks=[0, 1])
    cfg = nam56r_tiny()
    model = build_model(cfg, pc)
    recs = [r for r in sharded.sharded_state_dict(model, pc) if r.key == "decoder.layers.0.mixer.in_proj.weight"]
    sizes_full = cfg.mamba3.in_proj_sizes(cfg.hidden_size, 1)
    assert len(recs) == 7
    gpos = 0
    for r, full in zip(recs, sizes_full):
        assert r.global_shape == (sum(sizes_full), cfg.hidden_size)
        assert r.global_offset == (gpos + full // 2, 0) and r.data.shape[0] == full // 2
        gpos += full


def test_mtp_stage_embedding_is_a_replica():
    pc = _pc(pp=2, pp_rank=1, pp_ranks=[0, 1])
    model = build_model(nam56r_tiny(), pc)
    recs = sharded.sharded_state_dict(model, pc)
    emb = [r for r in recs if r.key.startswith("embedding.")]
    assert emb and all(r.replica_id[0] == 1 and not r.is_main_replica for r in emb)
    assert all(r.is_main_replica for r in recs if r.key.startswith("output_layer"))


def test_duplicate_main_replicas_are_rejected():
    idx = {"w": {"global_shape": [4, 4], "dtype": "float32",
                 "shards": [{"shape": [4, 4], "global_offset": [0, 0]}, {"shape": [4, 4], "global_offset": [0, 0]}]}}
    with pytest.raises(ValueError, match="duplicate"):
        sharded.validate_coverage(idx)


def test_save_load_round_trip_and_resume(tmp_path):
    pc = _pc()
    cfg = nam56r_tiny(seq_length=32)
    torch.manual_seed(0)
    model = build_model(cfg, pc)
    opt = DistributedOptimizer(model, OptimizerConfig(lr=1e-3), pc)
    ids = torch.randint(0, cfg.vocab_size, (2, 32))
    for _ in range(2):
        opt.zero_grad()
        model(ids, torch.roll(ids, -1, 1))["loss"].backward()
        opt.step()
    sharded.save_checkpoint(str(tmp_path), 2, model, pc, opt, extra={"tokens": 128})
    meta = json.load(open(os.path.join(tmp_path, "iter_0000002", "metadata.json")))
    assert meta["extra"]["tokens"] == 128 and sharded.latest_iteration(str(tmp_path)) == 2
    ref_loss = []
    for _ in range(2):
        opt.zero_grad()
        out = model(ids, torch.roll(ids, -1, 1))
        out["loss"].backward()
        opt.step()
        ref_loss.append(out["loss"].item())
    model2 = build_model(cfg, pc, seed=999)
    opt2 = DistributedOptimizer(model2, OptimizerConfig(lr=1e-3), pc)
    info = sharded.load_checkpoint(str(tmp_path), model2, pc, opt2)
    assert info["iteration"] == 2 and not info["missing"]
    got = []
    for _ in range(2):
        opt2.zero_grad()
        out = model2(ids, torch.roll(ids, -1, 1))
        out["loss"].backward()
        opt2.step()
        got.append(out["loss"].item())
    assert got == pytest.approx(ref_loss, rel=1e-5)


def test_load_reshards_tensor_parallel(tmp_path):
    cfg = nam56r_tiny(seq_length=32)
    pc1 = _pc()
    full = build_model(cfg, pc1)
    sharded.save_checkpoint(str(tmp_path), 1, full, pc1)
    for rank in (0, 1):
        pc2 = _pc(tp=2, tp_rank=rank, tp_ranks=[0, 1])
        part = build_model(cfg, pc2, seed=7)
        sharded.load_checkpoint(str(tmp_path), part, pc2)
        w_full = full.decoder.layers["0"].mixer.in_proj.weight
        w_part = part.decoder.layers["0"].mixer.in_proj.weight
        sizes = cfg.mamba3.in_proj_sizes(cfg.hidden_size, 1)
        pos, pieces = 0, []
        for s in sizes:
            pieces.append(w_full[pos + rank * s // 2: pos + (rank + 1) * s // 2])
            pos += s
        assert torch.equal(w_part, torch.cat(pieces))
        o_full = full.decoder.layers["0"].mixer.out_proj.weight
        o_part = part.decoder.layers["0"].mixer.out_proj.weight
        assert torch.equal(o_part, o_full.chunk(2, dim=1)[rank])
