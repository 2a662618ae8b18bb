"""Pattern language, typed configs and the Megatron-style argument surface (pure Python)."""
import dataclasses

import pytest

from cppmega_b200.config import pattern as P
from cppmega_b200.config.model import (DSAConfig, MoEConfig, ModelConfig, Mamba3Config, get_preset, nam56r_full,
                                       nam56r_tiny)
from cppmega_b200.parallel.state import ParallelConfig, group_rank_lists, rank_coordinates
from cppmega_b200.training.arguments import parse_args, render_args
from cppmega_b200.training.trainer import TrainConfig


def test_pattern_tiling_counts():
    c = P.count_symbols("AEMEAEMEAEMR", 52)
    assert c == {"A": 13, "E": 22, "M": 13, "R": 4}
    plan = P.translate_pattern("AEMEAEMEAEMR", 52, mtp_depths=2)
    assert plan.hybrid_pattern.startswith("*EME*EME*EMM*")
    assert plan.full_pattern.endswith("/*-/*-")
    assert plan.r_layer_numbers == (12, 24, 36, 48)
    assert len(plan.attention_layer_numbers) == 13


def test_pattern_rejects_bad_input():
    with pytest.raises(P.PatternError):
        P.expand_nam_pattern("AXM", 3)
    with pytest.raises(P.PatternError):
        P.expand_nam_pattern("AE|ME", 5)
    with pytest.raises(P.PatternError):
        P.expand_nam_pattern("", 4)
    assert P.expand_nam_pattern("AE|ME", 4) == list("AEME")


def test_pipeline_split():
    assert P.split_pattern_for_pipeline("*" * 52, 2, 2) == "|".join(["*" * 13] * 4)
    assert P.split_pattern_for_pipeline("MMMMMMMMMM", 4) == "MMM|MMM|MM|MM"
    main, mtp, chunks = P.parse_hybrid_pattern("*EM|E*E/*-/*-")
    assert main == list("*EME*E") and mtp == 2 and chunks == [3, 3]
    with pytest.raises(P.PatternError):
        P.parse_hybrid_pattern("*EM/*E")


def test_int_list():
    assert P.parse_int_list("1,2,5-7") == (1, 2, 5, 6, 7)
    assert P.parse_int_list("") == ()
    assert P.parse_int_list([3, 1, 3]) == (1, 3)


def test_nam56r_layout_matches_reference_facts():
    cfg = nam56r_full()
    kinds = cfg.layer_kinds()
    assert kinds.count("dsa") == 9 and kinds.count("mla") == 4
    assert kinds.count("mamba3") == 13 and kinds.count("m2rnn") == 4 and kinds.count("moe") == 22
    assert [i + 1 for i, k in enumerate(kinds) if k == "m2rnn"] == [12, 24, 36, 48]
    assert sum(cfg.mamba3.in_proj_sizes(cfg.hidden_size)) == 24960
    assert cfg.mamba3.num_rope_angles == 32 and cfg.mamba3.rotary_dim_divisor == 4
    pc = cfg.param_count()
    assert 7.5e9 < pc["total"] < 8.5e9 and pc["active"] < pc["total"]


def test_config_validation():
    with pytest.raises(ValueError):
        Mamba3Config(rope_fraction=0.3)
    with pytest.raises(ValueError):
        MoEConfig(dispatcher="ring")
    with pytest.raises(ValueError):
        DSAConfig(indexer_dtype="fp8")
    with pytest.raises(ValueError):
        ModelConfig(mamba_variant="s4")
    with pytest.raises(KeyError):
        get_preset("nope")
    with pytest.raises(ValueError):
        Mamba3Config().in_proj_sizes(4096, tp=3)


def test_tp_partition_sizes():
    m3 = Mamba3Config()
    full = m3.in_proj_sizes(4096, 1)
    half = m3.in_proj_sizes(4096, 2)
    assert all(f == 2 * h for f, h in zip(full, half))
    assert half == (4096, 4096, 2048, 2048, 64, 64, 64)


@pytest.mark.parametrize("preset", ["nam56r", "nam56r_tiny"])
def test_args_round_trip(preset):
    m = get_preset(preset)
    p = ParallelConfig(pp=2, ep=2, tp=1, distributed_optimizer=True, overlap_grad_reduce=True)
    t = TrainConfig(seq_length=m.seq_length, recompute="selective")
    argv = render_args(m, p, t, mock_data=True, save="/tmp/x", save_interval=10)
    m2, p2, t2, ex = parse_args(argv + ["--model-preset", preset])
    assert m2.layer_kinds() == m.layer_kinds()
    assert dataclasses.replace(m2, pattern=m.pattern) == m
    assert (p2.pp, p2.ep, p2.tp, p2.distributed_optimizer) == (2, 2, 1, True)
    assert t2.recompute == "selective" and ex["save"] == "/tmp/x" and ex["mock_data"]
    assert "--hybrid-layer-pattern" in argv and "--use-distributed-optimizer" in argv
    assert "--expert-model-parallel-size" in argv


def test_args_reject_unsupported():
    with pytest.raises(ValueError):
        parse_args(["--context-parallel-size", "2"])
    with pytest.raises(ValueError):
        parse_args(["--moe-token-dispatcher-type", "flex"])
    with pytest.raises(P.PatternError):
        parse_args(["--hybrid-layer-pattern", "*EM", "--r-layer-indices", "1"])


def test_rank_groups():
    cfg = ParallelConfig(tp=2, pp=2, ep=2)
    lists = group_rank_lists(16, cfg)
    assert [0, 1] in lists["tp"] and [0, 8] in lists["pp"]
    assert [0, 2, 4, 6] in lists["dp"] and [0, 2] in lists["ep"] and [0, 4] in lists["edp"]
    for kind, groups in lists.items():
        flat = sorted(r for g in groups for r in g)
        assert flat == list(range(16)), kind
    assert rank_coordinates(13, 16, cfg) == (1, 0, 1, 2, 1)
    with pytest.raises(ValueError):
        ParallelConfig(tp=3).dp(8)
    with pytest.raises(ValueError):
        ParallelConfig(cp=2)
    assert nam56r_tiny().plan().needs_mamba3


def test_precision_rules_scope_the_recipe_to_matching_modules():
    import torch
    import torch.nn as nn
    from cppmega_b200.ops import functional as F_

    seen = {}

    class Probe(nn.Module):
        def __init__(self, tag):
            super().__init__()
            self.tag = tag

        def forward(self, x):
            seen[self.tag] = F_.precision_recipe()
            return x

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.mixer = nn.Module()
            self.mixer.in_proj = Probe("in_proj")
            self.mixer.inner = Probe("inner")
            self.mlp = Probe("mlp")

        def forward(self, x):
            return self.mlp(self.mixer.inner(self.mixer.in_proj(x)))

    net = nn.Sequential(Layer())
    try:
        handles, matched = F_.install_precision_rules(net, [("*.mixer.in_proj", "mxfp8"), ("*.mlp", "tensorwise")], default="bf16")
        assert matched == ["0.mixer.in_proj", "0.mlp"]
        net(torch.zeros(1))
        assert seen == {"in_proj": "mxfp8", "inner": "bf16", "mlp": "tensorwise"}
        assert F_.precision_recipe() == "bf16"                      # restored after the forward
        with F_.precision_scope("mxfp8"):
            assert F_.precision_recipe() == "mxfp8"
        assert F_.precision_recipe() == "bf16"
        for h in handles:
            h.remove()
        with pytest.raises(ValueError):
            F_.set_precision_recipe("fp4")
    finally:
        F_.set_precision_recipe("bf16")


def test_fp8_arguments_round_trip_and_module_sets():
    from cppmega_b200.training.arguments import parse_args, render_args
    mcfg, pcfg, tcfg, _ = parse_args(["--model-preset", "nam56r_tiny", "--mock-data", "--fp8-recipe", "tensorwise", "--fp8-modules", "moe"])
    assert tcfg.precision_recipe == "tensorwise" and tcfg.precision_modules == ("moe",)
    argv = render_args(mcfg, pcfg, tcfg, mock_data=True)
    assert parse_args(argv)[2].precision_modules == ("moe",)
    from cppmega_b200.models import build_model
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.parallel.state import single_process_context
    from cppmega_b200.training.trainer import _install_precision
    model = build_model(mcfg, single_process_context())
    try:
        matched = _install_precision(model, tcfg)
        assert matched and all(".mlp" in m for m in matched)
        kinds = {n for n, m in model.named_modules() if type(m).__name__ == "MoELayer"}
        assert kinds <= set(matched)
        assert F_.precision_recipe() == "bf16"                      # default outside the selected modules
    finally:
        F_.set_precision_recipe("bf16")


def test_trainer_reports_which_fast_paths_are_off_and_why():
    import torch
    from cppmega_b200.config.model import nam56r_tiny
    from cppmega_b200.training.trainer import TrainConfig, Trainer
    tr = Trainer(nam56r_tiny(seq_length=32), TrainConfig(micro_batch_size=1, seq_length=32, dtype="fp32", log_interval=0),
                 device=torch.device("cpu"))
    paths = tr.describe_paths()
    assert paths["optimizer"].startswith("off: ") and paths["moe"].startswith("off: ") and paths["tp"].startswith("off: ")
    assert "no GPU" in paths["optimizer"] and "tensor-parallel size 1" in paths["tp"]
    assert paths["cuda_graphs"].startswith("off: ") and paths["recompute"] == "none"


def test_deterministic_mode_routes_atomic_kernels_to_their_definitions():
    import torch
    from cppmega_b200.ops import functional as F_
    from cppmega_b200.training.arguments import parse_args
    _m, _p, tcfg, _e = parse_args(["--model-preset", "nam56r_tiny", "--deterministic-mode", "--mock-data"])
    assert tcfg.deterministic
    try:
        F_.set_deterministic(True)
        assert F_.is_deterministic() and set(F_.ATOMIC_REDUCTION_OPS) <= F_._DISABLED
        assert torch.are_deterministic_algorithms_enabled()
    finally:
        F_.set_deterministic(False)
    assert not F_.is_deterministic() and not (set(F_.ATOMIC_REDUCTION_OPS) & F_._DISABLED)
    assert not torch.are_deterministic_algorithms_enabled()
