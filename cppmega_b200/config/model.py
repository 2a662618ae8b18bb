"""Typed model configuration for the NAM56R family.

A single frozen dataclass tree replaces the reference's three tiers (typed
profile -> rendered environment -> import-time reads; cppmega/recipes/run_profiles.py:41-279
and cppmega/megatron/nam56r_layout.py:14-71).  Every knob that changes model behaviour
lives here; nothing is read from the process environment.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

from .pattern import HybridPlan, attention_ranks, translate_pattern


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


@dataclass(frozen=True)
class Mamba3Config:
    """Mamba3 MIMO mixer dims (cppmega/features/mamba3/config.py:8-75)."""

    d_state: int = 128
    headdim: int = 64
    ngroups: int = 8
    expand: int = 2
    mimo_rank: int = 4
    chunk_size: int = 16
    rope_fraction: float = 0.5
    a_floor: float = 1e-4
    dt_min: float = 1e-3
    dt_max: float = 0.1
    dt_init_floor: float = 1e-4
    is_mimo: bool = True
    outproj_norm: bool = False

    def __post_init__(self):
        _check(self.rope_fraction in (0.5, 1.0), f"unsupported rope_fraction={self.rope_fraction}")
        _check(self.d_state % 4 == 0, "d_state must be a multiple of 4")
        _check(self.mimo_rank >= 1 and self.chunk_size >= 1, "mimo_rank/chunk_size must be positive")

    @property
    def rotary_dim_divisor(self) -> int:
        return int(round(2 / self.rope_fraction))

    @property
    def num_rope_angles(self) -> int:
        split = int(self.d_state * self.rope_fraction)
        split -= split % 2
        return split // 2

    def d_inner(self, hidden: int) -> int:
        return hidden * self.expand

    def nheads(self, hidden: int) -> int:
        d = self.d_inner(hidden)
        _check(d % self.headdim == 0, f"d_inner={d} not divisible by headdim={self.headdim}")
        return d // self.headdim

    def in_proj_sizes(self, hidden: int, tp: int = 1) -> Tuple[int, ...]:
        """Per-rank widths of the packed in_proj ``[z, x, B, C, dd_dt, dd_A, trap]``.

        B and C are laid out ``(group, rank, state)`` so that a tensor-parallel
        slice is a whole number of groups
        (cppmega/megatron/cppmega_mamba3_tp_mixer.py:167-242).
        """
        h = self.nheads(hidden)
        _check(h % tp == 0 and self.ngroups % tp == 0, "nheads and ngroups must divide by tp")
        _check(h % self.ngroups == 0, "nheads must be divisible by ngroups")
        di = self.d_inner(hidden) // tp
        bc = (self.ngroups // tp) * self.d_state * self.mimo_rank
        hl = h // tp
        return (di, di, bc, bc, hl, hl, hl)


@dataclass(frozen=True)
class M2RNNConfig:
    """Matrix-state RNN mixer dims (cppmega/features/m2rnn/config.py:20-46)."""

    k_head_dim: int = 64
    v_head_dim: int = 16
    conv_kernel: int = 4
    num_q_heads: int = 1
    num_k_heads: int = 1
    num_v_heads: int = 0      # 0 -> hidden // (k_head_dim + v_head_dim)
    use_residual: bool = True
    a_init_min: float = 0.0
    a_init_max: float = 16.0
    dt_init_min: float = 1e-3
    dt_init_max: float = 0.1
    dt_init_floor: float = 1e-4
    bwd_chunk_size: int = 64

    def heads(self, hidden: int) -> int:
        return self.num_v_heads or max(1, hidden // (self.k_head_dim + self.v_head_dim))


@dataclass(frozen=True)
class MLAConfig:
    """Multi-head latent attention dims (cppmega/recipes/megatron_args.py:38-42)."""

    num_heads: int = 32
    q_lora_rank: int = 64
    kv_lora_rank: int = 64
    qk_head_dim: int = 64
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 64
    rope_base: float = 500000.0

    @property
    def q_head_dim(self) -> int:
        return self.qk_head_dim + self.qk_pos_emb_head_dim


@dataclass(frozen=True)
class DSAConfig:
    """DeepSeek-style sparse attention: indexer + top-k + sparse MLA.

    ``full_layer_ranks`` are ranks *among DSA layers* that run the indexer and
    publish their indices; the remaining DSA layers reuse the nearest preceding
    publication within the same micro-batch
    (cppmega/megatron/index_cache_patch.py:37-278).
    """

    attention_ranks: Tuple[int, ...] = (1, 2, 3, 5, 6, 7, 9, 10, 11)
    index_n_heads: int = 32
    index_head_dim: int = 64
    index_topk: int = 256
    indexer_loss_coeff: float = 0.0
    warmup_dense: bool = False          # indexer warm-up: sparse layers attend densely while the KL loss trains the indexer
    index_cache: bool = True
    full_layer_ranks: Tuple[int, ...] = (0, 3, 6)
    indexer_dtype: str = "bf16"

    def __post_init__(self):
        _check(self.indexer_dtype == "bf16", "DSA indexer supports bf16 only")
        _check(self.index_topk > 0, "index_topk must be positive")


@dataclass(frozen=True)
class MoEConfig:
    """Mixture of experts (cppmega/recipes/megatron_args.py:47-57,108-135)."""

    num_experts: int = 16
    topk: int = 4
    expert_ffn: int = 896
    shared_expert_ffn: int = 1024
    score_function: str = "sigmoid"      # "sigmoid" | "softmax"
    expert_bias: bool = True
    bias_update_rate: float = 1e-3
    aux_loss_coeff: float = 1e-4
    router_dtype: str = "fp32"
    dispatcher: str = "alltoall"         # "alltoall" | "allgather" | "flex"
    flex_backend: str = "fused_p2p"      # peer-memory fused dispatch
    capacity_factor: Optional[float] = None
    norm_topk_prob: bool = True

    def __post_init__(self):
        _check(self.score_function in ("sigmoid", "softmax"), "score_function must be sigmoid|softmax")
        _check(self.dispatcher in ("alltoall", "allgather", "flex"), "dispatcher must be alltoall|allgather|flex")
        _check(1 <= self.topk <= self.num_experts, "topk must be in [1, num_experts]")


@dataclass(frozen=True)
class MTPConfig:
    """Multi-token prediction (cppmega/megatron/mtp_liger_ce.py:63-233)."""

    num_layers: int = 2
    loss_scaling_factor: float = 0.1
    fused_with_main_ce: bool = True
    # FastMTP alternative (cppmega/megatron/fastmtp_layer.py:32-47,389-406)
    fastmtp: bool = False
    fastmtp_depth: int = 3
    fastmtp_decay: float = 0.6
    fastmtp_lambda: float = 0.3


@dataclass(frozen=True)
class NgramHashConfig:
    """Hashed n-gram embedding (cppmega/features/engram/config.py:52-104)."""

    enabled: bool = True
    orders: Tuple[int, ...] = (2, 3)
    heads: int = 8
    table_size: int = 500_000
    embed_dim: int = 16
    dropout: float = 0.0
    offload: bool = False
    seed: int = 20240607

    def __post_init__(self):
        _check(len(self.orders) > 0 and all(o > 0 for o in self.orders), "ngram orders must be positive")
        _check(self.heads > 0 and self.table_size > 0 and self.embed_dim > 0, "ngram dims must be positive")

    @property
    def num_tables(self) -> int:
        return len(self.orders) * self.heads


@dataclass(frozen=True)
class StructureConfig:
    """Structure-aware additive embedding (cppmega/features/structure/embedding.py:15-69)."""

    enabled: bool = False
    components: str = "core"
    num_categories: int = 9
    max_dep_level: int = 16
    max_ast_depth: int = 64
    max_sibling_index: int = 64
    num_node_types: int = 256
    bottleneck_dim: int = 64


@dataclass(frozen=True)
class EngramConfig:
    """Per-layer n-gram memory branch; configuration surface only (no runtime in the
    reference either: cppmega/features/engram/config.py:13-50)."""

    enabled: bool = False
    layer_indices: Tuple[int, ...] = ()
    ngram_orders: Tuple[int, ...] = (2, 3, 4)
    bottleneck_dim: int = 0
    dropout: float = 0.0
    gated: bool = False


@dataclass(frozen=True)
class MHCConfig:
    """Sinkhorn hyper-connections; configuration surface only
    (cppmega/features/mhc/config.py:15)."""

    enabled: bool = False
    layer_indices: Tuple[int, ...] = ()
    n_streams: int = 4
    sinkhorn_iters: int = 5
    temperature: float = 1.0
    epsilon: float = 1e-6
    blend_alpha: float = 1.0
    dynamic: bool = False

    def __post_init__(self):
        _check(self.n_streams >= 1 and self.sinkhorn_iters >= 0, "invalid mHC sizes")
        _check(self.temperature > 0 and self.epsilon > 0, "mHC temperature/epsilon must be positive")


@dataclass(frozen=True)
class MoDConfig:
    """Mixture-of-depths routing; configuration surface only
    (cppmega/features/mod/config.py:11,75)."""

    enabled: bool = False
    layer_indices: Tuple[int, ...] = ()
    capacity: float = 0.5
    aux_loss_weight: float = 0.01
    routing: str = "topk"
    ffn_only: bool = False
    skip_first_n: int = 4
    skip_mamba: bool = True
    moda_enabled: bool = False

    def __post_init__(self):
        _check(0.0 < self.capacity <= 1.0, "MoD capacity must be in (0, 1]")
        _check(self.routing in ("topk", "threshold", "expert_choice"), "unknown MoD routing")


@dataclass(frozen=True)
class ModelConfig:
    name: str = "nam56r"
    pattern: str = "AEMEAEMEAEMR"
    depth: int = 52
    hidden_size: int = 4096
    ffn_hidden_size: int = 21504          # dense MLP (MTP layers, 'D' layers)
    vocab_size: int = 131072
    seq_length: int = 4096
    norm_eps: float = 1e-5
    init_std: float = 0.02
    tie_embeddings: bool = False
    mamba_variant: str = "mimo"           # "mimo" | "noconv_ssd" | "ssd" (see models/mamba_variants.py)
    mamba3: Mamba3Config = field(default_factory=Mamba3Config)
    m2rnn: M2RNNConfig = field(default_factory=M2RNNConfig)
    mla: MLAConfig = field(default_factory=MLAConfig)
    dsa: DSAConfig = field(default_factory=DSAConfig)
    moe: MoEConfig = field(default_factory=MoEConfig)
    mtp: MTPConfig = field(default_factory=MTPConfig)
    ngram_hash: NgramHashConfig = field(default_factory=NgramHashConfig)
    structure: StructureConfig = field(default_factory=StructureConfig)
    engram: EngramConfig = field(default_factory=EngramConfig)
    mhc: MHCConfig = field(default_factory=MHCConfig)
    mod: MoDConfig = field(default_factory=MoDConfig)

    def __post_init__(self):
        _check(self.hidden_size > 0 and self.vocab_size > 0 and self.depth > 0, "sizes must be positive")
        _check(self.mamba_variant in ("mimo", "noconv_ssd", "ssd"), "unknown mamba_variant")
        for feat, nm in ((self.engram, "engram"), (self.mhc, "mHC"), (self.mod, "MoD")):
            bad = [i for i in feat.layer_indices if i >= self.depth]
            _check(not bad, f"{nm} layer indices {bad} exceed depth={self.depth}")
        self.plan()  # validates the pattern

    # ---- derived layout -------------------------------------------------
    def plan(self) -> HybridPlan:
        return translate_pattern(self.pattern, self.depth, self.mtp.num_layers)

    def layer_kind(self, layer_number: int) -> str:
        """Kind of 1-indexed layer: mamba3 | m2rnn | dsa | mla | moe | mlp."""
        sym = self.plan().layer_symbols[layer_number - 1]
        if sym == "M":
            return "mamba3"
        if sym == "R":
            return "m2rnn"
        if sym == "E":
            return "moe"
        if sym == "D":
            return "mlp"
        if sym == "A":
            rank = attention_ranks(self.plan().layer_symbols)[layer_number]
            return "dsa" if rank in self.dsa.attention_ranks else "mla"
        raise ValueError(f"layer symbol {sym!r} has no runtime")

    def layer_kinds(self) -> Tuple[str, ...]:
        return tuple(self.layer_kind(i + 1) for i in range(self.depth))

    def dsa_rank_of_layer(self) -> dict:
        """1-indexed layer number -> rank among DSA layers."""
        out, r = {}, 0
        for i, k in enumerate(self.layer_kinds()):
            if k == "dsa":
                out[i + 1] = r
                r += 1
        return out

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)

    # ---- analytic counts -------------------------------------------------
    def param_count(self) -> dict:
        """Analytic parameter counts: total and active-per-token."""
        h = self.hidden_size
        m3, mla, moe = self.mamba3, self.mla, self.moe
        per = {}
        nh = m3.nheads(h)
        per["mamba3"] = (
            h                                                   # pre-norm
            + h * sum(m3.in_proj_sizes(h))                      # in_proj
            + h * m3.num_rope_angles                            # angle_proj
            + 2 * m3.d_state                                    # B/C norm
            + nh * (2 + 2 * m3.mimo_rank * m3.d_state + 3 * m3.mimo_rank * m3.headdim)
            + m3.d_inner(h) * h                                 # out_proj
        )
        r = self.m2rnn
        rh = r.heads(h)
        conv_dim = (r.num_q_heads + r.num_k_heads) * r.k_head_dim + rh * r.v_head_dim
        per["m2rnn"] = (
            h + h * (conv_dim + rh + rh * r.v_head_dim)
            + conv_dim * (r.conv_kernel + 1) + rh * r.v_head_dim * r.v_head_dim
            + 2 * rh + rh * r.v_head_dim * 2 + rh * r.v_head_dim * h
        )
        attn = (
            h + h * mla.q_lora_rank + mla.q_lora_rank
            + mla.q_lora_rank * mla.num_heads * mla.q_head_dim
            + h * (mla.kv_lora_rank + mla.qk_pos_emb_head_dim) + mla.kv_lora_rank
            + mla.kv_lora_rank * mla.num_heads * (mla.qk_head_dim + mla.v_head_dim)
            + mla.num_heads * mla.v_head_dim * h
        )
        per["mla"] = attn
        d = self.dsa
        per["dsa"] = attn + (
            mla.q_lora_rank * d.index_n_heads * d.index_head_dim
            + h * d.index_head_dim + d.index_head_dim + h * d.index_n_heads
        )
        expert = 3 * h * moe.expert_ffn
        shared = 3 * h * moe.shared_expert_ffn if moe.shared_expert_ffn else 0
        per["moe"] = h + h * moe.num_experts + (moe.num_experts if moe.expert_bias else 0) + moe.num_experts * expert + shared
        per["moe_active"] = h + h * moe.num_experts + moe.topk * expert + shared
        per["mlp"] = h + 3 * h * self.ffn_hidden_size
        total = active = 0
        for k in self.layer_kinds():
            total += per[k]
            active += per["moe_active"] if k == "moe" else per[k]
        emb = self.vocab_size * h
        ng = self.ngram_hash
        extra = 0
        if ng.enabled:
            extra += ng.num_tables * ng.table_size * ng.embed_dim + ng.num_tables * ng.embed_dim * h
        head = 0 if self.tie_embeddings else emb
        mtp = self.mtp.num_layers * (2 * h + 2 * h * h + per["mla"] + per["mlp"] + h)
        base = emb + head + h + extra + mtp
        return {"total": total + base, "active": active + base, "per_layer": per}

    def flops_per_token(self, seq_len: Optional[int] = None) -> float:
        """Approximate training FLOPs per token: 6 x active matmul params plus
        attention/scan terms (forward x3)."""
        s = seq_len or self.seq_length
        pc = self.param_count()
        dense = 6.0 * (pc["active"] - self.vocab_size * self.hidden_size)  # embedding gather is free
        m3 = self.mamba3
        nh = m3.nheads(self.hidden_size)
        L = m3.chunk_size * m3.mimo_rank
        scan = 2.0 * nh * m3.mimo_rank * (2 * m3.d_state * m3.headdim + L * (m3.d_state + m3.headdim))
        kinds = self.layer_kinds()
        n_m = sum(k == "mamba3" for k in kinds)
        n_mla = sum(k == "mla" for k in kinds) + self.mtp.num_layers
        n_dsa = sum(k == "dsa" for k in kinds)
        mla = self.mla
        att_full = 2.0 * mla.num_heads * (mla.q_head_dim + mla.v_head_dim) * s / 2
        att_sparse = 2.0 * mla.num_heads * (mla.kv_lora_rank + mla.qk_pos_emb_head_dim + mla.kv_lora_rank) * min(self.dsa.index_topk, s)
        idx = 2.0 * self.dsa.index_n_heads * self.dsa.index_head_dim * s / 2
        n_full_idx = len([r for r in range(n_dsa) if (not self.dsa.index_cache) or r in self.dsa.full_layer_ranks])
        return dense + 3.0 * (n_m * scan + n_mla * att_full + n_dsa * att_sparse + n_full_idx * idx)


# ---------------------------------------------------------------------------
# presets
# ---------------------------------------------------------------------------

def nam56r_full(**overrides) -> ModelConfig:
    """NAM56R production width: 52 layers, hidden 4096, 32 heads x 128, d_state 128,
    MIMO rank 4, 16 experts top-4 + shared, DSA top-k 256, 2 MTP depths, vocab 131072
    (cppmega/recipes/run_profiles.py:439-449, scripts/remote_smoke_h200_dsa_9_4_m.sh:706-710)."""
    return ModelConfig(**overrides)


def nam56r_tiny(**overrides) -> ModelConfig:
    """CPU plumbing configuration: 8 layers ``M E M E A(DSA) E M E``, hidden 256."""
    base = dict(
        name="nam56r_tiny",
        pattern="MEMEAEME",
        depth=8,
        hidden_size=256,
        ffn_hidden_size=512,
        vocab_size=4096,
        seq_length=256,
        mamba3=Mamba3Config(d_state=32, headdim=64, ngroups=2, mimo_rank=4, chunk_size=16),
        m2rnn=M2RNNConfig(k_head_dim=16, v_head_dim=16),
        mla=MLAConfig(num_heads=4, q_lora_rank=64, kv_lora_rank=64, qk_head_dim=32,
                      qk_pos_emb_head_dim=32, v_head_dim=64),
        dsa=DSAConfig(attention_ranks=(0,), index_n_heads=4, index_head_dim=32, index_topk=32,
                      full_layer_ranks=(0,)),
        moe=MoEConfig(num_experts=4, topk=2, expert_ffn=512, shared_expert_ffn=512),
        mtp=MTPConfig(num_layers=1),
        ngram_hash=NgramHashConfig(orders=(2, 3), heads=4, table_size=4096, embed_dim=16),
    )
    base.update(overrides)
    return ModelConfig(**base)


def nam56r_quarter(**overrides) -> ModelConfig:
    """13-layer quarter model used for single-GPU correctness lanes
    (cppmega/recipes/run_profiles.py:48-58 `local_gb10_quarter`)."""
    base = dict(
        name="nam56r_quarter", pattern="AEMEAEMEAEMR", depth=13, hidden_size=3584,
        ffn_hidden_size=18944, vocab_size=65536,
        mla=MLAConfig(num_heads=28),
        dsa=DSAConfig(attention_ranks=(1, 2), full_layer_ranks=(0,)),
        mtp=MTPConfig(num_layers=1),
    )
    base.update(overrides)
    return ModelConfig(**base)


def nam56r_slice(**overrides) -> ModelConfig:
    """One layer of every kind at the production kernel shapes (``M A(DSA) E R``: Mamba3 MIMO d_state 128 / headdim 64 /
    rank 4, 32-head MLA with 64+64 query dims, indexer 32 x 64 with top-k 256, 16 experts top-4, M2RNN 64 x 16) behind a
    small hidden size and vocabulary: the smallest model on which every hand-written kernel accepts its shapes."""
    base = dict(
        name="nam56r_slice", pattern="MAER", depth=4, hidden_size=1024, ffn_hidden_size=2048, vocab_size=8192,
        seq_length=512,
        dsa=DSAConfig(attention_ranks=(0,), full_layer_ranks=(0,)),
        mtp=MTPConfig(num_layers=1),
        ngram_hash=NgramHashConfig(orders=(2, 3), heads=4, table_size=4096, embed_dim=16),
    )
    base.update(overrides)
    return ModelConfig(**base)


PRESETS = {
    "nam56r": nam56r_full,
    "nam56r_full": nam56r_full,
    "nam56r_tiny": nam56r_tiny,
    "nam56r_quarter": nam56r_quarter,
    "nam56r_slice": nam56r_slice,
}


def get_preset(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return PRESETS[name](**overrides)


def human_count(n: float) -> str:
    for unit, div in (("T", 1e12), ("B", 1e9), ("M", 1e6), ("K", 1e3)):
        if abs(n) >= div:
            return f"{n / div:.2f}{unit}"
    return f"{n:.0f}"


__all__ = [
    "Mamba3Config", "M2RNNConfig", "MLAConfig", "DSAConfig", "MoEConfig", "MTPConfig",
    "NgramHashConfig", "StructureConfig", "EngramConfig", "MHCConfig", "MoDConfig", "ModelConfig",
    "nam56r_full", "nam56r_tiny", "nam56r_quarter", "nam56r_slice", "get_preset", "PRESETS", "human_count",
]
_ = math  # keep import for downstream formulas
