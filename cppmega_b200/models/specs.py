"""Stack specs: named descriptions of which module implements each symbol of the hybrid pattern.

The reference selects a stack with ``--spec <module> <builder>`` (cppmega/megatron/nam56r_full_spec.py:205-259 is the
production one; ``nam56r_noconv_spec.py``, ``nam56r_lite_spec.py``, ``mamba_local_spec.py``, ``dsa_local_spec.py`` are
the alternatives).  Here a spec is data: it maps pattern symbols to layer kinds and fixes the model-config switches
that the corresponding reference spec implies; ``apply_spec`` returns the ``ModelConfig`` to build and
``describe_stack`` lists, layer by layer, what will be instantiated (the reference's layout report,
cppmega/megatron/nam56r_layout.py).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, List, Tuple

from ..config.model import ModelConfig

MODULE_OF_KIND = {
    "mamba3": "cppmega_b200.models.mamba3.Mamba3Mixer",
    "m2rnn": "cppmega_b200.models.m2rnn.M2RNNMixer",
    "mla": "cppmega_b200.models.attention.MLAttention",
    "dsa": "cppmega_b200.models.attention.MLAttention(sparse)",
    "moe": "cppmega_b200.models.moe.MoELayer",
    "mlp": "cppmega_b200.models.common.DenseMLP",
}


@dataclass(frozen=True)
class StackSpec:
    name: str
    description: str
    mamba_variant: str = "mimo"            # which module answers for an ``M`` symbol
    use_dsa: bool = True                   # False: every ``A`` is dense MLA
    use_m2rnn: bool = True                 # False: ``R`` symbols run the Mamba mixer
    use_moe: bool = True                   # False: ``E`` symbols are dense MLPs
    mtp: bool = True


SPECS: Dict[str, StackSpec] = {s.name: s for s in (
    StackSpec("nam56r_full", "production stack: Mamba3 MIMO + M2RNN + MLA/DSA by attention rank + MoE + MTP"),
    StackSpec("nam56r_noconv", "'branch B': no-convolution SSD mixer with Mamba3 B/C features + M2RNN",
              mamba_variant="noconv_ssd"),
    StackSpec("nam56r_lite", "dense-attention lite stack: every A is MLA, R runs the Mamba mixer",
              use_dsa=False, use_m2rnn=False),
    StackSpec("mamba_local", "local smoke stack: classic SSD (conv1d) mixer, dense MLP instead of MoE, no MTP",
              mamba_variant="ssd", use_dsa=False, use_m2rnn=False, use_moe=False, mtp=False),
    StackSpec("dsa_local", "local DSA smoke stack: sparse attention everywhere an A rank asks for it, dense MLP",
              use_moe=False, mtp=False),
)}


def get_spec(name: str) -> StackSpec:
    if name not in SPECS:
        raise KeyError(f"unknown stack spec {name!r}; known: {sorted(SPECS)}")
    return SPECS[name]


def apply_spec(cfg: ModelConfig, spec: StackSpec) -> ModelConfig:
    """The model configuration that realises ``spec`` on top of ``cfg`` (same sizes, same pattern)."""
    upd = {"mamba_variant": spec.mamba_variant}
    if not spec.use_dsa:
        upd["dsa"] = dataclasses.replace(cfg.dsa, attention_ranks=())
    if not spec.mtp:
        upd["mtp"] = dataclasses.replace(cfg.mtp, num_layers=0)
    pattern = cfg.pattern
    if not spec.use_m2rnn:
        pattern = pattern.replace("R", "M")
    if not spec.use_moe:
        pattern = pattern.replace("E", "D")           # D: dense MLP symbol of the pattern language
    upd["pattern"] = pattern
    return dataclasses.replace(cfg, **upd)


def describe_stack(cfg: ModelConfig) -> List[Tuple[int, str, str]]:
    """[(layer number, kind, implementing module)] for the whole depth."""
    out = []
    for i, kind in enumerate(cfg.layer_kinds(), start=1):
        mod = MODULE_OF_KIND.get(kind, kind)
        if kind == "mamba3" and cfg.mamba_variant != "mimo":
            mod = f"cppmega_b200.models.mamba_variants.SSDMixer[{cfg.mamba_variant}]"
        out.append((i, kind, mod))
    return out


def custom_layer_indices(cfg: ModelConfig) -> Dict[str, List[int]]:
    """1-indexed layer numbers per kind (cppmega/recipes/nam56r_launch.py:97 ``get_custom_layer_indices``)."""
    idx: Dict[str, List[int]] = {}
    for i, kind in enumerate(cfg.layer_kinds(), start=1):
        idx.setdefault(kind, []).append(i)
    return idx
