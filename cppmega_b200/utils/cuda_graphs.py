"""CUDA-graph capture of static layer regions.

A layer whose shapes and control flow never change between steps (Mamba3 / M2RNN mixers, dense MLA attention, dense
MLP) can be captured once (forward and backward as two graphs over static buffers) and replayed with two launches per
micro-batch instead of several dozen.  ``scope`` names follow the reference's scoped graphs
(``--cuda-graph-scope attn mamba moe_router moe_preprocess``, scripts/remote_smoke_h200_dsa_9_4_m.sh:559-565):

    mamba   Mamba3 and M2RNN layers
    attn    dense MLA layers (DSA layers choose their keys on the host side of the IndexCache and stay eager)
    mlp     dense MLP layers

MoE layers are not capturable here: the dispatch plan is sized from the routing result on the host.  The reference
keeps graphs off in its production configuration because their private pools cost 39-63 GiB at MBS >= 8
(docs/production_status.md:32-36); the same trade applies (static input / output / saved-tensor buffers per captured
layer), so the default scope is empty.

Captured layers cannot take part in activation recomputation, and their weight gradients come back as ordinary
tensors (the GEMM-epilogue accumulation into the flat gradient buffer is a Python-visible side effect that a replay
would not repeat), so capture switches that off for their parameters.

``forbid_host_sync`` is the guard the reference applies by patching (upstream_patches/apply_dsa_cg_patches.py:58-75):
inside it any implicit device-to-host synchronisation raises instead of silently breaking a capture.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Iterable, List, Sequence, Tuple

import torch
import torch.nn as nn

SCOPE_KINDS: Dict[str, Tuple[str, ...]] = {"mamba": ("mamba3", "m2rnn"), "attn": ("mla",), "mlp": ("mlp",)}
NOT_CAPTURABLE = ("moe_router", "moe_preprocess", "moe")


def parse_scope(scope: Iterable[str]) -> Tuple[str, ...]:
    """Validate scope names; MoE scopes are accepted and ignored with a reason (see the module docstring)."""
    kinds: List[str] = []
    for name in scope:
        name = name.strip().lower()
        if not name or name in NOT_CAPTURABLE:
            continue
        if name not in SCOPE_KINDS:
            raise ValueError(f"unknown CUDA-graph scope {name!r}; known: {sorted(SCOPE_KINDS) + list(NOT_CAPTURABLE)}")
        kinds += [k for k in SCOPE_KINDS[name] if k not in kinds]
    return tuple(kinds)


@contextlib.contextmanager
def forbid_host_sync(enabled: bool = True):
    """Raise on any implicit host synchronisation inside the block (no-op without CUDA)."""
    if not enabled or not torch.cuda.is_available():
        yield
        return
    prev = torch.cuda.get_sync_debug_mode()
    torch.cuda.set_sync_debug_mode("error")
    try:
        yield
    finally:
        torch.cuda.set_sync_debug_mode(prev)


class _LayerBody(nn.Module):
    """Single-tensor view of a layer, which is what graph capture wants."""

    def __init__(self, layer: nn.Module):
        super().__init__()
        self.layer = layer

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.layer(x)


class GraphedLayer(nn.Module):
    """Drop-in replacement of a captured layer: replays the graphs in training, runs the eager layer otherwise (other
    shapes, evaluation, no CUDA)."""

    def __init__(self, layer: nn.Module, graphed, sample_shape: Sequence[int], dtype: torch.dtype):
        super().__init__()
        self.layer, self._graphed = layer, graphed
        self._shape, self._dtype = tuple(sample_shape), dtype
        self.kind = getattr(layer, "kind", None)
        self.layer_number = getattr(layer, "layer_number", None)
        self.replays = 0

    def forward(self, x: torch.Tensor, *args, **kwargs) -> torch.Tensor:
        # the captured kinds ignore the index cache / preselected indices that the stack passes to every layer
        if self.training and torch.is_grad_enabled() and x.is_cuda and tuple(x.shape) == self._shape and x.dtype == self._dtype:
            self.replays += 1
            return self._graphed(x)
        return self.layer(x, *args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("layer"), name)


def capture_layer(layer: nn.Module, sample_shape: Sequence[int], dtype: torch.dtype, device, warmup: int = 3) -> GraphedLayer:
    for p in layer.parameters():
        p.fuse_wgrad_accumulation = False
        p.cuda_graphed = True
    sample = torch.randn(*sample_shape, device=device, dtype=dtype, requires_grad=True)
    body = _LayerBody(layer)
    graphed = torch.cuda.make_graphed_callables(body, (sample,), num_warmup_iters=warmup)
    return GraphedLayer(layer, graphed, sample_shape, dtype)


def capture_model_layers(model: nn.Module, scope: Iterable[str], sample_shape: Sequence[int], dtype: torch.dtype, device,
                         warmup: int = 3) -> int:
    """Replace every layer of ``model.decoder.layers`` (or ``model.layers``) whose kind is in ``scope`` by its captured version.  Returns how many
    layers were captured.  Call after the optimizer has registered its hooks and before the first step."""
    kinds = parse_scope(scope)
    if not kinds or not torch.cuda.is_available():
        return 0
    layers = getattr(getattr(model, "decoder", model), "layers", None)
    if layers is None:
        return 0
    keys = list(layers.keys()) if isinstance(layers, nn.ModuleDict) else list(range(len(layers)))
    n = 0
    for key in keys:
        layer = layers[key]
        if getattr(layer, "kind", None) in kinds and not isinstance(layer, GraphedLayer):
            layers[key] = capture_layer(layer, sample_shape, dtype, device, warmup)
            n += 1
    return n
