"""FP8 compression of the activations that autograd keeps for backward.

Inside :func:`fp8_activation_context` every bf16 tensor that an operator saves for its backward (and every layer
input that a recomputed layer keeps) is stored as E4M3 bytes plus scales - half the bytes - and expanded back to bf16
when backward asks for it.  Two scale layouts on the same quantiser kernels (``ops/csrc/mxfp8.cu``):

* ``"mxfp8"``   one E8M0 scale per 32 consecutive values (block scaling: outliers cost one block, not the tensor);
* ``"tensor"``  one power-of-two scale for the whole tensor from its current absolute maximum, measured on the device
                (no host read-back); ``clamp=True`` limits that maximum to the E4M3 range first, so outliers saturate
                instead of flattening everything else.

Layer awareness: the layer loop publishes the index of the running layer (:func:`set_current_layer_idx`); the first
``bf16_first`` and last ``bf16_last`` layers keep bf16.  Modules that must keep exact saved tensors wrap their forward
in :class:`fp8_quantize_disabled` (also usable as the decorator :func:`no_fp8_quantize`).  Parameters, integer /
boolean tensors, fp32 tensors (softmax statistics, scan states) and tensors below ``min_elements`` pass through.

Counterpart of the reference's saved-tensor hooks (cppmega/megatron/fp8_activations.py:598-653 packer, :155-230 opt-out,
:246-270 first/last bf16 layers, :784-818 layer-aware packer, :820-878 context factory), on this package's own kernels
instead of Transformer Engine / Triton; the COAT backend and the inductor budget helper have no counterpart here.
"""
from __future__ import annotations

import functools
import threading
import weakref
from contextlib import nullcontext
from dataclasses import dataclass
from typing import Any, Optional, Tuple

import torch

MIN_ELEMENTS = 16384            # below this the two extra kernels cost more than the bytes saved (32 KB of bf16)
E4M3_MAX = 448.0

_state = threading.local()
STATS = {"packed": 0, "shared": 0, "passed": 0, "bytes_in": 0, "bytes_out": 0}


def reset_stats() -> None:
    for k in STATS:
        STATS[k] = 0


# ---- opt-out and layer index ------------------------------------------------------------------------------------------
class fp8_quantize_disabled:
    """``with fp8_quantize_disabled(): ...`` - tensors saved inside keep their dtype (nests; thread-local)."""

    def __enter__(self):
        _state.disabled = getattr(_state, "disabled", 0) + 1
        return self

    def __exit__(self, *exc):
        _state.disabled -= 1
        return False


def no_fp8_quantize(fn):
    """Decorator form of :class:`fp8_quantize_disabled` for a module's ``forward``."""

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        with fp8_quantize_disabled():
            return fn(*args, **kwargs)

    return wrapper


def _disabled() -> bool:
    return getattr(_state, "disabled", 0) > 0


def set_current_layer_idx(idx: int) -> None:
    """Called by the layer loop before each layer (0-based position in the stack); -1 = outside the stack."""
    _state.layer = idx


def current_layer_idx() -> int:
    return getattr(_state, "layer", -1)


def is_bf16_layer(layer_idx: int, n_layers: int, bf16_first: int, bf16_last: int) -> bool:
    if layer_idx < 0:
        return False
    return (bf16_first > 0 and layer_idx < bf16_first) or (bf16_last > 0 and layer_idx >= n_layers - bf16_last)


# ---- packer -----------------------------------------------------------------------------------------------------------
@dataclass(eq=False)
class PackedActivation:
    payload: torch.Tensor           # uint8 / float8_e4m3fn bytes, flat [rows, cols]
    scales: torch.Tensor            # uint8 E8M0, [rows, cols / 32]
    shape: Tuple[int, ...]
    dtype: torch.dtype


def _is_weight(t: torch.Tensor) -> bool:
    """A trainable leaf or a view of one (``w.t()`` saved by a matrix product): parameters are not activations."""
    if t.is_leaf and t.requires_grad:
        return True
    base = t._base
    return base is not None and base.is_leaf and base.requires_grad


def _as_rows(t: torch.Tensor) -> Optional[torch.Tensor]:
    """Contiguous 2-D view [rows, cols] with ``cols % 32 == 0`` (the last dimension when it allows, else rows of 32)."""
    n = t.numel()
    if n % 32:
        return None
    t = t.contiguous()
    cols = t.shape[-1] if (t.dim() >= 1 and t.shape[-1] % 32 == 0) else 32
    return t.view(n // cols, cols)


class Fp8ActivationPacker:
    """``pack`` / ``unpack`` pair for ``torch.autograd.graph.saved_tensors_hooks``."""

    def __init__(self, recipe: str = "mxfp8", clamp: bool = False, min_elements: int = MIN_ELEMENTS):
        if recipe not in ("mxfp8", "tensor"):
            raise ValueError(f"fp8 activation recipe must be 'mxfp8' or 'tensor', not {recipe!r}")
        self.recipe, self.clamp, self.min_elements = recipe, clamp, min_elements
        # one packed copy per distinct tensor: a normed activation that feeds three linears is saved three times
        self._seen: "weakref.WeakValueDictionary" = weakref.WeakValueDictionary()

    def pack(self, t: Any) -> Any:
        if (not isinstance(t, torch.Tensor) or _disabled() or t.dtype != torch.bfloat16 or t.numel() < self.min_elements
                or isinstance(t, torch.nn.Parameter) or _is_weight(t)):
            STATS["passed"] += 1
            return t
        key = (t.data_ptr(), t._version, tuple(t.shape), tuple(t.stride()))
        hit = self._seen.get(key)
        if hit is not None:
            STATS["shared"] += 1
            return hit
        x = _as_rows(t)
        if x is None:
            STATS["passed"] += 1
            return t
        if x.is_cuda:
            from ..ops.cuda import mxfp8 as mx
            tw = None
            if self.recipe == "tensor":
                tw = mx.tensor_amax(x)
                if self.clamp:
                    tw.clamp_(max=E4M3_MAX)
            q = mx.quantize_rowwise(x, tensorwise=tw)
            payload, scales = q.payload, q.scales
        else:
            from ..ops import reference as ref
            if self.recipe == "tensor":
                am = x.float().abs().amax()
                if self.clamp:
                    am = am.clamp(max=E4M3_MAX)
                sc = ref.e8m0_from_amax(am)
                mult = torch.exp2(127.0 - sc.float())
                payload = (x.float() * mult).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
                scales = sc.reshape(1, 1).expand(x.shape[0], x.shape[1] // 32).contiguous()
            else:
                payload, scales = ref.mxfp8_quantize(x)
        STATS["packed"] += 1
        STATS["bytes_in"] += t.numel() * 2
        STATS["bytes_out"] += payload.numel() + scales.numel()
        packed = PackedActivation(payload, scales, tuple(t.shape), t.dtype)
        self._seen[key] = packed
        return packed

    @staticmethod
    def unpack(p: Any) -> Any:
        if not isinstance(p, PackedActivation):
            return p
        if p.payload.is_cuda:
            from ..ops.cuda import mxfp8 as mx
            out = mx.dequantize(mx.Mxfp8Tensor(p.payload, p.scales, tuple(p.payload.shape), None))
        else:
            from ..ops import reference as ref
            out = ref.mxfp8_dequantize(p.payload, p.scales).to(p.dtype)
        return out.view(p.shape)


class LayerAwareFp8Packer(Fp8ActivationPacker):
    """Same, but the first ``bf16_first`` and last ``bf16_last`` layers of the stack keep their saved tensors in bf16."""

    def __init__(self, n_layers: int, bf16_first: int = 1, bf16_last: int = 1, **kw):
        super().__init__(**kw)
        self.n_layers, self.bf16_first, self.bf16_last = n_layers, bf16_first, bf16_last

    def pack(self, t: Any) -> Any:
        if is_bf16_layer(current_layer_idx(), self.n_layers, self.bf16_first, self.bf16_last):
            STATS["passed"] += 1
            return t
        return super().pack(t)


def fp8_activation_context(*, recipe: str = "mxfp8", n_layers: int = 0, bf16_first: int = 0, bf16_last: int = 0,
                           clamp: bool = False, min_elements: int = MIN_ELEMENTS, enabled: bool = True):
    """Context manager under which saved activations are FP8-compressed (``enabled=False``: a no-op context)."""
    if not enabled or recipe in (None, "", "off", "none"):
        return nullcontext()
    if bf16_first > 0 or bf16_last > 0:
        packer: Fp8ActivationPacker = LayerAwareFp8Packer(n_layers, bf16_first, bf16_last, recipe=recipe, clamp=clamp,
                                                          min_elements=min_elements)
    else:
        packer = Fp8ActivationPacker(recipe=recipe, clamp=clamp, min_elements=min_elements)
    return torch.autograd.graph.saved_tensors_hooks(packer.pack, packer.unpack)
