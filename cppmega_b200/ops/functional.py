"""Operator front door.

Every model calls the functions here.  On a CUDA tensor they run the sm_100a
kernels from :mod:`cppmega_b200.ops.cuda` (wrapped in autograd Functions); on a CPU
tensor they run the PyTorch definitions in :mod:`cppmega_b200.ops.reference`.  A CUDA call
for which no kernel is registered is counted in :func:`fallback_counts` and runs
the PyTorch definition on the GPU, so a training log can prove "zero fallbacks"
(the reference keeps equivalent counters for its MXFP8 routing,
scripts/cppmega_fp8_shim.py:445-500).  If the extension failed to load on a machine
that has a GPU, the first CUDA call raises instead of silently falling back.
"""
from __future__ import annotations

import collections
from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F

from . import reference as ref
from . import mimo_scan_ref

_CUDA_IMPL: Dict[str, Callable] = {}
_FALLBACKS: "collections.Counter[str]" = collections.Counter()
_LAUNCHES: "collections.Counter[str]" = collections.Counter()
_DISABLED: set = set()
_ext_checked = False


def register_cuda(name: str, fn: Callable) -> None:
    _CUDA_IMPL[name] = fn


def disable_cuda(*names: str) -> None:
    """Route the named ops through the PyTorch definitions (used by A/B benchmarks)."""
    _DISABLED.update(names)


def enable_cuda(*names: str) -> None:
    for n in names:
        _DISABLED.discard(n)


# kernels whose reductions use floating-point atomics (the order of the additions, hence the last bits, varies from run to run)
ATOMIC_REDUCTION_OPS = ("embedding", "ngram_hash_embed", "causal_conv1d_silu", "head_linear", "sparse_mla", "mimo_scan_bwd",
                        "causal_attention")
_deterministic = False


def set_deterministic(on: bool = True) -> None:
    """Bitwise-reproducible reruns for debugging: the operators in ``ATOMIC_REDUCTION_OPS`` go through their PyTorch
    definitions and the tensor library is put in deterministic mode (it then refuses or replaces its own atomic kernels).
    Slower; meant for comparing two runs of a few steps, e.g. when hunting a race in a new kernel."""
    global _deterministic
    _deterministic = bool(on)
    if on:
        disable_cuda(*ATOMIC_REDUCTION_OPS)
    else:
        enable_cuda(*ATOMIC_REDUCTION_OPS)
    torch.use_deterministic_algorithms(bool(on), warn_only=True)


def is_deterministic() -> bool:
    return _deterministic


def fallback_counts() -> Dict[str, int]:
    return dict(_FALLBACKS)


def launch_counts() -> Dict[str, int]:
    """Number of calls that reached one of this package's own CUDA kernels, per op."""
    return dict(_LAUNCHES)


def reset_counters() -> None:
    _FALLBACKS.clear()
    _LAUNCHES.clear()


def count_launch(name: str, n: int = 1) -> None:
    _LAUNCHES[name] += n


def _ensure_ext() -> None:
    global _ext_checked
    if _ext_checked:
        return
    _ext_checked = True
    from . import cuda  # noqa: F401  (registers kernels; raises if the .so is missing on a GPU box)


def _miss(name: str, t: torch.Tensor) -> None:
    """A CUDA call that ends in a PyTorch / library kernel instead of one of this package's kernels."""
    if t.is_cuda:
        _FALLBACKS[name] += 1


def _cuda(name: str, *tensors) -> Optional[Callable]:
    t = tensors[0]
    if not t.is_cuda:
        return None
    _ensure_ext()
    fn = _CUDA_IMPL.get(name)
    if fn is None or name in _DISABLED:
        _FALLBACKS[name] += 1
        return None
    return fn


# ---- dense ---------------------------------------------------------------

_PRECISION_RECIPE = "bf16"
RECIPES = ("bf16", "mxfp8", "tensorwise")


def set_precision_recipe(name: str) -> None:
    """Precision of the linear layers (2-D bf16 weight, all three dims multiples of 32) and the expert GEMMs:

    * ``bf16``: bf16 operands;
    * ``mxfp8``: operands rounded to E4M3 with one E8M0 scale per 32 values along the reduced dimension; the activation
      saved for the weight gradient is kept in that form;
    * ``tensorwise``: E4M3 with ONE power-of-two scale per tensor, measured from the tensor at every use (current
      scaling) - the reference's production FP8 recipe (docs/production_status.md:13-18) on the same kernels.

    This is the process-wide default; :func:`precision_scope` and :func:`install_precision_rules` narrow it to modules."""
    global _PRECISION_RECIPE
    if name not in RECIPES:
        raise ValueError(f"unknown precision recipe {name!r}")
    _PRECISION_RECIPE = name


def precision_recipe() -> str:
    return _PRECISION_RECIPE


class precision_scope:
    """``with precision_scope("mxfp8"): ...`` - the recipe of every linear called inside (forward; each op remembers its
    recipe for its backward)."""

    def __init__(self, name: str):
        if name not in RECIPES:
            raise ValueError(f"unknown precision recipe {name!r}")
        self.name = name

    def __enter__(self):
        self.prev = _PRECISION_RECIPE
        set_precision_recipe(self.name)
        return self

    def __exit__(self, *exc):
        set_precision_recipe(self.prev)
        return False


def install_precision_rules(model, rules, default: str = "bf16"):
    """Per-module precision selection.  ``rules``: sequence of ``(glob pattern, recipe)`` matched against the qualified
    module names of ``model`` (first match wins; e.g. ``("*.mixer.in_proj", "mxfp8")`` or ``("decoder.layers.*.mlp",
    "tensorwise")``); modules that match run their forward under that recipe, everything else under ``default``.
    Counterpart of the reference's layer-selective FP8 (cppmega/megatron/selective_fp8_moe_patch.py:60-149: FP8 on MoE
    layers only) and of its per-module precision file (configs/te_precision/mamba_mxfp8_eval_bf16.yaml:1-29: MXFP8 on
    the Mamba in / out projections only).  Returns ``(handles, matched module names)``; ``h.remove()`` undoes a hook."""
    import fnmatch
    set_precision_recipe(default)
    handles, matched = [], []
    for name, mod in model.named_modules():
        recipe = next((r for pat, r in rules if fnmatch.fnmatchcase(name, pat)), None)
        if recipe is None:
            continue
        if recipe not in RECIPES:
            raise ValueError(f"unknown precision recipe {recipe!r} for pattern matching {name!r}")
        stack = []

        def pre(_m, _args, recipe=recipe, stack=stack):
            stack.append(_PRECISION_RECIPE)
            set_precision_recipe(recipe)

        def post(_m, _args, _out, stack=stack):
            set_precision_recipe(stack.pop())

        handles.append(mod.register_forward_pre_hook(pre))
        handles.append(mod.register_forward_hook(post, always_call=True))
        matched.append(name)
    return handles, matched


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w^T``; w is [out, in]."""
    if _PRECISION_RECIPE != "bf16" and x.is_cuda:
        _ensure_ext()
        from .cuda import mxfp8
        y = mxfp8.linear(x, w, tensorwise=_PRECISION_RECIPE == "tensorwise")
        if y is not None:
            return y
        _FALLBACKS["fp8_linear(shape)"] += 1
    fn = _cuda("linear", x)
    if fn is not None:
        y = fn(x, w)
        if y is not None:
            return y
        _miss("linear(shape/dtype)", x)
    return F.linear(x, w.to(x.dtype) if w.dtype != x.dtype else w)


def linear_fp32out(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """fp32 ``x @ weight.T`` for an fp32 parameter.  On the GPU with bf16 activations the products run on the tensor
    cores (bf16 operands, fp32 accumulation and output); elsewhere plain fp32."""
    fn = _cuda("linear_fp32out", x) if x.is_cuda and x.dtype == torch.bfloat16 else None
    if fn is not None:
        y = fn(x, weight)
        if y is not None:
            return y
    _miss("linear_fp32out(shape/dtype)", x)
    return F.linear(x.float(), weight.float())


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, counts_host=None) -> torch.Tensor:
    """Rows of x sorted by expert; w [E, out, in]; counts [E] rows per expert."""
    fn = _cuda("grouped_linear", x)
    if fn is not None:
        y = fn(x, w, counts, counts_host)
        if y is not None:
            return y
        _miss("grouped_linear(shape)", x)
    ch = counts_host if counts_host is not None else counts.tolist()
    return ref.grouped_gemm(x, w.transpose(1, 2).to(x.dtype), ch)


def moe_experts(x_sorted: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, counts: torch.Tensor, counts_host=None):
    """SwiGLU expert MLP over expert-sorted rows: ``fc2(swiglu(fc1(x)))`` with per-expert weights
    ``w1`` [E, 2F, H] and ``w2`` [E, H, F]."""
    fn = _cuda("moe_experts", x_sorted)
    if fn is not None:
        y = fn(x_sorted, w1, w2, counts)
        if y is not None:
            return y
    h = grouped_linear(x_sorted, w1, counts, counts_host)
    return grouped_linear(swiglu(h), w2, counts, counts_host)


# ---- norms / activations ---------------------------------------------------

def rmsnorm(x, weight, eps: float = 1e-5):
    fn = _cuda("rmsnorm", x)
    if fn is not None:
        return fn(x, weight, eps)
    return ref.rmsnorm(x, weight, eps)


def rmsnorm_gated(x, weight, z=None, eps: float = 1e-5, group_size=None, norm_before_gate=True):
    _miss("rmsnorm_gated", x)          # PyTorch definition on every device
    return ref.rmsnorm_gated(x, weight, z, eps, group_size, norm_before_gate)


def head_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Per-head product ``y[..., h, :] = x[..., h, :] @ w[h]^T`` with ``x`` [..., H, in] and ``w`` [H, out, in] (the
    absorbed MLA up-projections of the sparse-attention path).  64-wide heads in bf16 run on the streaming tcgen05 kernel;
    anything else is a batched library GEMM and is counted."""
    fn = _cuda("head_linear", x)
    if fn is not None:
        y = fn(x, w)
        if y is not None:
            return y
    _miss("head_linear(library bmm)", x)
    return torch.einsum("...hi,hoi->...ho", x, w.to(x.dtype))


def swiglu(gate_up):
    fn = _cuda("swiglu", gate_up)
    if fn is not None:
        return fn(gate_up)
    return ref.swiglu(gate_up)


def apply_rope(x, cos, sin):
    fn = _cuda("apply_rope", x)
    if fn is not None:
        y = fn(x, cos, sin)
        if y is not None:
            return y
        _miss("apply_rope(shape)", x)
    return ref.apply_rope(x, cos, sin)


# ---- embeddings --------------------------------------------------------------

def ngram_hash_embed(token_ids, table, mults, bias, table_sizes, table_offsets, order_of_table):
    fn = _cuda("ngram_hash_embed", table)
    if fn is not None:
        out = fn(token_ids, table, mults, bias, table_sizes, table_offsets, order_of_table)
        if out is not None:
            return out
        _miss("ngram_hash_embed(shape)", table)
    return ref.ngram_hash_embed(token_ids, table, mults, bias, table_sizes, table_offsets, order_of_table)


# ---- sequence mixers ----------------------------------------------------------

def mimo_scan(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Psi, Zeta, Phi, angles, D, Z,
              rotary_dim_divisor: int = 4, chunk_size: int = 16):
    fn = _cuda("mimo_scan", V)
    if fn is not None:
        return fn(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Psi, Zeta, Phi, angles, D, Z,
                  rotary_dim_divisor, chunk_size)
    if V.is_cuda and None not in (Zeta, Phi, D, Z):
        from .mimo_scan_lean import mimo_scan_lean     # PyTorch on GPU, one head group at a time
        return mimo_scan_lean(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Psi, Zeta, Phi, angles, D, Z,
                              rotary_dim_divisor, 64)
    return mimo_scan_ref.mimo_scan_chunked(Q, K, V, ADT, DT, Trap, Q_bias, K_bias, Psi, Zeta, Phi,
                                           angles, D, Z, rotary_dim_divisor, chunk_size)


def angle_cumsum(angles_raw, dt):
    fn = _cuda("angle_cumsum", angles_raw)
    if fn is not None:
        out = fn(angles_raw, dt)
        if out is not None:
            return out
        _miss("angle_cumsum(shape)", angles_raw)
    return mimo_scan_ref.angle_cumsum(angles_raw, dt)


def m2rnn_scan(q, k, v, W, f):
    fn = _cuda("m2rnn_scan", v)
    if fn is not None:
        return fn(q, k, v, W, f)
    return ref.m2rnn_scan(q, k, v, W, f)[0]


# ---- DSA ---------------------------------------------------------------------

def indexer_topk(q_idx, k_idx, w, topk: int, q_offset: Optional[int] = None):
    """``q_offset``: sequence position of query 0 when the keys cover more than the queries (context parallelism: the
    keys are gathered over the group, the queries are this rank's chunk); ``None``: queries are the last positions."""
    plain = q_offset is None or (q_offset == 0 and k_idx.shape[1] == q_idx.shape[1])
    fn = _cuda("indexer_topk", q_idx) if plain else None
    if fn is not None:
        with torch.no_grad():
            out = fn(q_idx, k_idx, w, topk)
        if out is not None:
            return out
        _FALLBACKS["indexer_topk(shape)"] += 1
    elif not plain:
        _miss("indexer_topk(query offset)", q_idx)
    with torch.no_grad():
        return ref.indexer_topk(q_idx, k_idx, w, topk, q_offset)


def sparse_mla(q, kv, indices, scale: float, d_v: int):
    fn = _cuda("sparse_mla", q)
    if fn is not None:
        out = fn(q, kv, indices, scale, d_v)
        if out is not None:
            return out
        _FALLBACKS["sparse_mla(shape)"] += 1
    return ref.sparse_mla(q, kv, indices, scale, d_v)[0]


def causal_attention(q, k, v, scale: float):
    """Dense causal attention, q/k [B,S,H,Dqk], v [B,S,H,Dv]."""
    fn = _cuda("causal_attention", q)
    if fn is not None:
        return fn(q, k, v, scale)
    return causal_attention_library(q, k, v, scale)


def causal_attention_library(q, k, v, scale: float):
    """The library path (``scaled_dot_product_attention``): CPU, and shapes the kernel does not take."""
    dq, dv = q.shape[-1], v.shape[-1]
    if q.is_cuda and dv < dq:          # library flash kernels want one head size: zero-pad V
        v = F.pad(v, (0, dq - dv))
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                       is_causal=True, scale=scale)
    return o.transpose(1, 2)[..., :dv]


def embedding(ids, weight):
    """Row gather ``weight[ids]``; on the GPU the backward adds the gradient rows into the weight's gradient buffer with
    vector atomics instead of building a dense [vocab, hidden] gradient."""
    fn = _cuda("embedding", weight)
    if fn is not None:
        y = fn(ids, weight)
        if y is not None:
            return y
    return F.embedding(ids, weight)


def causal_conv1d_silu(x, weight, bias=None):
    """``silu(depthwise causal conv1d over the sequence)`` on a channels-last tensor: x [B, S, C], weight [C, k] (or the
    [C, 1, k] parameter of ``nn.Conv1d(groups=C)``), bias [C].  Output [B, S, C]."""
    if weight.dim() == 3:
        weight = weight.squeeze(1)
    fn = _cuda("causal_conv1d_silu", x)
    if fn is not None:
        y = fn(x, weight, bias)
        if y is not None:
            return y
    return ref.causal_conv1d_silu(x, weight, bias)


# ---- loss --------------------------------------------------------------------

def linear_cross_entropy(hidden, weight, labels, ignore_index: int = -100, reduction: str = "none"):
    fn = _cuda("linear_cross_entropy", hidden)
    if fn is not None:
        return fn(hidden, weight, labels, ignore_index, reduction)
    return ref.linear_cross_entropy(hidden, weight, labels, ignore_index, reduction)


def linear_cross_entropy_weighted(hidden, weight, labels, row_weights, ignore_index: int = -100):
    """Returns ``(sum_t row_weights[t] * CE_t, per-token CE)``; the second output carries no
    gradient.  This is the form the model uses: main and MTP heads are one call whose row
    weights hold mask / token-count / depth scaling."""
    fn = _cuda("linear_cross_entropy_weighted", hidden)
    if fn is not None:
        out = fn(hidden, weight, labels, row_weights, ignore_index)
        if out is not None:
            return out
        _miss("linear_cross_entropy(shape)", hidden)
    per_tok = ref.linear_cross_entropy(hidden, weight, labels, ignore_index, "none")
    return (per_tok * row_weights.to(per_tok.dtype)).sum(), per_tok.detach()


# ---- MoE ---------------------------------------------------------------------

def router_topk(logits, topk, score_function="sigmoid", expert_bias=None, norm_topk_prob=True):
    fn = _cuda("router_topk", logits)
    if fn is not None:
        out = fn(logits, topk, score_function, expert_bias, norm_topk_prob)
        if out is not None:
            return out
        _miss("router_topk(shape)", logits)
    return ref.router_topk(logits, topk, score_function, expert_bias, norm_topk_prob)
