"""Input embeddings: token table + hashed n-gram enrichment + structure embedding.

Module names follow the reference's checkpoint keys: ``word_embeddings``,
``cppmega_ngram_hash`` (``unified_table``, ``out_proj``) and ``cppmega_structure``
(``stacked_emb``, ``up_proj``, ``component_scales``)
(cppmega/megatron/custom_embedding.py:49-162).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..config.model import ModelConfig, NgramHashConfig, StructureConfig
from ..ops import functional as F_
from ..parallel.state import ParallelContext
from ..parallel.tensor_parallel import scatter_seq
from .common import seed_for

_PRIMES_NEAR_500K = [
    499_801, 499_819, 499_853, 499_879, 499_883, 499_897, 499_903, 499_927,
    499_943, 499_957, 499_969, 499_973, 499_979, 500_009, 500_029, 500_041,
]


def _is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n % 2 == 0:
        return n == 2
    i = 3
    while i * i <= n:
        if n % i == 0:
            return False
        i += 2
    return True


def pick_table_sizes(count: int, target: int) -> List[int]:
    """``count`` distinct table sizes near ``target``: the fixed primes near 500k when they
    fit (cppmega/features/engram/ngram_hash.py:14-38), otherwise the next primes at or above
    ``target`` so that tiny test tables are still co-prime."""
    near = [p for p in _PRIMES_NEAR_500K if abs(p - target) / target < 0.5]
    if len(near) >= count:
        return near[:count]
    out, n = [], max(target, 2)
    while len(out) < count:
        if _is_prime(n):
            out.append(n)
        n += 1
    return out


class NgramHashEmbedding(nn.Module):
    """Hash token n-grams into one unified table, concatenate the per-table rows and
    project to the hidden size with a zero-initialised matrix."""

    def __init__(self, hidden_size: int, cfg: NgramHashConfig, *, dtype=torch.float32, init_std: float = 0.02):
        super().__init__()
        self.cfg = cfg
        T = cfg.num_tables
        self.table_sizes = pick_table_sizes(T, cfg.table_size)
        offsets, total = [], 0
        for s in self.table_sizes:
            offsets.append(total)
            total += s
        gen = torch.Generator(device="cpu")
        gen.manual_seed(cfg.seed)
        max_order = max(cfg.orders)
        mults = torch.randint(1, 2**31, (T, max_order), dtype=torch.long, generator=gen) | 1
        bias = torch.randint(0, 2**31, (T,), dtype=torch.long, generator=gen)
        order = torch.tensor([o for o in cfg.orders for _ in range(cfg.heads)], dtype=torch.long)
        self.register_buffer("table_offsets", torch.tensor(offsets, dtype=torch.long))
        self.register_buffer("table_sizes_t", torch.tensor(self.table_sizes, dtype=torch.long))
        self.register_buffer("hash_mults", mults)
        self.register_buffer("hash_bias", bias)
        self.register_buffer("order_for_table", order)
        self.unified_table = nn.Embedding(total, cfg.embed_dim, dtype=dtype)
        with torch.no_grad():
            g2 = torch.Generator(device="cpu")
            g2.manual_seed(cfg.seed + 1)
            self.unified_table.weight.copy_(
                torch.empty(total, cfg.embed_dim).normal_(0, 1.0, generator=g2).to(dtype))
        self.out_proj = nn.Linear(T * cfg.embed_dim, hidden_size, bias=False, dtype=dtype)
        nn.init.zeros_(self.out_proj.weight)
        for p in (self.unified_table.weight, self.out_proj.weight):
            p.is_embedding_or_output_parameter = True

    def hash_indices(self, token_ids: torch.Tensor) -> torch.Tensor:
        from ..ops import reference as ref
        return ref.ngram_hash_indices(token_ids, self.hash_mults, self.hash_bias, self.table_sizes_t,
                                      self.table_offsets, self.order_for_table)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        table = self.unified_table.weight
        ids = token_ids
        if self.cfg.offload and table.device != ids.device:
            ids = ids.to(table.device)
        e = F_.ngram_hash_embed(ids, table, self.hash_mults, self.hash_bias, self.table_sizes_t,
                                self.table_offsets, self.order_for_table)
        e = e.to(device=self.out_proj.weight.device, dtype=self.out_proj.weight.dtype)
        y = F_.linear(e, self.out_proj.weight)
        return F.dropout(y, self.cfg.dropout, self.training) if self.cfg.dropout > 0 else y


class StructureEmbedding(nn.Module):
    """Additive embedding of per-token structure features through a bottleneck."""

    ALL = ("structure", "dep_level", "ast_depth", "sibling_index", "ast_node_type")
    CORE = ("structure", "dep_level")
    INPUT_KEYS = {"structure": "structure_ids", "dep_level": "dep_levels", "ast_depth": "ast_depth_ids",
                  "sibling_index": "sibling_index_ids", "ast_node_type": "node_type_ids"}

    def __init__(self, hidden_size: int, cfg: StructureConfig, *, dtype=torch.float32):
        super().__init__()
        self.cfg = cfg
        self.active = self.parse_components(cfg.components)
        vocab = {"structure": cfg.num_categories, "dep_level": cfg.max_dep_level, "ast_depth": cfg.max_ast_depth,
                 "sibling_index": cfg.max_sibling_index, "ast_node_type": cfg.num_node_types}
        self.offsets, self.clamp_max, total = [], [], 0
        for n in self.active:
            self.offsets.append(total)
            self.clamp_max.append(vocab[n] - 1)
            total += vocab[n]
        self.stacked_emb = nn.Embedding(total, cfg.bottleneck_dim, dtype=dtype)
        self.up_proj = nn.Linear(cfg.bottleneck_dim, hidden_size, bias=False, dtype=dtype)
        k = len(self.active)
        self.component_scales = nn.Parameter(torch.full((k,), 1.0 / max(k, 1), dtype=dtype))
        nn.init.zeros_(self.stacked_emb.weight)
        nn.init.zeros_(self.up_proj.weight)
        for p in (self.stacked_emb.weight, self.up_proj.weight):
            p.is_embedding_or_output_parameter = True

    @classmethod
    def parse_components(cls, spec: str):
        if spec == "all":
            return cls.ALL
        if spec == "core":
            return cls.CORE
        req = {s.strip() for s in spec.split(",") if s.strip()}
        bad = sorted(req - set(cls.ALL))
        if bad:
            raise ValueError(f"unknown structure components: {bad!r}")
        return tuple(n for n in cls.ALL if n in req)

    def forward(self, inputs: Dict[str, Optional[torch.Tensor]], target_dtype=None):
        tensors = [inputs.get(self.INPUT_KEYS[n]) for n in self.active]
        ref_t = next((t for t in tensors if t is not None), None)
        if ref_t is None:
            return None
        B, S = ref_t.shape[:2]
        ids, present = [], []
        for i, t in enumerate(tensors):
            if t is None:
                ids.append(torch.zeros(B, S, dtype=torch.long, device=ref_t.device))
                present.append(0.0)
            else:
                ids.append(t.long().clamp(0, self.clamp_max[i]) + self.offsets[i])
                present.append(1.0)
        emb = F.embedding(torch.stack(ids, dim=-1), self.stacked_emb.weight)        # [B,S,k,bd]
        scales = self.component_scales * torch.tensor(present, dtype=self.component_scales.dtype,
                                                      device=emb.device)
        w = (emb * scales.view(1, 1, -1, 1)).sum(dim=2)
        if target_dtype is not None:
            w = w.to(target_dtype)
        return F_.linear(w, self.up_proj.weight.to(w.dtype))


class VocabParallelEmbedding(nn.Module):
    """Token table split along the vocabulary over TP ranks; out-of-shard rows contribute
    zero and the partial results are summed."""

    def __init__(self, vocab: int, hidden: int, pc: ParallelContext, *, std: float, dtype, seed: int):
        super().__init__()
        if vocab % pc.tp:
            raise ValueError(f"vocab {vocab} not divisible by tp={pc.tp}")
        self.pc = pc
        self.per = vocab // pc.tp
        self.lo = pc.tp_rank * self.per
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        full = torch.empty(vocab, hidden, dtype=torch.float32).normal_(0, std, generator=gen)
        self.weight = nn.Parameter(full[self.lo:self.lo + self.per].clone().to(dtype))
        self.weight.tensor_model_parallel = pc.tp > 1
        self.weight.partition_dim = 0
        self.weight.is_embedding_or_output_parameter = True

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self.pc.tp == 1:
            return F_.embedding(ids, self.weight)
        local = ids - self.lo
        mask = (local < 0) | (local >= self.per)
        out = F_.embedding(local.masked_fill(mask, 0), self.weight)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        return _AllReduceSum.apply(out, self.pc.tp_group)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class LanguageModelEmbedding(nn.Module):
    """``word + ngram_hash + structure`` -> [B,S,H] (sequence-scattered under SP)."""

    def __init__(self, cfg: ModelConfig, pc: ParallelContext, *, dtype=torch.float32, seed: int = 1234):
        super().__init__()
        self.cfg, self.pc = cfg, pc
        self.word_embeddings = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, pc, std=cfg.init_std,
                                                      dtype=dtype, seed=seed_for("embedding.word_embeddings", seed))
        self.cppmega_ngram_hash = (NgramHashEmbedding(cfg.hidden_size, cfg.ngram_hash, dtype=dtype,
                                                      init_std=cfg.init_std)
                                   if cfg.ngram_hash.enabled else None)
        self.cppmega_structure = (StructureEmbedding(cfg.hidden_size, cfg.structure, dtype=dtype)
                                  if cfg.structure.enabled else None)

    def forward(self, input_ids: torch.Tensor, structure_inputs: Optional[Dict[str, torch.Tensor]] = None,
                scatter: bool = True) -> torch.Tensor:
        x = self.word_embeddings(input_ids)
        if self.cppmega_ngram_hash is not None:
            x = x + self.cppmega_ngram_hash(input_ids).to(x.dtype)
        if self.cppmega_structure is not None and structure_inputs:
            s = self.cppmega_structure(structure_inputs, target_dtype=x.dtype)
            if s is not None:
                x = x + s
        if scatter and self.pc.sequence_parallel:
            x = scatter_seq(x, self.pc)
        return x
