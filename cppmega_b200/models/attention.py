"""Multi-head latent attention (MLA) and DSA sparse attention with indexer + IndexCache.

Parameter names follow Megatron's MLA/DSA modules so checkpoints line up:
``linear_q_down_proj, q_layernorm, linear_q_up_proj, linear_kv_down_proj, kv_layernorm,
linear_kv_up_proj, linear_proj`` and, for DSA, ``core_attention.indexer.{linear_wq_b,
linear_wk, k_norm, linear_weights_proj}``.

* MLA layers run dense causal attention with per-head K/V (qk 64+64, v 64).
* DSA layers run the *absorbed* form: queries are mapped into the KV latent space
  (``q_nope W_uk``) and attend over one shared ``[latent | rope]`` key/value row per
  position selected by the indexer's causal top-k
  (contract at cppmega/megatron/sparse_mla_ops/sparse_mla.py:17-39, 610-686).
* IndexCache: DSA layers whose rank is in ``full_layer_ranks`` compute and publish their
  top-k; the others reuse the latest publication of the current micro-batch, and a
  reusing layer that finds no publication (e.g. first DSA layer of a pipeline stage)
  computes its own (cppmega/megatron/index_cache_patch.py:112-118,157-262).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn

from ..config.model import DSAConfig, MLAConfig
from ..ops import functional as F_
from ..ops import reference as ref
from ..parallel.state import ParallelContext
from ..parallel.tensor_parallel import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear, copy_to_tp, gather_seq
from .common import RMSNorm, cat_last_dim, seed_for, split_last_dim


@dataclass
class IndexCacheState:
    """Per-micro-batch store of published top-k indices; one instance per forward."""

    indices: Optional[torch.Tensor] = None
    published_by: int = -1
    stats: dict = field(default_factory=lambda: {"computed": 0, "reused": 0})

    def clear(self):
        self.indices, self.published_by = None, -1


class DSAIndexer(nn.Module):
    def __init__(self, hidden: int, mla: MLAConfig, dsa: DSAConfig, pc: ParallelContext, name: str, *,
                 std: float, dtype, seed: int, eps: float):
        super().__init__()
        self.h, self.d, self.topk = dsa.index_n_heads, dsa.index_head_dim, dsa.index_topk
        self.rope_dim = self.d // 2
        self.rope_base = mla.rope_base
        self.linear_wq_b = ReplicatedLinear(mla.q_lora_rank, self.h * self.d, pc, std=std, dtype=dtype, sp_partial_grad=False,
                                            seed=seed_for(name + ".linear_wq_b", seed))
        self.linear_wk = ReplicatedLinear(hidden, self.d, pc, std=std, dtype=dtype, sp_partial_grad=False,
                                          seed=seed_for(name + ".linear_wk", seed))
        self.k_norm = RMSNorm(self.d, eps=eps, dtype=dtype)
        self.linear_weights_proj = ReplicatedLinear(hidden, self.h, pc, std=std, dtype=dtype, sp_partial_grad=False,
                                                    seed=seed_for(name + ".linear_weights_proj", seed))
        self.scale = self.h ** -0.5 * self.d ** -0.5

    def project(self, x: torch.Tensor, q_latent: torch.Tensor, pos_offset: int = 0):
        B, S, _ = x.shape
        q = self.linear_wq_b(q_latent).reshape(B, S, self.h, self.d)
        k = self.k_norm(self.linear_wk(x))
        cos, sin = ref.rope_tables(S, self.rope_dim, self.rope_base, device=x.device, offset=pos_offset)
        if self.rope_dim < self.d:
            q_r, q_n = split_last_dim(q, (self.rope_dim, self.d - self.rope_dim))
            k_r, k_n = split_last_dim(k, (self.rope_dim, self.d - self.rope_dim))
            q = cat_last_dim([F_.apply_rope(q_r, cos, sin), q_n])
            k = cat_last_dim([F_.apply_rope(k_r, cos, sin), k_n])
        else:
            q, k = F_.apply_rope(q, cos, sin), F_.apply_rope(k, cos, sin)
        w = self.linear_weights_proj(x).float() * self.scale
        return q, k, w

    def forward(self, x: torch.Tensor, q_latent: torch.Tensor, cg=None):
        """Returns (indices int32 [B,S,topk], (q_idx, k_idx, w)); inputs are detached: the
        indexer learns only through the optional KL loss.  With a context group ``cg`` the index keys of all chunks are
        gathered and the indices address the whole sequence."""
        off = cg.q_offset(x.shape[1]) if cg is not None else 0
        q, k, w = self.project(x.detach(), q_latent.detach(), off)
        if cg is not None and cg.size > 1:
            from ..parallel.context_parallel import gather_context
            k = gather_context(k, cg)
            idx = F_.indexer_topk(q.detach(), k.detach(), w.detach(), self.topk, q_offset=off)
        else:
            idx = F_.indexer_topk(q.detach(), k.detach(), w.detach(), self.topk)
        return idx, (q, k, w)


class MLAttention(nn.Module):
    """One attention layer; ``sparse=True`` makes it a DSA layer."""

    def __init__(self, hidden: int, mla: MLAConfig, pc: ParallelContext, layer_name: str, *,
                 dsa: Optional[DSAConfig] = None, dsa_rank: int = -1, init_std: float = 0.02,
                 out_std: float = 0.02, eps: float = 1e-5, dtype=torch.float32, seed: int = 1234):
        super().__init__()
        self.mla, self.pc, self.dsa, self.dsa_rank = mla, pc, dsa, dsa_rank
        self.sparse = dsa is not None
        tp = pc.tp
        if mla.num_heads % tp:
            raise ValueError(f"num_heads={mla.num_heads} not divisible by tp={tp}")
        self.heads_local = mla.num_heads // tp
        n = layer_name + ".self_attention"
        self.linear_q_down_proj = ReplicatedLinear(hidden, mla.q_lora_rank, pc, std=init_std, dtype=dtype, sp_partial_grad=False,
                                                   seed=seed_for(n + ".linear_q_down_proj", seed))
        self.q_layernorm = RMSNorm(mla.q_lora_rank, eps=eps, dtype=dtype)
        self.linear_q_up_proj = ColumnParallelLinear(mla.q_lora_rank, mla.num_heads * mla.q_head_dim, pc,
                                                     std=init_std, dtype=dtype, sequence_parallel_input=False,
                                                     seed=seed_for(n + ".linear_q_up_proj", seed), name=n + ".linear_q_up_proj")
        self.linear_kv_down_proj = ReplicatedLinear(hidden, mla.kv_lora_rank + mla.qk_pos_emb_head_dim, pc,
                                                    std=init_std, dtype=dtype, sp_partial_grad=False,
                                                    seed=seed_for(n + ".linear_kv_down_proj", seed))
        self.kv_layernorm = RMSNorm(mla.kv_lora_rank, eps=eps, dtype=dtype)
        self.linear_kv_up_proj = ColumnParallelLinear(mla.kv_lora_rank, mla.num_heads * (mla.qk_head_dim + mla.v_head_dim),
                                                      pc, std=init_std, dtype=dtype, sequence_parallel_input=False,
                                                      seed=seed_for(n + ".linear_kv_up_proj", seed), name=n + ".linear_kv_up_proj")
        self.linear_proj = RowParallelLinear(mla.num_heads * mla.v_head_dim, hidden, pc, std=out_std, dtype=dtype,
                                             seed=seed_for(n + ".linear_proj", seed), name=n + ".linear_proj")
        self.softmax_scale = 1.0 / math.sqrt(mla.q_head_dim)
        if self.sparse:
            self.core_attention = nn.Module()
            self.core_attention.indexer = DSAIndexer(hidden, mla, dsa, pc, n + ".core_attention.indexer",
                                                     std=init_std, dtype=dtype, seed=seed, eps=eps)
        self.last_indexer_loss: Optional[torch.Tensor] = None
        self.context_group = None        # parallel.context_parallel.ContextGroup: DSA layers only, set by the caller

    @property
    def is_index_publisher(self) -> bool:
        return self.sparse and ((not self.dsa.index_cache) or self.dsa_rank in self.dsa.full_layer_ranks)

    @torch.no_grad()
    def select_indices(self, x: torch.Tensor, index_cache: Optional[IndexCacheState]) -> torch.Tensor:
        """Top-k selection alone (no autograd graph), for callers that recompute the layer in
        backward and must replay it with the indices of the first pass."""
        if self.pc.sequence_parallel:
            x = gather_seq(x, self.pc, reduce_grad=False)
        q_lat = self.q_layernorm(self.linear_q_down_proj(x))
        return self._indices(x, q_lat, index_cache, None)

    def forward(self, x: torch.Tensor, index_cache: Optional[IndexCacheState] = None,
                indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        mla, pc = self.mla, self.pc
        if pc.sequence_parallel:
            x = gather_seq(x, pc, reduce_grad=False)
        B, S, _ = x.shape
        Hl = self.heads_local
        dq, dr, dv, dc = mla.qk_head_dim, mla.qk_pos_emb_head_dim, mla.v_head_dim, mla.kv_lora_rank
        q_lat = self.q_layernorm(self.linear_q_down_proj(x))
        q = self.linear_q_up_proj(q_lat).reshape(B, S, Hl, dq + dr)
        kv_c = self.linear_kv_down_proj(x)
        kv_lat, k_pe = split_last_dim(kv_c, (dc, dr))
        kv_lat = self.kv_layernorm(kv_lat)
        cg = self.context_group if self.sparse else None
        if cg is not None and cg.size > 1 and self.dsa.indexer_loss_coeff > 0:
            raise NotImplementedError("the indexer KL loss is not defined over a split sequence")
        cos, sin = ref.rope_tables(S, dr, mla.rope_base, device=x.device, offset=cg.q_offset(S) if cg is not None else 0)
        q_nope, q_pe = split_last_dim(q, (dq, dr))
        q_pe = F_.apply_rope(q_pe, cos, sin)
        k_pe = copy_to_tp(F_.apply_rope(k_pe, cos, sin), pc)                    # [B,S,dr] shared by heads
        self.last_indexer_loss = None
        if not self.sparse:
            kv = self.linear_kv_up_proj(kv_lat).reshape(B, S, Hl, dq + dv)
            k_nope, v = split_last_dim(kv, (dq, dv))
            k = cat_last_dim([k_nope, k_pe.unsqueeze(2).expand(B, S, Hl, dr)])
            o = F_.causal_attention(cat_last_dim([q_nope, q_pe]), k, v.contiguous(), self.softmax_scale)
        elif self.dsa.warmup_dense and self.training and self.dsa.indexer_loss_coeff > 0 and indices is None:
            # indexer warm-up: dense attention output and the KL loss that trains the indexer, from the same score blocks
            kv = self.linear_kv_up_proj(kv_lat).reshape(B, S, Hl, dq + dv)
            k_nope, v = split_last_dim(kv, (dq, dv))
            k = cat_last_dim([k_nope, k_pe.unsqueeze(2).expand(B, S, Hl, dr)])
            _idx, (qi, ki, wi) = self.core_attention.indexer(x, q_lat, self.context_group)
            o, self.last_indexer_loss = ref.dsa_warmup_attention_and_kl(
                cat_last_dim([q_nope, q_pe]), k, v, self.softmax_scale, qi, ki, wi, self.dsa.indexer_loss_coeff)
        else:
            idx = indices if indices is not None else self._indices(x, q_lat, index_cache, (q_nope, q_pe, kv_lat, k_pe))
            w_up = self.linear_kv_up_proj.weight.reshape(Hl, dq + dv, dc)
            w_uk, w_uv = w_up[:, :dq], w_up[:, dq:]
            lat_tp = copy_to_tp(kv_lat, pc)
            q_abs = F_.head_linear(q_nope, w_uk.transpose(1, 2))                 # [B,S,Hl,dc] = q_nope . W_uk
            q_full = cat_last_dim([q_abs, q_pe])                                # [B,S,Hl,dc+dr]
            kv_full = cat_last_dim([lat_tp, k_pe])                               # [B,S,dc+dr]
            if cg is not None and cg.size > 1:                                  # keys of every chunk; indices are global
                from ..parallel.context_parallel import gather_context
                kv_full = gather_context(kv_full, cg)
            o_lat = F_.sparse_mla(q_full, kv_full, idx, self.softmax_scale, dc)  # [B,S,Hl,dc]
            o = F_.head_linear(o_lat, w_uv)                                      # [B,S,Hl,dv] = o_lat . W_uv^T
        return self.linear_proj(o.reshape(B, S, Hl * dv))

    def _indices(self, x, q_lat, cache: Optional[IndexCacheState], attn_parts) -> torch.Tensor:
        indexer = self.core_attention.indexer
        reuse = (cache is not None and self.dsa.index_cache and not self.is_index_publisher
                 and cache.indices is not None and cache.indices.shape[:2] == x.shape[:2])
        if reuse:
            cache.stats["reused"] += 1
            return cache.indices
        idx, (qi, ki, wi) = indexer(x, q_lat, self.context_group)
        if cache is not None:
            cache.stats["computed"] += 1
            if self.dsa.index_cache:
                cache.indices, cache.published_by = idx, self.dsa_rank
        if self.dsa.indexer_loss_coeff > 0 and self.training and attn_parts is not None:
            q_nope, q_pe, kv_lat, k_pe = attn_parts
            Hl, dq = self.heads_local, self.mla.qk_head_dim
            w_up = self.linear_kv_up_proj.weight.reshape(Hl, -1, self.mla.kv_lora_rank)
            k_nope = torch.einsum("bsc,hdc->bshd", kv_lat.detach(), w_up[:, :dq].detach().to(kv_lat.dtype))
            kk = torch.cat([k_nope, k_pe.detach().unsqueeze(2).expand(-1, -1, Hl, -1)], dim=-1)
            qq = torch.cat([q_nope, q_pe], dim=-1).detach()
            kl = ref.indexer_kl_loss if qq.shape[1] <= 1024 else ref.indexer_kl_loss_chunked      # bounded transient at long S
            self.last_indexer_loss = kl(qq, kk, self.softmax_scale, qi, ki, wi, self.dsa.indexer_loss_coeff)
        return idx
