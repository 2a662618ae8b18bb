"""FastMTP: one shared attention + SwiGLU block applied K times on a *detached* trunk.

Per step k = 1..K: ids and targets are rolled one position to the left (the tail is masked), the next-token
embedding is looked up (teacher forcing), ``h <- block(proj([rms(h) | rms(emb)]))``, ``h <- rms(h)``, and a fused
linear cross-entropy against the detached LM head gives the step loss; steps are weighted ``decay^k`` normalised
to sum to one; the trainer adds ``lambda * loss`` to the main loss
(cppmega/megatron/fastmtp_layer.py:32-47 weights, :128-183 block, :266-373 forward, :389-406 defaults).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config.model import ModelConfig
from ..ops import functional as F_
from ..ops import reference as ref

IGNORE = -100


def step_weights(depth: int, decay: float) -> torch.Tensor:
    w = torch.tensor([decay ** k for k in range(depth)], dtype=torch.float32)
    return w / w.sum()


class SharedMTPBlock(nn.Module):
    def __init__(self, hidden: int, heads: int, ffn: int, dtype, eps: float = 1e-5):
        super().__init__()
        self.heads, self.head_dim, self.eps = heads, hidden // heads, eps
        self.ln1 = nn.Parameter(torch.ones(hidden, dtype=dtype))
        self.qkv = nn.Linear(hidden, 3 * hidden, bias=False, dtype=dtype)
        self.out_proj = nn.Linear(hidden, hidden, bias=False, dtype=dtype)
        self.ln2 = nn.Parameter(torch.ones(hidden, dtype=dtype))
        self.gate_up = nn.Linear(hidden, 2 * ffn, bias=False, dtype=dtype)
        self.down = nn.Linear(ffn, hidden, bias=False, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:          # [B,S,H]
        B, S, H = x.shape
        h = F_.rmsnorm(x, self.ln1, self.eps)
        qkv = F_.linear(h, self.qkv.weight).reshape(B, S, 3, self.heads, self.head_dim)
        o = F_.causal_attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], self.head_dim ** -0.5)
        x = x + F_.linear(o.reshape(B, S, H), self.out_proj.weight)
        h = F_.rmsnorm(x, self.ln2, self.eps)
        return x + F_.linear(F_.swiglu(F_.linear(h, self.gate_up.weight)), self.down.weight)


class FastMTPHead(nn.Module):
    def __init__(self, cfg: ModelConfig, *, dtype=torch.float32, seed: int = 1234):
        super().__init__()
        h = cfg.hidden_size
        self.depth = cfg.mtp.fastmtp_depth
        self.eps = cfg.norm_eps
        g = torch.Generator(device="cpu").manual_seed(seed + 4242)
        self.proj = nn.Linear(2 * h, h, bias=False, dtype=dtype)
        self.shared_block = SharedMTPBlock(h, cfg.mla.num_heads, min(cfg.ffn_hidden_size, 4 * h), dtype, cfg.norm_eps)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() >= 2:
                    p.copy_(torch.empty(p.shape).normal_(0, cfg.init_std, generator=g).to(dtype))
        self.register_buffer("step_weights", step_weights(self.depth, cfg.mtp.fastmtp_decay), persistent=False)
        self._ones = None

    def forward(self, trunk_hidden, input_ids, labels, loss_mask, embedding, lm_head_weight) -> torch.Tensor:
        """``trunk_hidden`` [B,S,H] (detached by the caller); returns the weighted scalar loss."""
        h = trunk_hidden.detach()
        B, S, H = h.shape
        if S <= 1:
            return h.sum() * 0.0
        ids = labels.clone()
        tgt = labels.masked_fill(loss_mask == 0, IGNORE)
        ones = torch.ones(H, dtype=h.dtype, device=h.device)
        total = h.new_zeros((), dtype=torch.float32)
        for k in range(self.depth):
            ids = torch.roll(ids, -1, dims=1)
            ids[:, -1] = 0
            tgt = torch.roll(tgt, -1, dims=1)
            tgt[:, -1] = IGNORE
            emb = embedding.word_embeddings(ids).to(h.dtype)
            x = torch.cat([ref.rmsnorm(h, ones, self.eps), ref.rmsnorm(emb, ones, self.eps)], dim=-1)
            h = self.shared_block(F_.linear(x, self.proj.weight))
            h = ref.rmsnorm(h, ones, self.eps)
            flat_t = tgt.reshape(-1)
            valid = (flat_t != IGNORE).float()
            w = valid / valid.sum().clamp_min(1.0)
            step_loss, _ = F_.linear_cross_entropy_weighted(h.reshape(B * S, H), lm_head_weight, flat_t, w, IGNORE)
            total = total + self.step_weights[k] * step_loss
        return total


_ = F
