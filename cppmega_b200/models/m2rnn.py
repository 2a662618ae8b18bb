"""M2RNN mixer (the ``R`` layers): matrix-state recurrent layer.

in-proj -> depthwise causal conv1d(k) + SiLU -> q, k, v and forget gate
``f = exp(-exp(A_log) * softplus(x + dt_bias))`` -> recurrence
``h = f h + (1 - f) tanh(h W + k (x) v)`` -> ``y = q . h + D v`` -> ``* SiLU(g)`` -> RMSNorm -> out-proj
(cppmega/megatron/m2rnn_spec.py:102-274).  The layer is replicated across tensor-parallel
ranks, as in the reference (plain ``nn.Linear`` projections).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config.model import M2RNNConfig
from ..ops import functional as F_
from ..parallel.state import ParallelContext
from .common import RMSNorm, fp32_param, seed_for


class M2RNNMixer(nn.Module):
    def __init__(self, hidden: int, cfg: M2RNNConfig, pc: ParallelContext, layer_number: int, *,
                 init_std: float = 0.02, out_std: float = 0.02, eps: float = 1e-5, dtype=torch.float32,
                 seed: int = 1234):
        super().__init__()
        self.cfg, self.pc = cfg, pc
        H = cfg.heads(hidden)
        self.num_heads = H
        self.q_dim = cfg.num_q_heads * cfg.k_head_dim
        self.k_dim = cfg.num_k_heads * cfg.k_head_dim
        self.v_dim = H * cfg.v_head_dim
        self.g_dim = H * cfg.v_head_dim
        self.conv_dim = self.q_dim + self.k_dim + self.v_dim
        name = f"decoder.layers.{layer_number - 1}.mixer"
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed_for(name, seed))
        self.in_dim = self.conv_dim + H + self.g_dim
        # rows padded to a multiple of 8 (zero, never read) so that the projection is a tensor-core GEMM shape
        self.in_dim_padded = (self.in_dim + 7) // 8 * 8
        w_in = torch.zeros(self.in_dim_padded, hidden)
        w_in[:self.in_dim].normal_(0, init_std, generator=gen)
        self.input_projection = nn.Linear(hidden, self.in_dim_padded, bias=False, dtype=dtype)
        self.output_projection = nn.Linear(self.g_dim, hidden, bias=False, dtype=dtype)
        with torch.no_grad():
            self.input_projection.weight.copy_(w_in.to(dtype))
            self.output_projection.weight.copy_(
                torch.empty(hidden, self.g_dim).normal_(0, out_std, generator=gen).to(dtype))
        A = torch.empty(H).uniform_(max(cfg.a_init_min, 1e-4), cfg.a_init_max, generator=gen)
        dt = torch.exp(torch.rand(H, generator=gen) * (math.log(cfg.dt_init_max) - math.log(cfg.dt_init_min))
                       + math.log(cfg.dt_init_min)).clamp(min=cfg.dt_init_floor)
        self.A_log = fp32_param(torch.log(A))
        self.dt_bias = fp32_param(dt + torch.log(-torch.expm1(-dt)))
        if cfg.conv_kernel > 0:
            self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, cfg.conv_kernel, groups=self.conv_dim,
                                    padding=cfg.conv_kernel - 1, bias=True, dtype=dtype)
            with torch.no_grad():
                bound = 1.0 / math.sqrt(cfg.conv_kernel)
                self.conv1d.weight.copy_(torch.empty(self.conv1d.weight.shape).uniform_(-bound, bound, generator=gen).to(dtype))
                self.conv1d.bias.zero_()
        else:
            self.conv1d = None
        self.state_weight = nn.Parameter(torch.eye(cfg.v_head_dim, dtype=dtype).unsqueeze(0).repeat(H, 1, 1))
        self.D = nn.Parameter(torch.ones(H, cfg.v_head_dim, dtype=dtype)) if cfg.use_residual else None
        self.g_norm = RMSNorm(H * cfg.v_head_dim, eps=eps, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, S, _ = x.shape
        H = self.num_heads
        proj = F_.linear(x, self.input_projection.weight)
        conv_in, f_in, g = proj[..., :self.in_dim].split((self.conv_dim, H, self.g_dim), dim=-1)
        f = torch.exp(-torch.exp(self.A_log) * F.softplus(f_in.float() + self.dt_bias))       # [B,S,H] fp32
        if self.conv1d is not None:
            conv_in = F_.causal_conv1d_silu(conv_in, self.conv1d.weight, self.conv1d.bias)    # read in place from proj
        q = conv_in[..., :self.q_dim].reshape(B, S, cfg.num_q_heads, cfg.k_head_dim)
        k = conv_in[..., self.q_dim:self.q_dim + self.k_dim].reshape(B, S, cfg.num_k_heads, cfg.k_head_dim)
        v = conv_in[..., self.q_dim + self.k_dim:].reshape(B, S, H, cfg.v_head_dim)
        y = F_.m2rnn_scan(q, k, v, self.state_weight, f)                                       # [B,S,H,V]
        if self.D is not None:
            y = y + v * self.D
        y = y.flatten(-2, -1) * F.silu(g)
        y = self.g_norm(y)
        return F_.linear(y, self.output_projection.weight)
