"""Mamba3 MIMO mixer (tensor-parallel aware).

Packed in_proj ``[z, x, B, C, dd_dt, dd_A, trap]`` is column-parallel with B/C laid
out ``(group, rank, state)``; the small angle projection is replicated and its
output is gathered along the sequence under sequence parallelism; per-head fp32
parameters are sharded on dim 0 and initialised from a CPU generator so TP=1 and
TP=n build the same model; out_proj is row-parallel
(cppmega/megatron/cppmega_mamba3_tp_mixer.py:113-375 for construction, :404-556 for the
forward order that is kept here).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config.model import Mamba3Config
from ..ops import functional as F_
from ..parallel.state import ParallelContext
from ..parallel.tensor_parallel import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear, gather_seq
from .common import RMSNorm, fp32_param, seed_for, split_last_dim


class Mamba3Mixer(nn.Module):
    def __init__(self, hidden: int, cfg: Mamba3Config, pc: ParallelContext, layer_number: int, *,
                 init_std: float = 0.02, out_std: float = 0.02, dtype=torch.float32, seed: int = 1234):
        super().__init__()
        if not cfg.is_mimo:
            raise NotImplementedError("Mamba3Mixer implements the MIMO path; use models.mamba_variants for SISO")
        if pc.config.cp != 1:
            raise ValueError("Mamba3Mixer does not support context parallelism")
        self.cfg, self.pc, self.hidden = cfg, pc, hidden
        tp = pc.tp
        self.nheads = cfg.nheads(hidden)
        self.nheads_local = self.nheads // tp
        self.ngroups_local = cfg.ngroups // tp
        self.d_inner_local = cfg.d_inner(hidden) // tp
        self.sizes_local = cfg.in_proj_sizes(hidden, tp)
        name = f"decoder.layers.{layer_number - 1}.mixer"
        self.in_proj = ColumnParallelLinear(hidden, sum(cfg.in_proj_sizes(hidden, 1)), pc, std=init_std,
                                            dtype=dtype, seed=seed_for(name + ".in_proj", seed),
                                            partition_sizes=list(cfg.in_proj_sizes(hidden, 1)),
                                            name=name + ".in_proj")
        self.angle_proj = ReplicatedLinear(hidden, cfg.num_rope_angles, pc, dtype=dtype,
                                           seed=7919 + 100003 * layer_number,
                                           uniform_bound=1.0 / math.sqrt(hidden))
        gen = torch.Generator(device="cpu")
        gen.manual_seed(1337 + 100003 * layer_number)
        full_dt = torch.exp(torch.rand(self.nheads, generator=gen, dtype=torch.float32)
                            * (math.log(cfg.dt_max) - math.log(cfg.dt_min)) + math.log(cfg.dt_min)
                            ).clamp(min=cfg.dt_init_floor)
        full_dt_bias = full_dt + torch.log(-torch.expm1(-full_dt))
        lo, hi = pc.tp_rank * self.nheads_local, (pc.tp_rank + 1) * self.nheads_local
        sh = tp > 1
        R, N, P = cfg.mimo_rank, cfg.d_state, cfg.headdim
        self.dt_bias = fp32_param(full_dt_bias[lo:hi].clone(), tp_sharded=sh)
        self.B_bias = fp32_param(torch.ones(self.nheads_local, R, N), tp_sharded=sh)
        self.C_bias = fp32_param(torch.ones(self.nheads_local, R, N), tp_sharded=sh)
        self.mimo_x = fp32_param(torch.ones(self.nheads_local, R, P) / R, tp_sharded=sh, no_wd=False)
        self.mimo_z = fp32_param(torch.ones(self.nheads_local, R, P), tp_sharded=sh, no_wd=False)
        self.mimo_o = fp32_param(torch.ones(self.nheads_local, R, P) / R, tp_sharded=sh, no_wd=False)
        self.D = fp32_param(torch.ones(self.nheads_local), tp_sharded=sh)
        self.B_norm = RMSNorm(N, eps=1e-5, dtype=dtype)
        self.C_norm = RMSNorm(N, eps=1e-5, dtype=dtype)
        self.out_proj = RowParallelLinear(cfg.d_inner(hidden), hidden, pc, std=out_std, dtype=dtype,
                                          seed=seed_for(name + ".out_proj", seed), name=name + ".out_proj")

    def project(self, x: torch.Tensor):
        """Everything before the scan.  Returns the scan's argument tuple."""
        cfg, pc = self.cfg, self.pc
        R, N, P = cfg.mimo_rank, cfg.d_state, cfg.headdim
        Hl, Gl = self.nheads_local, self.ngroups_local
        angles_raw = self.angle_proj(x)
        if pc.sequence_parallel:
            angles_raw = gather_seq(angles_raw, pc, reduce_grad=True)
        packed = self.in_proj(x)                                    # [B,S,sum(sizes_local)]
        Bsz, S = packed.shape[:2]
        z, xv, Bm, Cm, dd_dt, dd_A, trap = split_last_dim(packed, self.sizes_local)
        z = z.reshape(Bsz, S, Hl, P)
        xv = xv.reshape(Bsz, S, Hl, P)
        Bm = self.B_norm(Bm.reshape(Bsz, S, Gl, R, N)).permute(0, 1, 3, 2, 4)     # [B,S,R,G,N]
        Cm = self.C_norm(Cm.reshape(Bsz, S, Gl, R, N)).permute(0, 1, 3, 2, 4)
        A = torch.clamp(-F.softplus(dd_A.float()), max=-cfg.a_floor)
        DT = F.softplus(dd_dt.float() + self.dt_bias)
        ADT = (A * DT).transpose(1, 2)                               # [B,H,S]
        DT = DT.transpose(1, 2)
        trap_t = trap.float().transpose(1, 2)
        angles = F_.angle_cumsum(angles_raw, DT)                     # [B,S,H,A] fp32
        return Cm, Bm, xv, ADT, DT, trap_t, angles, z

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        Cm, Bm, xv, ADT, DT, trap_t, angles, z = self.project(x)
        y = F_.mimo_scan(Cm, Bm, xv, ADT, DT, trap_t, self.C_bias, self.B_bias, self.mimo_x, self.mimo_z,
                         self.mimo_o, angles, self.D, z, cfg.rotary_dim_divisor, cfg.chunk_size)
        Bsz, S = y.shape[:2]
        return self.out_proj(y.reshape(Bsz, S, self.d_inner_local).to(x.dtype))
