"""Alternative SSM mixers: the single-input (SISO) Mamba2/Mamba3 family.

One configurable module covers the reference's variants
(cppmega/megatron/noconv_mamba_mixer.py:64-979 and cppmega/megatron/mamba3_mixer.py:48-396):

* ``ssd``         Mamba2 block: causal depthwise conv1d(4) + SiLU on [x|B|C], constant per-head A, SSD scan,
                  gated RMSNorm, out-proj;
* ``noconv_ssd``  no convolution (SiLU on x only); optional Mamba3 features on the B/C path: QK-norm with learnt
                  weights, zero-initialised B/C bias, data-dependent A, trapezoidal discretisation and rotary on the
                  state dimension with cumulative, dt-scaled angles.

The scan itself is the rank-1 case of the MIMO operator (``R = 1``, ``Psi = Phi = 1``): the trapezoid can be switched
off by a large positive ``trap`` (``gamma = dt``, no look-ahead term) and the rotation by zero angles, so these
mixers run on the same kernels / oracles as the MIMO mixer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config.model import ModelConfig
from ..ops import functional as F_
from ..ops import mimo_scan_ref
from ..parallel.state import ParallelContext
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from .common import RMSNorm, fp32_param, seed_for


@dataclass(frozen=True)
class SSDVariant:
    conv_kernel: int = 4          # 0 = no convolution
    qk_norm: bool = False
    bc_bias: bool = False
    data_dependent_a: bool = False
    trapezoid: bool = False
    rope_on_state: bool = False


VARIANTS = {
    "ssd": SSDVariant(conv_kernel=4),
    "noconv_ssd": SSDVariant(conv_kernel=0, qk_norm=True, bc_bias=True, data_dependent_a=True, trapezoid=True,
                             rope_on_state=True),
}


class SSDMixer(nn.Module):
    def __init__(self, cfg: ModelConfig, pc: ParallelContext, layer_number: int, variant: SSDVariant, *, dtype, seed: int,
                 out_std: float):
        super().__init__()
        m3, h = cfg.mamba3, cfg.hidden_size
        if pc.tp > 1 and variant.conv_kernel > 0:
            raise NotImplementedError("the convolutional SSD mixer is not tensor-parallel; use the MIMO mixer for TP")
        self.cfg, self.pc, self.v = cfg, pc, variant
        self.d_inner, self.nheads, self.G, self.N, self.P = m3.d_inner(h), m3.nheads(h), m3.ngroups, m3.d_state, m3.headdim
        self.n_angles = m3.num_rope_angles if variant.rope_on_state else 0
        name = f"decoder.layers.{layer_number - 1}.mixer"
        sizes = [self.d_inner, self.d_inner, self.G * self.N, self.G * self.N, self.nheads]
        if variant.data_dependent_a:
            sizes.append(self.nheads)
        if variant.trapezoid:
            sizes.append(self.nheads)
        if self.n_angles:
            sizes.append(self.n_angles)
        # pad the packed width to a multiple of 32 so block-scaled (1x32) recipes can quantise it
        self.sizes = sizes
        width = (sum(sizes) + 31) // 32 * 32
        self.in_proj = ColumnParallelLinear(h, width, pc, std=cfg.init_std, dtype=dtype, seed=seed_for(name + ".in_proj", seed),
                                            name=name + ".in_proj")
        self.out_proj = RowParallelLinear(self.d_inner, h, pc, std=out_std, dtype=dtype,
                                          seed=seed_for(name + ".out_proj", seed), name=name + ".out_proj")
        gen = torch.Generator(device="cpu").manual_seed(1337 + 100003 * layer_number)
        dt = torch.exp(torch.rand(self.nheads, generator=gen) * (math.log(m3.dt_max) - math.log(m3.dt_min)) + math.log(m3.dt_min)
                       ).clamp(min=m3.dt_init_floor)
        self.dt_bias = fp32_param(dt + torch.log(-torch.expm1(-dt)))
        self.A_log = fp32_param(torch.log(torch.empty(self.nheads).uniform_(1, 16, generator=gen)))
        self.D = fp32_param(torch.ones(self.nheads))
        conv_dim = self.d_inner + 2 * self.G * self.N
        self.conv1d = (nn.Conv1d(conv_dim, conv_dim, variant.conv_kernel, groups=conv_dim, padding=variant.conv_kernel - 1,
                                 dtype=dtype) if variant.conv_kernel > 0 else None)
        if variant.qk_norm:
            self.B_norm_weight = nn.Parameter(torch.ones(self.N, dtype=dtype))
            self.C_norm_weight = nn.Parameter(torch.ones(self.N, dtype=dtype))
        if variant.bc_bias:
            self.B_bias = fp32_param(torch.zeros(self.nheads, 1, self.N))
            self.C_bias = fp32_param(torch.zeros(self.nheads, 1, self.N))
        self.norm = RMSNorm(self.d_inner, cfg.norm_eps, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        v, B_, S = self.v, x.shape[0], x.shape[1]
        H, G, N, P = self.nheads, self.G, self.N, self.P
        parts = list(torch.split(self.in_proj(x)[..., :sum(self.sizes)], self.sizes, dim=-1))
        z, xs, Bm, Cm, dd_dt = parts[:5]
        rest = parts[5:]
        dd_A = rest.pop(0) if v.data_dependent_a else None
        trap = rest.pop(0) if v.trapezoid else None
        ang = rest.pop(0) if self.n_angles else None
        if self.conv1d is not None:
            xbc = F_.causal_conv1d_silu(torch.cat([xs, Bm, Cm], dim=-1), self.conv1d.weight, self.conv1d.bias)
            xs, Bm, Cm = torch.split(xbc, [self.d_inner, G * N, G * N], dim=-1)
        else:
            xs = F.silu(xs)
        Bm = Bm.reshape(B_, S, 1, G, N)
        Cm = Cm.reshape(B_, S, 1, G, N)
        if v.qk_norm:
            Bm = F_.rmsnorm(Bm, self.B_norm_weight, 1e-5)
            Cm = F_.rmsnorm(Cm, self.C_norm_weight, 1e-5)
        DT = F.softplus(dd_dt.float() + self.dt_bias)                          # [B,S,H]
        if v.data_dependent_a:
            A = torch.clamp(-F.softplus(dd_A.float()), max=-self.cfg.mamba3.a_floor)
        else:
            A = -torch.exp(self.A_log).expand_as(DT)
        ADT = (A * DT).transpose(1, 2)
        DTt = DT.transpose(1, 2)
        trap_t = trap.float().transpose(1, 2) if trap is not None else torch.full_like(DTt, 30.0)
        n_ang = self.n_angles or self.cfg.mamba3.num_rope_angles
        angles = (mimo_scan_ref.angle_cumsum(ang, DTt) if ang is not None
                  else torch.zeros(B_, S, H, n_ang, dtype=torch.float32, device=x.device))
        zeros = torch.zeros(H, 1, N, dtype=torch.float32, device=x.device)
        ones = torch.ones(H, 1, P, dtype=torch.float32, device=x.device)
        y = mimo_scan_ref.mimo_scan_chunked(
            Cm, Bm, xs.reshape(B_, S, H, P), ADT, DTt, trap_t, self.C_bias if v.bc_bias else zeros,
            self.B_bias if v.bc_bias else zeros, ones, None, ones, angles, self.D, None,
            self.cfg.mamba3.rotary_dim_divisor, max(self.cfg.mamba3.chunk_size, 32))
        y = self.norm(y.reshape(B_, S, self.d_inner).to(x.dtype)) * F.silu(z)
        return self.out_proj(y)


def build_variant_mixer(cfg: ModelConfig, pc: ParallelContext, layer_number: int, *, dtype, seed: int, out_std: float):
    if cfg.mamba_variant not in VARIANTS:
        raise ValueError(f"unknown mamba_variant {cfg.mamba_variant!r}")
    return SSDMixer(cfg, pc, layer_number, VARIANTS[cfg.mamba_variant], dtype=dtype, seed=seed, out_std=out_std)
