"""Mixture-of-experts MLP: fp32 router (sigmoid/softmax scores, bias-corrected top-k),
dropless expert-parallel dispatch, grouped SwiGLU experts, shared expert.

Checkpoint keys mirror Megatron's MoE layer: ``router.weight``, ``router.expert_bias``,
``experts.linear_fc1.weight<e>`` / ``experts.linear_fc2.weight<e>`` (stored here stacked
as ``experts.weight1`` [E_local, 2*ffn, H] and ``experts.weight2`` [E_local, H, ffn]) and
``shared_experts.linear_fc{1,2}.weight`` (cppmega/recipes/megatron_args.py:47-57,108-135;
router options at cppmega/recipes/nam56r_nemo_recipe.py:321-337).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config.model import MoEConfig
from ..ops import functional as F_
from ..ops import reference as ref
from ..parallel.expert_parallel import AllToAllDispatcher
from ..parallel.state import ParallelContext
from .common import DenseMLP, seed_for


class Router(nn.Module):
    def __init__(self, hidden: int, cfg: MoEConfig, *, std: float, seed: int, sequence_parallel: bool):
        super().__init__()
        self.cfg = cfg
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        w = torch.empty(cfg.num_experts, hidden, dtype=torch.float32).normal_(0, std, generator=gen)
        self.weight = nn.Parameter(w)                 # router runs in fp32
        self.weight.keep_fp32 = True
        self.weight.sequence_parallel_grad = sequence_parallel
        if cfg.expert_bias:
            self.register_buffer("expert_bias", torch.zeros(cfg.num_experts, dtype=torch.float32))
            self.register_buffer("tokens_per_expert", torch.zeros(cfg.num_experts, dtype=torch.float32),
                                 persistent=False)
        else:
            self.expert_bias = None

    def forward(self, x: torch.Tensor):
        logits = F_.linear_fp32out(x, self.weight)
        probs, ids, scores = F_.router_topk(logits, self.cfg.topk, self.cfg.score_function,
                                            self.expert_bias, self.cfg.norm_topk_prob)
        if self.expert_bias is not None and self.training:
            with torch.no_grad():
                self.tokens_per_expert += torch.bincount(ids.reshape(-1), minlength=self.cfg.num_experts).float()
        return probs, ids, scores

    @torch.no_grad()
    def update_expert_bias(self, group=None):
        """Auxiliary-loss-free balancing: nudge the selection bias toward under-used experts."""
        if self.expert_bias is None:
            return
        cnt = self.tokens_per_expert.clone()
        if group is not None and dist.is_initialized():
            dist.all_reduce(cnt, group=group)
        if cnt.sum() > 0:
            self.expert_bias += self.cfg.bias_update_rate * torch.sign(cnt.mean() - cnt)
        self.tokens_per_expert.zero_()


_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index
    st = _SIDE_STREAMS.get(key)
    if st is None:
        st = _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return st


class GroupedExperts(nn.Module):
    """``E_local`` SwiGLU experts evaluated with grouped GEMMs over expert-sorted rows."""

    def __init__(self, hidden: int, cfg: MoEConfig, pc: ParallelContext, name: str, *, std: float,
                 out_std: float, dtype, seed: int):
        super().__init__()
        self.e_local = cfg.num_experts // pc.ep
        lo = pc.ep_rank * self.e_local
        w1 = torch.empty(self.e_local, 2 * cfg.expert_ffn, hidden, dtype=torch.float32)
        w2 = torch.empty(self.e_local, hidden, cfg.expert_ffn, dtype=torch.float32)
        for i in range(self.e_local):
            gen = torch.Generator(device="cpu")
            gen.manual_seed(seed_for(f"{name}.expert{lo + i}", seed))
            w1[i].normal_(0, std, generator=gen)
            w2[i].normal_(0, out_std, generator=gen)
        self.weight1 = nn.Parameter(w1.to(dtype))
        self.weight2 = nn.Parameter(w2.to(dtype))
        for p in (self.weight1, self.weight2):
            p.is_expert = True
            p.expert_offset = lo
            p.sequence_parallel_grad = pc.sequence_parallel
        self.last_counts: Optional[torch.Tensor] = None

    def forward(self, x: torch.Tensor, counts: torch.Tensor, counts_host=None) -> torch.Tensor:
        return F_.moe_experts(x, self.weight1, self.weight2, counts, counts_host)


class MoELayer(nn.Module):
    def __init__(self, hidden: int, cfg: MoEConfig, pc: ParallelContext, layer_name: str, *,
                 init_std: float = 0.02, out_std: float = 0.02, dtype=torch.float32, seed: int = 1234):
        super().__init__()
        self.cfg, self.pc = cfg, pc
        n = layer_name + ".mlp"
        self.router = Router(hidden, cfg, std=init_std, seed=seed_for(n + ".router", seed),
                             sequence_parallel=pc.sequence_parallel)
        self.experts = GroupedExperts(hidden, cfg, pc, n + ".experts", std=init_std, out_std=out_std,
                                      dtype=dtype, seed=seed)
        self.shared_experts = (DenseMLP(hidden, cfg.shared_expert_ffn, pc, std=init_std, out_std=out_std,
                                        dtype=dtype, name=n + ".shared_experts", seed=seed)
                               if cfg.shared_expert_ffn > 0 else None)
        self.dispatcher = AllToAllDispatcher(pc, cfg.num_experts)
        self.fused_dispatcher = None          # set by parallel.fused_moe.attach() on peer-capable GPUs
        self.overlap_shared_expert = False    # opt-in, EP > 1: shared expert on a second stream beside the routed path
        self.last_aux_loss: Optional[torch.Tensor] = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        flat = x.reshape(B * S, H)
        probs, ids, scores = self.router(flat)
        self.last_aux_loss = None
        if self.cfg.aux_loss_coeff > 0 and self.training:
            self.last_aux_loss = ref.moe_aux_loss(scores, ids, self.cfg.num_experts, self.cfg.topk,
                                                  self.cfg.aux_loss_coeff)
        shared = None
        overlap = (self.shared_experts is not None and self.fused_dispatcher is not None and flat.is_cuda and self.pc.ep > 1
                   and self.overlap_shared_expert)
        if overlap:
            # The routed path spends most of its time in NVLink row transfers and flag waits, which leave the SMs'
            # tensor cores idle: the shared expert (no communication) runs beside it on a second stream, forward and,
            # through autograd's stream bookkeeping, backward.
            main = torch.cuda.current_stream()
            side = _side_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                shared = self.shared_experts(x)
        if self.fused_dispatcher is not None and flat.is_cuda:
            y = self.fused_dispatcher(flat, probs, ids, self.experts)
        else:
            xs, plan = self.dispatcher.dispatch(flat, ids)
            ys = self.experts(xs, plan.counts_local, plan.counts_local_host)
            y = self.dispatcher.combine(ys, probs, plan)
        y = y.reshape(B, S, H)
        if overlap:
            main.wait_stream(side)
            shared.record_stream(main)
            y = y + shared
        elif self.shared_experts is not None:
            y = y + self.shared_experts(x)
        return y
