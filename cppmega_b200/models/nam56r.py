"""NAM56R hybrid language model: embedding -> hybrid stack -> final norm -> fused linear CE,
plus multi-token-prediction heads.

The module tree uses the key names of the reference's checkpoints
(``embedding.*``, ``decoder.layers.N.{norm,mixer | input_layernorm,self_attention |
pre_mlp_layernorm,mlp}``, ``decoder.final_norm``, ``output_layer``, ``mtp.layers.D.*``), the
layer selection of its production spec (Mamba3 vs M2RNN per ``M`` layer, DSA vs MLA per
attention rank; cppmega/megatron/nam56r_full_spec.py:77-259), and the loss composition
of its MTP patches (cppmega/megatron/mtp_liger_ce.py:99-233 and the single-launch
main+MTP cross entropy of cppmega/megatron/mtp_native_hopper_ce.py:185-267).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn
from ..utils.recompute import checkpoint

from ..config.model import ModelConfig
from ..ops import functional as F_
from ..parallel.state import ParallelContext, get_context
from ..parallel.tensor_parallel import ColumnParallelLinear, gather_seq
from .attention import IndexCacheState, MLAttention
from .common import DenseMLP, RMSNorm, cast_module_params, seed_for
from .embedding import LanguageModelEmbedding
from .m2rnn import M2RNNMixer
from .mamba3 import Mamba3Mixer
from .moe import MoELayer

IGNORE_INDEX = -100


class HybridLayer(nn.Module):
    """pre-norm -> mixer/attention/MLP -> residual add.  One symbol of the pattern."""

    def __init__(self, cfg: ModelConfig, pc: ParallelContext, layer_number: int, kind: str, *,
                 dtype, seed: int, dsa_rank: int = -1, name_prefix: str = "decoder.layers"):
        super().__init__()
        self.kind, self.layer_number = kind, layer_number
        h = cfg.hidden_size
        out_std = cfg.init_std / (2.0 * cfg.depth) ** 0.5
        lname = f"{name_prefix}.{layer_number - 1}"
        norm = RMSNorm(h, cfg.norm_eps, dtype=dtype, sequence_parallel=pc.sequence_parallel)
        if kind == "mamba3":
            self.norm = norm
            if cfg.mamba_variant == "mimo":
                self.mixer = Mamba3Mixer(h, cfg.mamba3, pc, layer_number, init_std=cfg.init_std, out_std=out_std,
                                         dtype=dtype, seed=seed)
            else:
                from .mamba_variants import build_variant_mixer
                self.mixer = build_variant_mixer(cfg, pc, layer_number, dtype=dtype, seed=seed, out_std=out_std)
        elif kind == "m2rnn":
            self.norm = norm
            self.mixer = M2RNNMixer(h, cfg.m2rnn, pc, layer_number, init_std=cfg.init_std, out_std=out_std,
                                    eps=cfg.norm_eps, dtype=dtype, seed=seed)
        elif kind in ("mla", "dsa"):
            self.input_layernorm = norm
            self.self_attention = MLAttention(h, cfg.mla, pc, lname, dsa=cfg.dsa if kind == "dsa" else None,
                                              dsa_rank=dsa_rank, init_std=cfg.init_std, out_std=out_std,
                                              eps=cfg.norm_eps, dtype=dtype, seed=seed)
        elif kind == "moe":
            self.pre_mlp_layernorm = norm
            self.mlp = MoELayer(h, cfg.moe, pc, lname, init_std=cfg.init_std, out_std=out_std, dtype=dtype, seed=seed)
        elif kind == "mlp":
            self.pre_mlp_layernorm = norm
            self.mlp = DenseMLP(h, cfg.ffn_hidden_size, pc, std=cfg.init_std, out_std=out_std, dtype=dtype,
                                name=lname + ".mlp", seed=seed)
        else:
            raise ValueError(f"unknown layer kind {kind!r}")

    def forward(self, x: torch.Tensor, index_cache: Optional[IndexCacheState] = None,
                indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        k = self.kind
        if k in ("mamba3", "m2rnn"):
            return x + self.mixer(self.norm(x))
        if k in ("mla", "dsa"):
            return x + self.self_attention(self.input_layernorm(x), index_cache, indices)
        return x + self.mlp(self.pre_mlp_layernorm(x))

    @torch.no_grad()
    def select_indices(self, x: torch.Tensor, index_cache: Optional[IndexCacheState]) -> torch.Tensor:
        return self.self_attention.select_indices(self.input_layernorm(x), index_cache)


class MTPLayer(nn.Module):
    """One prediction depth: ``eh_proj([enorm(emb(shifted ids)) | hnorm(h_prev)])`` ->
    attention + dense MLP -> final norm."""

    def __init__(self, cfg: ModelConfig, pc: ParallelContext, depth_index: int, *, dtype, seed: int):
        super().__init__()
        h = cfg.hidden_size
        sp = pc.sequence_parallel
        self.enorm = RMSNorm(h, cfg.norm_eps, dtype=dtype, sequence_parallel=sp)
        self.hnorm = RMSNorm(h, cfg.norm_eps, dtype=dtype, sequence_parallel=sp)
        n = f"mtp.layers.{depth_index}"
        self.eh_proj = ColumnParallelLinear(2 * h, h, pc, std=cfg.init_std, dtype=dtype, gather_output=True,
                                            seed=seed_for(n + ".eh_proj", seed), name=n + ".eh_proj")
        self.transformer_layer = nn.ModuleList([
            HybridLayer(cfg, pc, 1, "mla", dtype=dtype, seed=seed + 17 * (depth_index + 1), name_prefix=n + ".attn"),
            HybridLayer(cfg, pc, 1, "mlp", dtype=dtype, seed=seed + 31 * (depth_index + 1), name_prefix=n + ".mlp"),
        ])
        self.final_layernorm = RMSNorm(h, cfg.norm_eps, dtype=dtype, sequence_parallel=sp)
        self.pc = pc

    def forward(self, h_prev: torch.Tensor, emb: torch.Tensor) -> torch.Tensor:
        x = torch.cat([self.enorm(emb), self.hnorm(h_prev)], dim=-1)
        x = self.eh_proj(x)
        if self.pc.sequence_parallel:
            from ..parallel.tensor_parallel import scatter_seq
            x = scatter_seq(x, self.pc)
        for layer in self.transformer_layer:
            x = layer(x)
        return x


def roll_left(t: torch.Tensor, shifts: int = 1, fill=0) -> torch.Tensor:
    """Shift along the sequence (dim 1) to the left, filling the tail."""
    out = torch.roll(t, shifts=-shifts, dims=1)
    out[:, -shifts:] = fill
    return out


class NAM56RModel(nn.Module):
    def __init__(self, cfg: ModelConfig, pc: Optional[ParallelContext] = None, *, dtype=torch.float32,
                 seed: int = 1234, layer_numbers: Optional[Sequence[int]] = None,
                 pre_process: bool = True, post_process: bool = True,
                 recompute: str = "none", device=None, recompute_keep_last: int = 0):
        """``layer_numbers`` (1-indexed) selects the layers of this pipeline stage; ``recompute``
        is ``none`` | ``full`` (checkpoint every layer) | ``selective`` (checkpoint the
        mixer layers only, cppmega/megatron/mamba_recompute_patch.py:41-118)."""
        super().__init__()
        pc = pc or get_context()
        self.cfg, self.pc, self.dtype = cfg, pc, dtype
        self.pre_process, self.post_process = pre_process, post_process
        self.recompute = recompute
        self.recompute_keep_last = recompute_keep_last      # the last K layers of this stage keep their activations
        kinds = cfg.layer_kinds()
        dsa_ranks = cfg.dsa_rank_of_layer()
        self.layer_numbers = list(layer_numbers) if layer_numbers is not None else list(range(1, cfg.depth + 1))
        has_mtp = post_process and cfg.mtp.num_layers > 0 and not cfg.mtp.fastmtp
        if pre_process or has_mtp or (post_process and cfg.mtp.fastmtp):
            self.embedding = LanguageModelEmbedding(cfg, pc, dtype=dtype, seed=seed)
            self.embedding.is_mtp_copy = not pre_process
        self.decoder = nn.Module()
        self.decoder.layers = nn.ModuleDict({
            str(n - 1): HybridLayer(cfg, pc, n, kinds[n - 1], dtype=dtype, seed=seed, dsa_rank=dsa_ranks.get(n, -1))
            for n in self.layer_numbers
        })
        if post_process:
            self.decoder.final_norm = RMSNorm(cfg.hidden_size, cfg.norm_eps, dtype=dtype,
                                              sequence_parallel=pc.sequence_parallel)
            if cfg.tie_embeddings and pre_process:
                self.output_layer = None
            else:
                self.output_layer = ColumnParallelLinear(cfg.hidden_size, cfg.vocab_size, pc, std=cfg.init_std,
                                                         dtype=dtype, seed=seed_for("output_layer", seed),
                                                         name="output_layer")
                self.output_layer.weight.is_embedding_or_output_parameter = True
            if has_mtp:
                self.mtp = nn.Module()
                self.mtp.layers = nn.ModuleList([MTPLayer(cfg, pc, d, dtype=dtype, seed=seed)
                                                 for d in range(cfg.mtp.num_layers)])
            if cfg.mtp.fastmtp:
                from .fastmtp import FastMTPHead
                self.fastmtp = FastMTPHead(cfg, dtype=dtype, seed=seed)
        cast_module_params(self, dtype)
        if device is not None:
            self.to(device)
        self.last_metrics: Dict[str, torch.Tensor] = {}

    # ---- pieces -----------------------------------------------------------
    def output_weight(self) -> torch.Tensor:
        if self.output_layer is None:
            return self.embedding.word_embeddings.weight
        return self.output_layer.weight

    def run_layers(self, x: torch.Tensor, index_cache: Optional[IndexCacheState] = None) -> torch.Tensor:
        cache = index_cache if index_cache is not None else IndexCacheState()
        self.index_cache = cache
        n_layers = len(self.decoder.layers)
        from ..utils import fp8_activations as fa
        act = getattr(self, "fp8_activations", None) or {}
        for pos, (key, layer) in enumerate(self.decoder.layers.items()):
            fa.set_current_layer_idx(pos)
            with fa.fp8_activation_context(n_layers=n_layers, enabled=bool(act) and self.training, **act):
                x = self._run_layer(pos, n_layers, layer, x, cache)
        fa.set_current_layer_idx(-1)
        return x

    def _run_layer(self, pos: int, n_layers: int, layer, x: torch.Tensor, cache) -> torch.Tensor:
        ck = self.training and (self.recompute == "full" or
                                (self.recompute == "selective" and layer.kind in ("mamba3", "m2rnn")))
        if pos >= n_layers - self.recompute_keep_last or getattr(layer, "_graphed", None) is not None:
            ck = False      # kept layers and CUDA-graph-captured layers hold their activations
        if ck and layer.kind == "dsa" and self.cfg.dsa.indexer_loss_coeff > 0:
            ck = False      # the indexer loss needs the layer's own graph
        if ck and layer.kind == "dsa":
            # pick the indices once, outside the checkpoint, so the recomputation in
            # backward replays the layer with the same selection
            idx = layer.select_indices(x, cache)
            x = checkpoint(layer, x, None, idx)
        elif ck:
            x = checkpoint(layer, x, None, None)
        else:
            x = layer(x, cache)
        return x

    def aux_losses(self) -> Optional[torch.Tensor]:
        total = None
        for layer in self.decoder.layers.values():
            for t in (getattr(getattr(layer, "mlp", None), "last_aux_loss", None),
                      getattr(getattr(layer, "self_attention", None), "last_indexer_loss", None)):
                if t is not None:
                    total = t if total is None else total + t
        return total

    # ---- forward ----------------------------------------------------------
    def forward(self, input_ids: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                loss_mask: Optional[torch.Tensor] = None, hidden_in: Optional[torch.Tensor] = None,
                structure_inputs: Optional[Dict[str, torch.Tensor]] = None):
        """First stage consumes ``input_ids``; later stages consume ``hidden_in``.  Stages
        without ``post_process`` return hidden states; the last stage returns a dict with
        ``loss`` (scalar to differentiate), ``lm_loss``, ``mtp_losses`` and ``num_tokens``
        when ``labels`` is given, else the final hidden states."""
        if self.pre_process:
            x = self.embedding(input_ids, structure_inputs)
        else:
            x = hidden_in
        x = self.run_layers(x)
        if not self.post_process:
            return x
        if labels is None:
            return self.decoder.final_norm(x)
        return self.compute_loss(x, input_ids, labels, loss_mask, structure_inputs)

    def compute_loss(self, x, input_ids, labels, loss_mask, structure_inputs=None):
        cfg, pc = self.cfg, self.pc
        B, S = labels.shape
        if loss_mask is None:
            loss_mask = torch.ones_like(labels, dtype=torch.float32)
        loss_mask = loss_mask.float()
        hiddens = [self.decoder.final_norm(x)]
        label_list = [labels.masked_fill(loss_mask == 0, IGNORE_INDEX)]
        mask_list = [loss_mask]
        if hasattr(self, "mtp"):
            h_prev, ids_d, lab_d, msk_d = x, input_ids, labels, loss_mask
            for layer in self.mtp.layers:
                ids_d = roll_left(ids_d, 1, 0)
                lab_d = roll_left(lab_d, 1, 0)
                msk_d = roll_left(msk_d, 1, 0.0)
                emb = self.embedding(ids_d, structure_inputs)
                h_prev = layer(h_prev, emb)
                hiddens.append(layer.final_layernorm(h_prev))
                label_list.append(lab_d.masked_fill(msk_d == 0, IGNORE_INDEX))
                mask_list.append(msk_d)
        w = self.output_weight()
        if pc.sequence_parallel:
            hiddens = [gather_seq(h, pc, reduce_grad=False) for h in hiddens]   # CE all-reduces dh itself
        # one weighted cross-entropy over [main | depth 1 | ... | depth D]: the row weights carry the
        # loss mask, the per-head token count and the MTP depth scaling
        D = len(hiddens) - 1
        counts = [m.sum().clamp_min(1.0) for m in mask_list]
        scales = [1.0] + [cfg.mtp.loss_scaling_factor / max(D, 1)] * D
        row_w = torch.cat([(m * (sc / n)).reshape(-1) for m, sc, n in zip(mask_list, scales, counts)])
        if cfg.mtp.fused_with_main_ce or D == 0:
            hcat = torch.cat([h.reshape(B * S, -1) for h in hiddens], dim=0) if D else hiddens[0].reshape(B * S, -1)
            lcat = torch.cat([l.reshape(-1) for l in label_list], dim=0)
            total, per_tok = self._ce(hcat, w, lcat, row_w)
        else:
            total, parts = None, []
            for i, (h, l) in enumerate(zip(hiddens, label_list)):
                t_i, p_i = self._ce(h.reshape(B * S, -1), w, l.reshape(-1), row_w[i * B * S:(i + 1) * B * S])
                total = t_i if total is None else total + t_i
                parts.append(p_i)
            per_tok = torch.cat(parts)
        per_tok = per_tok.view(D + 1, B * S)
        n_main = counts[0]
        lm_loss = (per_tok[0] * mask_list[0].reshape(-1)).sum() / n_main
        mtp_losses: List[torch.Tensor] = []
        for d in range(1, D + 1):
            mtp_losses.append(((per_tok[d] * mask_list[d].reshape(-1)).sum() / counts[d]).detach())
        if hasattr(self, "fastmtp"):
            fl = self.fastmtp(x.detach(), input_ids, labels, loss_mask, self.embedding, w.detach())
            total = total + cfg.mtp.fastmtp_lambda * fl
            mtp_losses.append(fl.detach())
        aux = self.aux_losses()
        if aux is not None:
            total = total + aux
        out = {"loss": total, "lm_loss": lm_loss.detach(), "mtp_losses": mtp_losses,
               "num_tokens": n_main.detach(), "aux_loss": None if aux is None else aux.detach()}
        self.last_metrics = out
        return out

    def _ce(self, hidden, weight, labels, row_weights):
        if self.pc.tp > 1:
            from ..parallel.vocab_parallel import vocab_parallel_linear_cross_entropy
            per_tok = vocab_parallel_linear_cross_entropy(hidden, weight, labels, self.pc, IGNORE_INDEX)
            return (per_tok * row_weights).sum(), per_tok.detach()
        return F_.linear_cross_entropy_weighted(hidden, weight, labels, row_weights, IGNORE_INDEX)

    # ---- housekeeping -----------------------------------------------------
    def moe_layers(self):
        return [l.mlp for l in self.decoder.layers.values() if l.kind == "moe"]

    @torch.no_grad()
    def update_router_biases(self):
        grp = self.pc.dp_group if self.pc.dp > 1 else None
        for m in self.moe_layers():
            m.router.update_expert_bias(grp)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())


def build_model(cfg: ModelConfig, pc: Optional[ParallelContext] = None, *, dtype=torch.float32,
                seed: int = 1234, recompute: str = "none", device=None, recompute_keep_last: int = 0) -> NAM56RModel:
    """Build the model chunk of this rank's pipeline stage."""
    pc = pc or get_context()
    if pc.pp == 1:
        return NAM56RModel(cfg, pc, dtype=dtype, seed=seed, recompute=recompute, device=device,
                           recompute_keep_last=recompute_keep_last)
    from ..parallel.pipeline import stage_layer_numbers
    layers = stage_layer_numbers(cfg.depth, pc.pp, pc.pp_rank)
    return NAM56RModel(cfg, pc, dtype=dtype, seed=seed, layer_numbers=layers,
                       pre_process=pc.is_first_pp, post_process=pc.is_last_pp,
                       recompute=recompute, device=device, recompute_keep_last=recompute_keep_last)


_ = dist
