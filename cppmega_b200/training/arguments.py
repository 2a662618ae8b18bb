"""Megatron-style command line <-> typed configuration.

``parse_args(argv)`` accepts the flag names the reference's launchers pass to Megatron
(``--hybrid-layer-pattern``, ``--tensor-model-parallel-size``, ``--expert-model-parallel-size``,
``--use-distributed-optimizer``, ``--mtp-num-layers``, MLA / DSA / MoE flags; see
cppmega/recipes/megatron_args.py:34-173 and scripts/remote_smoke_h200_dsa_9_4_m.sh:691-740) and returns
``(ModelConfig, ParallelConfig, TrainConfig, extras)``.  ``render_args`` is the inverse and is what
the recipes and run profiles emit.  There is no environment-variable tier.
"""
from __future__ import annotations

import argparse
import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

from ..config.model import (DSAConfig, MLAConfig, Mamba3Config, ModelConfig, MoEConfig, MTPConfig, NgramHashConfig,
                            StructureConfig, get_preset)
from ..config.pattern import PatternError, parse_hybrid_pattern, parse_int_list
from ..parallel.dist_optimizer import OptimizerConfig
from ..parallel.state import ParallelConfig
from .lr import LRSchedule
from .trainer import TrainConfig

HYBRID_TO_NAM = {"*": "A", "M": "M", "E": "E", "-": "D", "G": "G"}


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="cppmega_b200.pretrain", allow_abbrev=False,
                                description="NAM56R pre-training (B200-native)")
    g = p.add_argument_group("model")
    g.add_argument("--model-preset", default="nam56r")
    g.add_argument("--hybrid-layer-pattern", default=None,
                   help="main stack in the hybrid alphabet (*, M, E, -), pipes between pipeline chunks, "
                        "'/*-' per MTP depth")
    g.add_argument("--nam-pattern", default=None, help="recipe alphabet (A, M, R, E, D), tiled to --num-layers")
    g.add_argument("--num-layers", type=int, default=None)
    g.add_argument("--hidden-size", type=int, default=None)
    g.add_argument("--ffn-hidden-size", type=int, default=None)
    g.add_argument("--num-attention-heads", type=int, default=None)
    g.add_argument("--seq-length", type=int, default=None)
    g.add_argument("--max-position-embeddings", type=int, default=None)
    g.add_argument("--vocab-size", type=int, default=None)
    g.add_argument("--make-vocab-size-divisible-by", type=int, default=128)
    g.add_argument("--norm-epsilon", type=float, default=None)
    g.add_argument("--init-method-std", type=float, default=None)
    g.add_argument("--rotary-base", type=float, default=None)
    g.add_argument("--untie-embeddings-and-output-weights", action="store_true", default=None)
    g.add_argument("--r-layer-indices", default=None, help="1-indexed mixer layers that run M2RNN")
    g.add_argument("--dsa-a-layer-ranks", default=None, help="attention ranks that run DSA")
    g = p.add_argument_group("mamba3")
    g.add_argument("--mamba-state-dim", type=int, default=None)
    g.add_argument("--mamba-head-dim", type=int, default=None)
    g.add_argument("--mamba-num-groups", type=int, default=None)
    g.add_argument("--mamba-expand", type=int, default=None)
    g.add_argument("--mamba3-mimo-rank", type=int, default=None)
    g.add_argument("--mamba3-chunk-size", type=int, default=None)
    g.add_argument("--mamba3-rope-fraction", type=float, default=None)
    g.add_argument("--mamba-variant", default=None, choices=["mimo", "noconv_ssd", "ssd"])
    g = p.add_argument_group("mla / dsa")
    g.add_argument("--multi-latent-attention", action="store_true", default=None)
    g.add_argument("--q-lora-rank", type=int, default=None)
    g.add_argument("--kv-lora-rank", type=int, default=None)
    g.add_argument("--qk-head-dim", type=int, default=None)
    g.add_argument("--qk-pos-emb-head-dim", type=int, default=None)
    g.add_argument("--v-head-dim", type=int, default=None)
    g.add_argument("--experimental-attention-variant", default=None, choices=["dsa"])
    g.add_argument("--dsa-indexer-n-heads", type=int, default=None)
    g.add_argument("--dsa-indexer-head-dim", type=int, default=None)
    g.add_argument("--dsa-indexer-topk", type=int, default=None)
    g.add_argument("--dsa-indexer-loss-coeff", type=float, default=None)
    g.add_argument("--dsa-warmup-dense", action="store_true", default=None,
                   help="indexer warm-up: sparse layers attend densely while the KL loss trains the indexer")
    g.add_argument("--index-cache", dest="index_cache", action="store_true", default=None)
    g.add_argument("--no-index-cache", dest="index_cache", action="store_false")
    g.add_argument("--index-cache-full-layers", default=None)
    g = p.add_argument_group("moe")
    g.add_argument("--num-experts", type=int, default=None)
    g.add_argument("--moe-router-topk", type=int, default=None)
    g.add_argument("--moe-ffn-hidden-size", type=int, default=None)
    g.add_argument("--moe-shared-expert-intermediate-size", type=int, default=None)
    g.add_argument("--moe-token-dispatcher-type", default=None, choices=["alltoall", "allgather", "flex"])
    g.add_argument("--moe-flex-dispatcher-backend", default=None)
    g.add_argument("--moe-router-dtype", default=None, choices=["fp32", "bf16"])
    g.add_argument("--moe-router-score-function", default=None, choices=["sigmoid", "softmax"])
    g.add_argument("--moe-router-enable-expert-bias", action="store_true", default=None)
    g.add_argument("--moe-aux-loss-coeff", type=float, default=None)
    g.add_argument("--moe-grouped-gemm", action="store_true", default=None)
    g.add_argument("--moe-router-fusion", action="store_true", default=None)
    g.add_argument("--moe-permute-fusion", action="store_true", default=None)
    g = p.add_argument_group("mtp / loss")
    g.add_argument("--mtp-num-layers", type=int, default=None)
    g.add_argument("--mtp-loss-scaling-factor", type=float, default=None)
    g.add_argument("--multi-token-prediction", action="store_true", default=None)
    g.add_argument("--fastmtp", action="store_true", default=None)
    g.add_argument("--fastmtp-depth", type=int, default=None)
    g.add_argument("--fastmtp-decay", type=float, default=None)
    g.add_argument("--fastmtp-lambda", type=float, default=None)
    g.add_argument("--no-fuse-main-mtp-ce", action="store_true", default=None)
    g = p.add_argument_group("embeddings")
    g.add_argument("--ngram-hash", dest="ngram_hash", action="store_true", default=None)
    g.add_argument("--no-ngram-hash", dest="ngram_hash", action="store_false")
    g.add_argument("--ngram-hash-orders", default=None)
    g.add_argument("--ngram-hash-heads", type=int, default=None)
    g.add_argument("--ngram-hash-table-size", type=int, default=None)
    g.add_argument("--ngram-hash-embed-dim", type=int, default=None)
    g.add_argument("--ngram-hash-offload", action="store_true", default=None)
    g.add_argument("--structure-embedding", action="store_true", default=None)
    g.add_argument("--structure-components", default=None)
    g.add_argument("--structure-bottleneck-dim", type=int, default=None)
    g = p.add_argument_group("parallelism")
    g.add_argument("--tensor-model-parallel-size", type=int, default=1)
    g.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    g.add_argument("--virtual-pipeline-model-parallel-size", type=int, default=1)
    g.add_argument("--expert-model-parallel-size", type=int, default=1)
    g.add_argument("--context-parallel-size", type=int, default=1)
    g.add_argument("--sequence-parallel", action="store_true")
    g.add_argument("--use-distributed-optimizer", action="store_true")
    g.add_argument("--overlap-grad-reduce", action="store_true")
    g.add_argument("--overlap-param-gather", action="store_true")
    g.add_argument("--no-fused-collectives", action="store_true",
                   help="use the plain NCCL collectives (the measured baseline) instead of the peer-memory kernels")
    g.add_argument("--pipeline-schedule", default="1f1b", choices=["1f1b", "interleaved", "dualpipev"])
    g = p.add_argument_group("training")
    g.add_argument("--micro-batch-size", type=int, default=4)
    g.add_argument("--global-batch-size", type=int, default=None)
    g.add_argument("--train-iters", type=int, default=100)
    g.add_argument("--bf16", action="store_true")
    g.add_argument("--fp32", action="store_true")
    g.add_argument("--fp8-recipe", default=None, choices=["mxfp8", "tensorwise"],
                   help="mxfp8: E4M3 with E8M0 scales per 32 values; tensorwise: E4M3 with one current-scaling scale per tensor")
    g.add_argument("--fp8-modules", nargs="*", default=[],
                   help="restrict the FP8 recipe to modules whose qualified name matches one of these glob patterns "
                        "(shorthands: moe, mamba_proj); everything else stays bf16")
    g.add_argument("--fp8-activations", default="off", choices=["off", "mxfp8", "tensor"],
                   help="store the activations saved for backward as E4M3 + scales (block scales / one scale per tensor)")
    g.add_argument("--fp8-activations-bf16-first", type=int, default=1, help="layers at the start of the stack that keep bf16")
    g.add_argument("--fp8-activations-bf16-last", type=int, default=1, help="layers at the end of the stack that keep bf16")
    g.add_argument("--fp8-activations-clamp", action="store_true", help="tensor recipe: limit the measured maximum to 448")
    g.add_argument("--recompute-granularity", default=None, choices=["selective", "full"])
    g.add_argument("--cuda-graph-scope", nargs="*", default=[],
                   help="layer kinds captured as CUDA graphs: mamba attn mlp (moe_router / moe_preprocess are accepted and ignored)")
    g.add_argument("--seed", type=int, default=1234)
    g.add_argument("--deterministic-mode", action="store_true",
                   help="debugging: bitwise-reproducible reruns (kernels with atomic reductions run their PyTorch definitions)")
    g.add_argument("--inject-failure-at-iteration", type=int, default=0,
                   help="testing aid: the last rank raises after this iteration unless the run was resumed from a checkpoint")
    g.add_argument("--optimizer", default="adamw", choices=["adam", "adamw", "adam8bit", "muon"])
    g.add_argument("--muon-scalar-optimizer", default="adamw", choices=["adamw", "adam8bit"],
                   help="optimizer of the parameters Muon does not take (scalars, norms, embeddings, output layer)")
    g.add_argument("--lr", type=float, default=1e-5)
    g.add_argument("--min-lr", type=float, default=0.0)
    g.add_argument("--lr-decay-style", default="constant", choices=["constant", "cosine", "linear", "wsd"])
    g.add_argument("--lr-warmup-iters", type=int, default=0)
    g.add_argument("--lr-decay-iters", type=int, default=0)
    g.add_argument("--weight-decay", type=float, default=0.1)
    g.add_argument("--adam-beta1", type=float, default=0.9)
    g.add_argument("--adam-beta2", type=float, default=0.95)
    g.add_argument("--adam-eps", type=float, default=1e-8)
    g.add_argument("--clip-grad", type=float, default=1.0)
    g.add_argument("--grad-reduce-in-bf16", action="store_true")
    g.add_argument("--muon-momentum", type=float, default=0.95)
    g.add_argument("--muon-quantized-momentum", action="store_true")
    g.add_argument("--no-check-for-nan-in-loss-and-grad", action="store_true")
    g = p.add_argument_group("data / io")
    g.add_argument("--data-path", default=None, help="prefix of an indexed .bin/.idx token dataset")
    g.add_argument("--mock-data", action="store_true", help="synthetic uniform tokens")
    g.add_argument("--save", default=None)
    g.add_argument("--load", default=None)
    g.add_argument("--no-load-optim", action="store_true",
                   help="when the optimizer shards cannot be restored (other parallel layout, missing file), continue from "
                        "the weights with fresh AdamW moments instead of failing")
    g.add_argument("--save-interval", type=int, default=0)
    g.add_argument("--log-interval", type=int, default=1)
    g.add_argument("--log-throughput", action="store_true")
    g.add_argument("--monitor-port", type=int, default=0)
    g.add_argument("--profile", action="store_true")
    g.add_argument("--profile-step-start", type=int, default=3)
    g.add_argument("--profile-step-end", type=int, default=4)
    g.add_argument("--step-timeout-s", type=float, default=0.0, help="watchdog: abort when a step exceeds this")
    return p


def _set(d: Dict, key: str, val) -> None:
    if val is not None:
        d[key] = val


def configs_from_namespace(ns: argparse.Namespace) -> Tuple[ModelConfig, ParallelConfig, TrainConfig, Dict]:
    base = get_preset(ns.model_preset)
    top: Dict = {}
    mtp_layers = ns.mtp_num_layers
    if ns.hybrid_layer_pattern:
        main, mtp_d, chunks = parse_hybrid_pattern(ns.hybrid_layer_pattern)
        nam = [HYBRID_TO_NAM[s] for s in main]
        for i in parse_int_list(ns.r_layer_indices):
            if not (1 <= i <= len(nam)) or nam[i - 1] != "M":
                raise PatternError(f"--r-layer-indices: layer {i} is not a mixer layer")
            nam[i - 1] = "R"
        top["pattern"] = "|".join("".join(nam[sum(chunks[:c]):sum(chunks[:c + 1])]) for c in range(len(chunks)))
        top["depth"] = len(nam)
        if mtp_layers is None and mtp_d:
            mtp_layers = mtp_d
        if ns.num_layers is not None and ns.num_layers != len(nam):
            raise PatternError(f"--num-layers {ns.num_layers} disagrees with the pattern ({len(nam)} layers)")
    else:
        _set(top, "pattern", ns.nam_pattern)
        _set(top, "depth", ns.num_layers)
    _set(top, "hidden_size", ns.hidden_size)
    _set(top, "ffn_hidden_size", ns.ffn_hidden_size)
    _set(top, "seq_length", ns.seq_length)
    if ns.vocab_size is not None:
        m = ns.make_vocab_size_divisible_by
        top["vocab_size"] = (ns.vocab_size + m - 1) // m * m
    _set(top, "norm_eps", ns.norm_epsilon)
    _set(top, "init_std", ns.init_method_std)
    _set(top, "mamba_variant", ns.mamba_variant)
    if ns.untie_embeddings_and_output_weights:
        top["tie_embeddings"] = False

    m3: Dict = {}
    _set(m3, "d_state", ns.mamba_state_dim)
    _set(m3, "headdim", ns.mamba_head_dim)
    _set(m3, "ngroups", ns.mamba_num_groups)
    _set(m3, "expand", ns.mamba_expand)
    _set(m3, "mimo_rank", ns.mamba3_mimo_rank)
    _set(m3, "chunk_size", ns.mamba3_chunk_size)
    _set(m3, "rope_fraction", ns.mamba3_rope_fraction)
    mla: Dict = {}
    _set(mla, "num_heads", ns.num_attention_heads)
    _set(mla, "q_lora_rank", ns.q_lora_rank)
    _set(mla, "kv_lora_rank", ns.kv_lora_rank)
    _set(mla, "qk_head_dim", ns.qk_head_dim)
    _set(mla, "qk_pos_emb_head_dim", ns.qk_pos_emb_head_dim)
    _set(mla, "v_head_dim", ns.v_head_dim)
    _set(mla, "rope_base", ns.rotary_base)
    dsa: Dict = {}
    _set(dsa, "index_n_heads", ns.dsa_indexer_n_heads)
    _set(dsa, "index_head_dim", ns.dsa_indexer_head_dim)
    _set(dsa, "index_topk", ns.dsa_indexer_topk)
    _set(dsa, "indexer_loss_coeff", ns.dsa_indexer_loss_coeff)
    _set(dsa, "warmup_dense", ns.dsa_warmup_dense)
    _set(dsa, "index_cache", ns.index_cache)
    if ns.index_cache_full_layers is not None:
        dsa["full_layer_ranks"] = parse_int_list(ns.index_cache_full_layers)
    if ns.dsa_a_layer_ranks is not None:
        dsa["attention_ranks"] = parse_int_list(ns.dsa_a_layer_ranks)
    moe: Dict = {}
    _set(moe, "num_experts", ns.num_experts)
    _set(moe, "topk", ns.moe_router_topk)
    _set(moe, "expert_ffn", ns.moe_ffn_hidden_size)
    _set(moe, "shared_expert_ffn", ns.moe_shared_expert_intermediate_size)
    _set(moe, "dispatcher", ns.moe_token_dispatcher_type)
    _set(moe, "flex_backend", ns.moe_flex_dispatcher_backend)
    _set(moe, "router_dtype", ns.moe_router_dtype)
    _set(moe, "score_function", ns.moe_router_score_function)
    _set(moe, "expert_bias", ns.moe_router_enable_expert_bias)
    _set(moe, "aux_loss_coeff", ns.moe_aux_loss_coeff)
    mtp: Dict = {}
    _set(mtp, "num_layers", mtp_layers)
    _set(mtp, "loss_scaling_factor", ns.mtp_loss_scaling_factor)
    _set(mtp, "fastmtp", ns.fastmtp)
    _set(mtp, "fastmtp_depth", ns.fastmtp_depth)
    _set(mtp, "fastmtp_decay", ns.fastmtp_decay)
    _set(mtp, "fastmtp_lambda", ns.fastmtp_lambda)
    if ns.no_fuse_main_mtp_ce:
        mtp["fused_with_main_ce"] = False
    ng: Dict = {}
    _set(ng, "enabled", ns.ngram_hash)
    if ns.ngram_hash_orders is not None:
        ng["orders"] = parse_int_list(ns.ngram_hash_orders)
    _set(ng, "heads", ns.ngram_hash_heads)
    _set(ng, "table_size", ns.ngram_hash_table_size)
    _set(ng, "embed_dim", ns.ngram_hash_embed_dim)
    _set(ng, "offload", ns.ngram_hash_offload)
    st: Dict = {}
    _set(st, "enabled", ns.structure_embedding)
    _set(st, "components", ns.structure_components)
    _set(st, "bottleneck_dim", ns.structure_bottleneck_dim)

    def rep(obj, d):
        return dataclasses.replace(obj, **d) if d else obj

    if moe.get("dispatcher") == "flex" and (ns.expert_model_parallel_size <= 1 or moe.get("router_dtype", base.moe.router_dtype) != "fp32"):
        raise ValueError("the flex dispatcher needs --expert-model-parallel-size > 1 and an fp32 router")
    mcfg = dataclasses.replace(
        base, mamba3=rep(base.mamba3, m3), mla=rep(base.mla, mla), dsa=rep(base.dsa, dsa), moe=rep(base.moe, moe),
        mtp=rep(base.mtp, mtp), ngram_hash=rep(base.ngram_hash, ng), structure=rep(base.structure, st), **top)
    if ns.context_parallel_size != 1:
        raise ValueError("--context-parallel-size must be 1: the sequence mixers do not support context parallelism")
    pcfg = ParallelConfig(tp=ns.tensor_model_parallel_size, pp=ns.pipeline_model_parallel_size,
                          vpp=ns.virtual_pipeline_model_parallel_size, ep=ns.expert_model_parallel_size,
                          sequence_parallel=ns.sequence_parallel, distributed_optimizer=ns.use_distributed_optimizer,
                          overlap_grad_reduce=ns.overlap_grad_reduce, overlap_param_gather=ns.overlap_param_gather,
                          fused_collectives=not ns.no_fused_collectives)
    ocfg = OptimizerConfig(optimizer="adamw" if ns.optimizer in ("adam", "adamw") else ns.optimizer, lr=ns.lr,
                           min_lr=ns.min_lr, weight_decay=ns.weight_decay, beta1=ns.adam_beta1, beta2=ns.adam_beta2,
                           eps=ns.adam_eps, clip_grad=ns.clip_grad, grad_dtype="bf16" if ns.grad_reduce_in_bf16 else "fp32",
                           muon_momentum=ns.muon_momentum, muon_quantized_momentum=ns.muon_quantized_momentum,
                           muon_scalar_optimizer=ns.muon_scalar_optimizer)
    sched = LRSchedule(lr=ns.lr, min_lr=ns.min_lr, warmup_steps=ns.lr_warmup_iters, decay_steps=ns.lr_decay_iters,
                       style=ns.lr_decay_style)
    tcfg = TrainConfig(micro_batch_size=ns.micro_batch_size, global_batch_size=ns.global_batch_size,
                       seq_length=mcfg.seq_length, dtype="fp32" if ns.fp32 else "bf16",
                       recompute=ns.recompute_granularity or "none", seed=ns.seed, log_interval=ns.log_interval,
                       check_finite=not ns.no_check_for_nan_in_loss_and_grad,
                       precision_recipe=ns.fp8_recipe or "bf16", precision_modules=tuple(ns.fp8_modules),
                       fp8_activations=ns.fp8_activations, fp8_activations_bf16_first=ns.fp8_activations_bf16_first,
                       fp8_activations_bf16_last=ns.fp8_activations_bf16_last, fp8_activations_clamp=ns.fp8_activations_clamp,
                       deterministic=ns.deterministic_mode,
                       optimizer=ocfg, lr_schedule=sched,
                       pipeline_schedule=ns.pipeline_schedule, cuda_graph_scope=tuple(ns.cuda_graph_scope))
    extras = {k: getattr(ns, k) for k in ("train_iters", "data_path", "mock_data", "save", "load", "save_interval",
                                          "log_throughput", "monitor_port", "profile", "profile_step_start",
                                          "profile_step_end", "step_timeout_s", "no_load_optim", "inject_failure_at_iteration")}
    return mcfg, pcfg, tcfg, extras


def parse_args(argv: Optional[Sequence[str]] = None):
    return configs_from_namespace(build_parser().parse_args(argv))


def render_args(mcfg: ModelConfig, pcfg: ParallelConfig, tcfg: TrainConfig, *, train_iters: int = 100,
                data_path: Optional[str] = None, save: Optional[str] = None, load: Optional[str] = None,
                save_interval: int = 0, mock_data: bool = False) -> List[str]:
    """Argument vector that reproduces the given configuration through :func:`parse_args`."""
    plan = mcfg.plan()
    a: List[str] = []

    def kv(flag, val):
        a.extend([flag, str(val)])

    pat = plan.split_for_pipeline(pcfg.pp, pcfg.vpp) if pcfg.pp * pcfg.vpp > 1 else plan.hybrid_pattern
    kv("--hybrid-layer-pattern", pat + "".join("/*-" for _ in range(mcfg.mtp.num_layers)))
    if plan.r_layer_numbers:
        kv("--r-layer-indices", ",".join(map(str, plan.r_layer_numbers)))
    kv("--dsa-a-layer-ranks", ",".join(map(str, mcfg.dsa.attention_ranks)))
    kv("--hidden-size", mcfg.hidden_size)
    kv("--ffn-hidden-size", mcfg.ffn_hidden_size)
    kv("--num-attention-heads", mcfg.mla.num_heads)
    kv("--seq-length", mcfg.seq_length)
    kv("--max-position-embeddings", mcfg.seq_length)
    kv("--vocab-size", mcfg.vocab_size)
    kv("--norm-epsilon", mcfg.norm_eps)
    kv("--init-method-std", mcfg.init_std)
    kv("--rotary-base", mcfg.mla.rope_base)
    if not mcfg.tie_embeddings:
        a.append("--untie-embeddings-and-output-weights")
    m3 = mcfg.mamba3
    kv("--mamba-state-dim", m3.d_state)
    kv("--mamba-head-dim", m3.headdim)
    kv("--mamba-num-groups", m3.ngroups)
    kv("--mamba-expand", m3.expand)
    kv("--mamba3-mimo-rank", m3.mimo_rank)
    kv("--mamba3-chunk-size", m3.chunk_size)
    kv("--mamba3-rope-fraction", m3.rope_fraction)
    kv("--mamba-variant", mcfg.mamba_variant)
    a.append("--multi-latent-attention")
    kv("--q-lora-rank", mcfg.mla.q_lora_rank)
    kv("--kv-lora-rank", mcfg.mla.kv_lora_rank)
    kv("--qk-head-dim", mcfg.mla.qk_head_dim)
    kv("--qk-pos-emb-head-dim", mcfg.mla.qk_pos_emb_head_dim)
    kv("--v-head-dim", mcfg.mla.v_head_dim)
    if mcfg.dsa.attention_ranks:
        kv("--experimental-attention-variant", "dsa")
        kv("--dsa-indexer-n-heads", mcfg.dsa.index_n_heads)
        kv("--dsa-indexer-head-dim", mcfg.dsa.index_head_dim)
        kv("--dsa-indexer-topk", mcfg.dsa.index_topk)
        kv("--dsa-indexer-loss-coeff", mcfg.dsa.indexer_loss_coeff)
        if mcfg.dsa.warmup_dense:
            a.append("--dsa-warmup-dense")
        a.append("--index-cache" if mcfg.dsa.index_cache else "--no-index-cache")
        kv("--index-cache-full-layers", ",".join(map(str, mcfg.dsa.full_layer_ranks)))
    moe = mcfg.moe
    kv("--num-experts", moe.num_experts)
    kv("--moe-router-topk", moe.topk)
    kv("--moe-ffn-hidden-size", moe.expert_ffn)
    kv("--moe-shared-expert-intermediate-size", moe.shared_expert_ffn)
    kv("--moe-token-dispatcher-type", moe.dispatcher)
    if moe.dispatcher == "flex":
        kv("--moe-flex-dispatcher-backend", moe.flex_backend)
    kv("--moe-router-dtype", moe.router_dtype)
    kv("--moe-router-score-function", moe.score_function)
    if moe.expert_bias:
        a.append("--moe-router-enable-expert-bias")
    kv("--moe-aux-loss-coeff", moe.aux_loss_coeff)
    a.extend(["--moe-grouped-gemm", "--moe-router-fusion", "--moe-permute-fusion"])
    kv("--mtp-num-layers", mcfg.mtp.num_layers)
    kv("--mtp-loss-scaling-factor", mcfg.mtp.loss_scaling_factor)
    if mcfg.mtp.fastmtp:
        a.append("--fastmtp")
        kv("--fastmtp-depth", mcfg.mtp.fastmtp_depth)
        kv("--fastmtp-decay", mcfg.mtp.fastmtp_decay)
        kv("--fastmtp-lambda", mcfg.mtp.fastmtp_lambda)
    if not mcfg.mtp.fused_with_main_ce:
        a.append("--no-fuse-main-mtp-ce")
    ng = mcfg.ngram_hash
    a.append("--ngram-hash" if ng.enabled else "--no-ngram-hash")
    if ng.enabled:
        kv("--ngram-hash-orders", ",".join(map(str, ng.orders)))
        kv("--ngram-hash-heads", ng.heads)
        kv("--ngram-hash-table-size", ng.table_size)
        kv("--ngram-hash-embed-dim", ng.embed_dim)
        if ng.offload:
            a.append("--ngram-hash-offload")
    if mcfg.structure.enabled:
        a.append("--structure-embedding")
        kv("--structure-components", mcfg.structure.components)
        kv("--structure-bottleneck-dim", mcfg.structure.bottleneck_dim)
    kv("--tensor-model-parallel-size", pcfg.tp)
    kv("--pipeline-model-parallel-size", pcfg.pp)
    if pcfg.vpp > 1:
        kv("--virtual-pipeline-model-parallel-size", pcfg.vpp)
    kv("--expert-model-parallel-size", pcfg.ep)
    kv("--context-parallel-size", 1)
    if pcfg.sequence_parallel:
        a.append("--sequence-parallel")
    if pcfg.distributed_optimizer:
        a.append("--use-distributed-optimizer")
    if pcfg.overlap_grad_reduce:
        a.append("--overlap-grad-reduce")
    if pcfg.overlap_param_gather:
        a.append("--overlap-param-gather")
    if not pcfg.fused_collectives:
        a.append("--no-fused-collectives")
    kv("--pipeline-schedule", tcfg.pipeline_schedule)
    kv("--micro-batch-size", tcfg.micro_batch_size)
    if tcfg.global_batch_size:
        kv("--global-batch-size", tcfg.global_batch_size)
    kv("--train-iters", train_iters)
    a.append("--fp32" if tcfg.dtype == "fp32" else "--bf16")
    if tcfg.precision_recipe != "bf16":
        kv("--fp8-recipe", tcfg.precision_recipe)
        if tcfg.precision_modules:
            a.extend(["--fp8-modules", *tcfg.precision_modules])
    if tcfg.fp8_activations != "off":
        kv("--fp8-activations", tcfg.fp8_activations)
        kv("--fp8-activations-bf16-first", tcfg.fp8_activations_bf16_first)
        kv("--fp8-activations-bf16-last", tcfg.fp8_activations_bf16_last)
        if tcfg.fp8_activations_clamp:
            a.append("--fp8-activations-clamp")
    if tcfg.deterministic:
        a.append("--deterministic-mode")
    if tcfg.recompute != "none":
        kv("--recompute-granularity", tcfg.recompute)
    if tcfg.cuda_graph_scope:
        a.append("--cuda-graph-scope")
        a.extend(tcfg.cuda_graph_scope)
    kv("--seed", tcfg.seed)
    o = tcfg.optimizer
    kv("--optimizer", o.optimizer)
    kv("--lr", o.lr)
    kv("--min-lr", o.min_lr)
    sched = tcfg.lr_schedule or LRSchedule(lr=o.lr, style="constant")
    kv("--lr-decay-style", sched.style)
    kv("--lr-warmup-iters", sched.warmup_steps)
    kv("--lr-decay-iters", sched.decay_steps)
    kv("--weight-decay", o.weight_decay)
    kv("--adam-beta1", o.beta1)
    kv("--adam-beta2", o.beta2)
    kv("--adam-eps", o.eps)
    kv("--clip-grad", o.clip_grad)
    if o.grad_dtype == "bf16":
        a.append("--grad-reduce-in-bf16")
    if o.optimizer == "muon" and o.muon_scalar_optimizer != "adamw":
        kv("--muon-scalar-optimizer", o.muon_scalar_optimizer)
    if o.optimizer == "muon":
        kv("--muon-momentum", o.muon_momentum)
        if o.muon_quantized_momentum:
            a.append("--muon-quantized-momentum")
    if not tcfg.check_finite:
        a.append("--no-check-for-nan-in-loss-and-grad")
    kv("--log-interval", tcfg.log_interval)
    a.append("--log-throughput")
    if mock_data:
        a.append("--mock-data")
    if data_path:
        kv("--data-path", data_path)
    if save:
        kv("--save", save)
        kv("--save-interval", save_interval)
    if load:
        kv("--load", load)
    return a


__all__ = ["build_parser", "parse_args", "render_args", "configs_from_namespace"]
_ = (DSAConfig, MLAConfig, Mamba3Config, MoEConfig, MTPConfig, NgramHashConfig, StructureConfig)
