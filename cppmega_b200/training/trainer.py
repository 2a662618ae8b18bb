"""Training loop: micro-batch accumulation, pipeline schedule, optimizer step, logging.

The reference delegates all of this to Megatron's ``pretrain`` (scripts/remote_smoke_h200_dsa_9_4_m.sh:691-740);
here it is a small explicit loop.  The batch / loss contract matches the schedules of the
reference: a batch carries ``tokens, labels, loss_mask`` and the loss function returns
``(sum(loss*mask), num_tokens)`` (cppmega/megatron/hybrid_schedule_plan.py:403-452).

Public entry points: :class:`Trainer` (``train_step(batch)``, ``fit(iterator, steps)``) and
:func:`synthetic_batches`.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional

import torch
import torch.distributed as dist

from ..config.model import ModelConfig
from ..models.nam56r import NAM56RModel, build_model
from ..parallel import state as pstate
from ..parallel.dist_optimizer import DistributedOptimizer, OptimizerConfig
from ..parallel.state import ParallelConfig, ParallelContext
from ..parallel.tensor_parallel import allreduce_sequence_parallel_grads
from .lr import LRSchedule


@dataclass
class TrainConfig:
    micro_batch_size: int = 4
    global_batch_size: Optional[int] = None      # default: micro_batch_size * dp
    seq_length: int = 4096
    dtype: str = "bf16"                          # bf16 | fp32
    recompute: str = "none"                      # none | selective | full
    recompute_keep_last: int = 0                 # the last K layers of a stage are not recomputed (spend spare memory)
    seed: int = 1234
    log_interval: int = 1
    check_finite: bool = True
    precision_recipe: str = "bf16"               # bf16 | mxfp8 (E8M0 1x32 block scales) | tensorwise (one scale per tensor)
    precision_modules: tuple = ()                # glob patterns of module names that run under precision_recipe; the rest
                                                 # stays bf16.  Empty: every eligible linear.  Shorthands: "moe", "mamba_proj"
    fp8_activations: str = "off"                 # off | mxfp8 | tensor: FP8-compress the activations saved for backward
    fp8_activations_bf16_first: int = 1          # layers at the start / end of the stack whose saved tensors stay bf16
    fp8_activations_bf16_last: int = 1
    fp8_activations_clamp: bool = False          # "tensor" recipe: limit the measured maximum to the E4M3 range
    deterministic: bool = False                  # debugging: atomic-reduction kernels -> PyTorch definitions, library deterministic mode
    cuda_graph_scope: tuple = ()                 # subset of ("mamba", "attn", "mlp"): layers captured as CUDA graphs
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    lr_schedule: Optional[LRSchedule] = None
    update_router_bias: bool = True
    pipeline_schedule: str = "1f1b"              # 1f1b | interleaved | dualpipev

    def torch_dtype(self) -> torch.dtype:
        return {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[self.dtype]


class NonFiniteLossError(RuntimeError):
    pass


PRECISION_MODULE_SETS = {
    # FP8 on the MoE layers only (cppmega/megatron/selective_fp8_moe_patch.py:60-149)
    "moe": ("*.mlp.experts", "*.mlp.shared_experts", "*.mlp.shared_experts.*", "*.mlp"),
    # FP8 on the Mamba in / out projections only (configs/te_precision/mamba_mxfp8_eval_bf16.yaml:1-29)
    "mamba_proj": ("*.mixer.in_proj", "*.mixer.out_proj"),
}


def _install_precision(model, cfg: "TrainConfig"):
    """Global recipe, or - with ``precision_modules`` - the recipe on the named modules and bf16 elsewhere."""
    from ..ops import functional as F_
    if cfg.precision_recipe not in F_.RECIPES:
        raise ValueError(f"unknown precision recipe {cfg.precision_recipe!r}; known: {F_.RECIPES}")
    if not cfg.precision_modules or cfg.precision_recipe == "bf16":
        F_.set_precision_recipe(cfg.precision_recipe)
        return []
    pats = []
    for p in cfg.precision_modules:
        pats.extend(PRECISION_MODULE_SETS.get(p, (p,)))
    if "moe" in cfg.precision_modules:                      # "*.mlp" must only hit MoE layers, not dense MLPs
        moe_names = {n for n, m in model.named_modules() if type(m).__name__ == "MoELayer"}
        pats = [p for p in pats if p != "*.mlp"] + sorted(moe_names)
    _handles, matched = F_.install_precision_rules(model, [(p, cfg.precision_recipe) for p in pats], default="bf16")
    if not matched:
        raise ValueError(f"precision_modules {cfg.precision_modules} match no module of the model")
    return matched


class Trainer:
    def __init__(self, model_cfg: ModelConfig, train_cfg: TrainConfig,
                 pc: Optional[ParallelContext] = None, device: Optional[torch.device] = None,
                 model: Optional[NAM56RModel] = None):
        self.model_cfg, self.cfg = model_cfg, train_cfg
        self.pc = pc or pstate.get_context()
        if device is None:
            device = (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                      else torch.device("cpu"))
        self.device = device
        self.chunked = (model is None and self.pc.pp > 1 and train_cfg.pipeline_schedule in ("interleaved", "dualpipev")
                        and (train_cfg.pipeline_schedule == "dualpipev" or self.pc.config.vpp > 1))
        if self.chunked:
            from ..parallel.pipeline import build_chunked_model
            self.model = build_chunked_model(model_cfg, self.pc, train_cfg.pipeline_schedule, dtype=train_cfg.torch_dtype(),
                                             seed=train_cfg.seed, recompute=train_cfg.recompute, device=device)
        else:
            self.model = model or build_model(model_cfg, self.pc, dtype=train_cfg.torch_dtype(), seed=train_cfg.seed,
                                              recompute=train_cfg.recompute, device=device,
                                              recompute_keep_last=train_cfg.recompute_keep_last)
        # with pipeline stages the embedding copies are summed before the data-parallel reduction,
        # so the reduction cannot start from inside backward
        from ..ops import functional as F_
        if train_cfg.deterministic:
            F_.set_deterministic(True)
        self.precision_modules = _install_precision(self.model, train_cfg)
        if train_cfg.fp8_activations not in ("off", "", None):
            act = {"recipe": train_cfg.fp8_activations, "bf16_first": train_cfg.fp8_activations_bf16_first,
                   "bf16_last": train_cfg.fp8_activations_bf16_last, "clamp": train_cfg.fp8_activations_clamp}
            for m in (self.model.chunks if self.chunked else [self.model]):
                m.fp8_activations = act
        self.fused = {"optimizer": False, "moe": False}
        opt_cls = DistributedOptimizer
        if device.type == "cuda" and self.pc.world_size > 1 and train_cfg.optimizer.optimizer == "adamw":
            from ..parallel.fused_optimizer import FusedDistributedOptimizer, fused_optimizer_supported
            if fused_optimizer_supported(self.pc, device) and self.pc.pp == 1:
                opt_cls = FusedDistributedOptimizer
                self.fused["optimizer"] = True
        self.optimizer = opt_cls(self.model, train_cfg.optimizer, self.pc,
                                 overlap=False if self.pc.pp > 1 else None)
        if self.pc.world_size > 1 and device.type == "cuda" and self.pc.config.fused_collectives:
            self._attach_fused_paths()
        if (device.type == "cuda" and self.pc.ep == 1 and self.pc.tp == 1 and self.pc.config.fused_collectives
                and train_cfg.torch_dtype() == torch.bfloat16 and model_cfg.hidden_size % 8 == 0):
            from ..parallel import fused_moe          # permute-fused MoE kernels on local buffers
            self._moe_bufs = fused_moe.attach(self.model, self.pc, device, tokens_per_rank=0)
            self.fused["moe"] = self._moe_bufs is not None
        self.graphed_layers = 0
        if train_cfg.cuda_graph_scope and device.type == "cuda" and not self.chunked and self.pc.tp == 1:
            from ..utils.cuda_graphs import capture_model_layers
            shape = (train_cfg.micro_batch_size, train_cfg.seq_length, model_cfg.hidden_size)
            self.graphed_layers = capture_model_layers(self.model, train_cfg.cuda_graph_scope, shape, train_cfg.torch_dtype(), device)
        self.lr_schedule = train_cfg.lr_schedule or LRSchedule(lr=train_cfg.optimizer.lr, style="constant")
        self.step = 0
        dp = self.pc.dp
        gbs = train_cfg.global_batch_size or train_cfg.micro_batch_size * dp
        if gbs % (train_cfg.micro_batch_size * dp):
            raise ValueError(f"global batch {gbs} not divisible by micro_batch*dp={train_cfg.micro_batch_size * dp}")
        self.global_batch_size = gbs
        self.num_microbatches = gbs // (train_cfg.micro_batch_size * dp)
        self._sp_params = [p for p in self.model.parameters() if getattr(p, "sequence_parallel_grad", False)]
        self.history: List[Dict[str, float]] = []
        self.tokens_seen = 0
        self.watchdog = None

    def describe_paths(self) -> Dict[str, str]:
        """Which of the optional fast paths this run takes, and for those it does not, why: ``{"optimizer": "on", "moe":
        "off: pipeline stages > 1", ...}``.  Printed once at start-up by ``pretrain``."""
        pc, cfg, dev = self.pc, self.cfg, self.device
        bf16 = cfg.torch_dtype() == torch.bfloat16

        def first(*checks):
            for bad, why in checks:
                if bad:
                    return "off: " + why
            return "on"

        peers = True
        if dev.type == "cuda" and pc.world_size > 1:
            from ..parallel.symm_mem import peer_access_available
            peers = peer_access_available(pc)
        common = ((dev.type != "cuda", "no GPU"), (not pc.config.fused_collectives, "fused collectives disabled"),
                  (not peers, "no peer access between the GPUs of the group"))
        out = {
            "optimizer": "on" if self.fused.get("optimizer") else first(
                *common, (pc.world_size == 1, "single process"), (cfg.optimizer.optimizer != "adamw", "optimizer is not adamw"),
                (pc.pp > 1, "pipeline stages > 1"), (not pc.config.distributed_optimizer, "distributed optimizer off"),
                (pc.dp == 1, "data-parallel size 1"), (True, "not selected")),
            "moe": "on" if self.fused.get("moe") else first(
                *common, (not bf16, "dtype is not bf16"), (not self.model.moe_layers() if hasattr(self.model, "moe_layers") else True, "no MoE layers"),
                (pc.ep == 1 and pc.tp > 1, "EP 1 with TP > 1"), (True, "not selected")),
            "tp": "on" if self.fused.get("tp") else first(
                (pc.tp == 1, "tensor-parallel size 1"), *common, (not pc.sequence_parallel, "sequence parallelism off"),
                (not bf16, "dtype is not bf16"), (True, "not selected")),
            "cuda_graphs": f"on ({self.graphed_layers} layers)" if self.graphed_layers else first(
                (not cfg.cuda_graph_scope, "no --cuda-graph-scope"), (dev.type != "cuda", "no GPU"), (self.chunked, "chunked pipeline"),
                (pc.tp > 1, "TP > 1"), (True, "no layer of the requested kinds")),
            "precision": cfg.precision_recipe + (f" on {len(self.precision_modules)} modules" if self.precision_modules else ""),
            "fp8_activations": cfg.fp8_activations,
            "recompute": cfg.recompute + (f" (last {cfg.recompute_keep_last} layers kept)" if cfg.recompute_keep_last else ""),
        }
        return out

    def _attach_fused_paths(self):
        """Swap the NCCL collectives for the peer-memory kernels where the topology allows it."""
        from ..parallel.symm_mem import peer_access_available
        pc = self.pc
        if not peer_access_available(pc):
            return
        if pc.tp > 1 and pc.sequence_parallel and self.cfg.torch_dtype() == torch.bfloat16:
            from ..parallel import fused_tp
            from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
            width = self.model_cfg.hidden_size
            for m in self.model.modules():
                if isinstance(m, (ColumnParallelLinear, RowParallelLinear)):
                    width = max(width, m.weight.shape[0], m.weight.shape[1])
            rows = self.cfg.micro_batch_size * (self.cfg.seq_length // pc.tp)
            self._tp_bufs = fused_tp.install(pc, self.device, rows, width)
            self.fused["tp"] = self._tp_bufs is not None
        if pc.ep > 1 and self.cfg.torch_dtype() == torch.bfloat16:
            from ..parallel import fused_moe
            # under sequence parallelism every TP rank routes its own sequence shard through the experts of its EP group;
            # the shared expert's TP GEMMs then stay on the main stream (one TP transfer in flight at a time)
            seq_local = self.cfg.seq_length // pc.tp if pc.sequence_parallel else self.cfg.seq_length
            bufs = fused_moe.attach(self.model, pc, self.device,
                                    tokens_per_rank=self.cfg.micro_batch_size * seq_local,
                                    per_layer=self.cfg.recompute != "full" or self.cfg.recompute_keep_last > 0,
                                    overlap_shared_expert=pc.tp == 1)
            self.fused["moe"] = bufs is not None
            self._moe_bufs = bufs

    def close(self) -> None:
        """Release the peer-mapped heaps (every rank of the group must call this in the same phase)."""
        opt_close = getattr(self.optimizer, "close", None)
        if opt_close is not None:
            opt_close()
        for name in ("_moe_bufs", "_tp_bufs"):
            bufs = getattr(self, name, None)
            heap = getattr(bufs, "heap", None)
            if heap is not None and hasattr(heap, "close"):
                heap.close()
            setattr(self, name, None)

    # ---- one optimizer step ------------------------------------------------
    def _to_device(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}

    def forward_backward(self, microbatches: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        pc = self.pc
        if pc.pp > 1:
            if self.chunked:
                from ..parallel.pipeline import run_chunked_schedule
                return run_chunked_schedule(self, microbatches)
            from ..parallel.pipeline import run_pipeline_schedule
            return run_pipeline_schedule(self, microbatches)
        n = len(microbatches)
        tot_loss = None
        tot_lm = None
        mtp: Optional[List[torch.Tensor]] = None
        for i, mb in enumerate(microbatches):
            mb = self._to_device(mb)
            self.optimizer.set_microbatch(is_last=(i == n - 1), grad_scale=1.0)
            out = self.model(mb["input_ids"], mb["labels"], mb.get("loss_mask"),
                             structure_inputs=mb.get("structure_inputs"))
            (out["loss"] / n).backward()
            l = out["loss"].detach()
            tot_loss = l if tot_loss is None else tot_loss + l
            tot_lm = out["lm_loss"] if tot_lm is None else tot_lm + out["lm_loss"]
            if out["mtp_losses"]:
                mtp = out["mtp_losses"] if mtp is None else [a + b for a, b in zip(mtp, out["mtp_losses"])]
        res = {"loss": tot_loss / n, "lm_loss": tot_lm / n}
        if mtp is not None:
            res["mtp_losses"] = [m / n for m in mtp]
        return res

    def train_step(self, batch) -> Dict[str, torch.Tensor]:
        """``batch``: one dict (split into micro-batches along dim 0) or a list of micro-batch
        dicts.  Tensors may live in pinned host memory; they are copied to the device here.
        Returns device scalars (no host sync) - call ``.item()`` on what you need."""
        cfg = self.cfg
        mbs = batch if isinstance(batch, list) else self._split(batch)
        self.optimizer.zero_grad()
        res = self.forward_backward(mbs)
        if self._sp_params and self.pc.sequence_parallel and not getattr(self.optimizer, "handles_sequence_parallel_grads", False):
            self.optimizer.finish_grad_sync()      # sums commute: TP all-reduce after the DP reduction
            allreduce_sequence_parallel_grads_main(self._sp_params, self.pc)
        lr = self.lr_schedule(self.step)
        stats = self.optimizer.step(lr)
        if cfg.update_router_bias:
            self.model.update_router_biases()
        self.step += 1
        self.tokens_seen += self.global_batch_size * cfg.seq_length
        res.update(stats)
        res["lr"] = lr
        if self.watchdog is not None:
            self.watchdog.beat(self.step)
        return res

    def _split(self, batch: Dict[str, torch.Tensor]) -> List[Dict[str, torch.Tensor]]:
        n = self.num_microbatches
        if n == 1:
            return [batch]
        out = []
        for i in range(n):
            out.append({k: (v.chunk(n, dim=0)[i] if torch.is_tensor(v) else v) for k, v in batch.items()})
        return out

    def reduce_loss_for_logging(self, res: Dict[str, torch.Tensor]) -> Dict[str, float]:
        """Average the reported losses over data-parallel ranks (one small all-reduce) and
        move them to the host; raises on NaN/Inf when ``check_finite``."""
        pc = self.pc
        keys = ["loss", "lm_loss"]
        vals = [res["loss"].float(), res["lm_loss"].float()]
        for i, m in enumerate(res.get("mtp_losses", [])):
            keys.append(f"mtp_{i + 1}_loss")
            vals.append(m.float())
        keys.append("grad_norm")
        vals.append(res["grad_norm"].float())
        t = torch.stack([v.reshape(()) for v in vals])
        if pc.dp > 1:
            gn = t[-1].clone()
            dist.all_reduce(t, group=pc.dp_group)
            t /= pc.dp
            t[-1] = gn
        host = t.tolist()
        out = dict(zip(keys, host))
        if self.cfg.check_finite and not all(math.isfinite(v) for v in host):
            raise NonFiniteLossError(f"non-finite training statistics at step {self.step}: {out}")
        return out

    # ---- loop ---------------------------------------------------------------
    def fit(self, batches: Iterator, steps: int, log=None) -> List[Dict[str, float]]:
        cfg = self.cfg
        flops_tok = self.model_cfg.flops_per_token(cfg.seq_length)
        t_last = time.perf_counter()
        for _ in range(steps):
            res = self.train_step(next(batches))
            if cfg.log_interval and self.step % cfg.log_interval == 0:
                rec = self.reduce_loss_for_logging(res)
                if self.device.type == "cuda":
                    from ..ops import cuda as cu
                    cu.check_errors(self.device)      # raises if a kernel's bounded wait ran out since the last check
                now = time.perf_counter()
                dt = (now - t_last) / cfg.log_interval
                t_last = now
                toks = self.global_batch_size * cfg.seq_length
                rec.update(step=self.step, lr=res["lr"], step_ms=dt * 1e3, tokens_per_s=toks / dt,
                           tflops_per_gpu=flops_tok * toks / dt / 1e12 / max(self.pc.world_size, 1))
                self.history.append(rec)
                if log is not None and self.pc.rank == 0:
                    log(rec)
        return self.history


def allreduce_sequence_parallel_grads_main(params, pc: ParallelContext) -> None:
    """Same as :func:`allreduce_sequence_parallel_grads` but on ``main_grad`` buffers."""
    if pc.tp == 1 or not pc.sequence_parallel:
        return
    for p in params:
        g = getattr(p, "main_grad", None)
        if g is not None:
            dist.all_reduce(g, group=pc.tp_group)


def synthetic_batches(vocab: int, micro_batch: int, seq: int, num_microbatches: int = 1, seed: int = 0,
                      pin: bool = True, rank: int = 0, skip: int = 0) -> Iterator[List[Dict[str, torch.Tensor]]]:
    """Endless stream of uniform-random token batches in (pinned) host memory; labels are
    the next token.  ``skip`` steps are generated and dropped first (resume)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed + 7919 * rank)
    pin = pin and torch.cuda.is_available()
    for _ in range(skip * num_microbatches):
        torch.randint(0, vocab, (micro_batch, seq + 1), generator=gen, dtype=torch.long)
    while True:
        mbs = []
        for _ in range(num_microbatches):
            tok = torch.randint(0, vocab, (micro_batch, seq + 1), generator=gen, dtype=torch.long)
            ids, lab = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
            if pin:
                ids, lab = ids.pin_memory(), lab.pin_memory()
            mbs.append({"input_ids": ids, "labels": lab})
        yield mbs


_ = (ParallelConfig, allreduce_sequence_parallel_grads)
