"""Flat gradient/parameter buffers, bucketed gradient reduction and the ZeRO-1
distributed optimizer.

What the reference gets from Megatron (``--use-distributed-optimizer --overlap-grad-reduce
--overlap-param-gather``; scripts/remote_smoke_h200_dsa_9_4_m.sh:700,
cppmega/recipes/nam56r_nemo_recipe.py:236-240) is owned here:

* parameters of one reduction domain (dense -> data-parallel group, experts ->
  expert-data-parallel group) live in one contiguous buffer per dtype; gradients
  accumulate into a matching buffer (``main_grad``), fp32 or bf16;
* the buffer is cut into buckets; when every gradient of a bucket has been produced the
  bucket is reduce-scattered (distributed optimizer) or all-reduced, asynchronously
  when ``overlap_grad_reduce`` is set;
* each rank owns a 1/dp slice of every bucket: fp32 master weights and the optimizer
  state exist for that slice only; after the update the new low-precision slice is
  all-gathered back into the parameter buffer.

On CPU (gloo) reduce-scatter is emulated by all-reduce + slice.  On GPUs with peer
access the reduce-scatter + update is replaced by the fused kernel in
:mod:`cppmega_b200.parallel.fused_optimizer`; this file is the plain-collective baseline.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


@dataclass
class OptimizerConfig:
    optimizer: str = "adamw"           # adamw | adam8bit | muon
    lr: float = 1e-4
    min_lr: float = 0.0
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    clip_grad: float = 1.0
    grad_dtype: str = "fp32"           # fp32 | bf16 accumulation / reduction dtype
    bucket_mb: int = 256
    muon_momentum: float = 0.95
    muon_ns_steps: int = 5
    muon_quantized_momentum: bool = False
    muon_scalar_optimizer: str = "adamw"   # adamw | adam8bit: optimizer of the parameters Muon does not take
    loss_scale: float = 1.0


def _pad_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class Bucket:
    def __init__(self, index: int, start: int, end: int):
        self.index, self.start, self.end = index, start, end
        self.params: List[nn.Parameter] = []
        self.pending = 0
        self.reduced = False
        self.handle = None


class ParamGroupBuffer:
    """One reduction domain x dtype: contiguous params, grads, buckets, shard bookkeeping."""

    def __init__(self, params: List[nn.Parameter], group, group_size: int, group_rank: int,
                 grad_dtype: torch.dtype, bucket_bytes: int, distributed: bool, is_expert: bool = False,
                 alloc: Optional[Callable] = None):
        self.params = params
        self.is_expert = is_expert
        self.group, self.n, self.rank = group, group_size, group_rank
        self.distributed = distributed
        dev, dtype = params[0].device, params[0].dtype
        self.dtype = dtype
        align = 128 * self.n                       # every bucket divides evenly and stays 256B aligned
        offsets, pos = [], 0
        bucket_elems = max(bucket_bytes // max(dtype.itemsize, 1), 1)
        self.buckets: List[Bucket] = []
        cur_start = 0
        cur_params: List[Tuple[nn.Parameter, int]] = []
        for p in params:
            pos = _pad_to(pos, 64)
            offsets.append(pos)
            cur_params.append((p, pos))
            pos += p.numel()
            if pos - cur_start >= bucket_elems:
                pos = _pad_to(pos, align)
                b = Bucket(len(self.buckets), cur_start, pos)
                b.params = [q for q, _ in cur_params]
                self.buckets.append(b)
                cur_start, cur_params = pos, []
        if cur_params:
            pos = _pad_to(pos, align)
            b = Bucket(len(self.buckets), cur_start, pos)
            b.params = [q for q, _ in cur_params]
            self.buckets.append(b)
        self.numel = pos
        if alloc is not None:          # e.g. peer-mapped symmetric memory
            self.param_buffer = alloc(self, self.numel, dtype)
            self.grad_buffer = alloc(self, self.numel, grad_dtype)
        else:
            self.param_buffer = torch.zeros(self.numel, dtype=dtype, device=dev)
            self.grad_buffer = torch.zeros(self.numel, dtype=grad_dtype, device=dev)
        self.offsets: Dict[nn.Parameter, int] = {}
        self.bucket_of: Dict[nn.Parameter, Bucket] = {}
        for b in self.buckets:
            for p in b.params:
                self.bucket_of[p] = b
        for p, off in zip(params, offsets):
            self.offsets[p] = off
            view = self.param_buffer[off:off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad_buffer[off:off + p.numel()].view(p.shape)

    # shard of bucket b owned by this rank, as (start, end) into the flat buffer
    def shard_range(self, b: Bucket) -> Tuple[int, int]:
        if not self.distributed or self.n == 1:
            return b.start, b.end
        per = (b.end - b.start) // self.n
        return b.start + self.rank * per, b.start + (self.rank + 1) * per

    def zero_grad(self):
        self.grad_buffer.zero_()
        for b in self.buckets:
            b.pending = len(b.params)
            b.reduced = False
            b.handle = None

    def reduce_bucket(self, b: Bucket, async_op: bool, scale: float):
        b.reduced = True
        g = self.grad_buffer[b.start:b.end]
        if scale != 1.0:
            g.mul_(scale)
        if self.n == 1:
            return
        if self.distributed and g.device.type != "cpu":
            lo, hi = self.shard_range(b)
            b.handle = dist.reduce_scatter_tensor(self.grad_buffer[lo:hi], g, group=self.group, async_op=async_op)
        else:
            b.handle = dist.all_reduce(g, group=self.group, async_op=async_op)
        if not async_op:
            b.handle = None

    def finish(self):
        for b in self.buckets:
            if b.handle is not None:
                b.handle.wait()
                b.handle = None

    def gather_params(self):
        if not self.distributed or self.n == 1:
            return
        for b in self.buckets:
            lo, hi = self.shard_range(b)
            full = self.param_buffer[b.start:b.end]
            if full.device.type == "cpu":
                parts = [torch.empty(hi - lo, dtype=full.dtype) for _ in range(self.n)]
                dist.all_gather(parts, self.param_buffer[lo:hi].clone(), group=self.group)
                full.copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(full, self.param_buffer[lo:hi], group=self.group)


def _muon_eligible(p) -> bool:
    """Matrices (and stacks of expert matrices) other than the embedding / output layer."""
    return p.dim() in (2, 3) and not getattr(p, "is_embedding_or_output_parameter", False)


def _bucket_has_cut_matrix(buf: "ParamGroupBuffer", b: Bucket) -> bool:
    """True when some Muon matrix of bucket ``b`` is split between two ranks' shards.  Depends only on the bucket
    layout, so every rank of the reduction group gets the same answer."""
    if not buf.distributed or buf.n == 1:
        return False
    per = (b.end - b.start) // buf.n
    for p in b.params:
        if not _muon_eligible(p):
            continue
        off = buf.offsets[p]
        mats = p.shape[0] if p.dim() == 3 else 1
        sz = p.numel() // mats
        for i in range(mats):
            a, e = off + i * sz - b.start, off + (i + 1) * sz - 1 - b.start
            if a // per != e // per:
                return True
    return False


class DistributedOptimizer:
    """AdamW (and Muon for matrices) over sharded fp32 master weights."""

    def __init__(self, model: nn.Module, cfg: OptimizerConfig, pc, *, distributed: Optional[bool] = None,
                 overlap: Optional[bool] = None):
        self.cfg, self.pc, self.model = cfg, pc, model
        self.distributed = pc.config.distributed_optimizer if distributed is None else distributed
        self.overlap = pc.config.overlap_grad_reduce if overlap is None else overlap
        gd = torch.float32 if cfg.grad_dtype == "fp32" else torch.bfloat16
        dense: Dict[torch.dtype, List[nn.Parameter]] = {}
        expert: Dict[torch.dtype, List[nn.Parameter]] = {}
        for p in model.parameters():
            if not p.requires_grad:
                continue
            (expert if getattr(p, "is_expert", False) else dense).setdefault(p.dtype, []).append(p)
        self.buffers: List[ParamGroupBuffer] = []
        bb = cfg.bucket_mb << 20
        for dt, ps in dense.items():
            g = gd if dt != torch.float32 else torch.float32
            self.buffers.append(ParamGroupBuffer(ps, pc.dp_group, pc.dp, pc.dp_rank, g, bb, self.distributed,
                                                 alloc=self._buffer_allocator(False, ps, g)))
        for dt, ps in expert.items():
            g = gd if dt != torch.float32 else torch.float32
            self.buffers.append(ParamGroupBuffer(ps, pc.edp_group, pc.edp, pc.edp_rank, g, bb, self.distributed,
                                                 is_expert=True, alloc=self._buffer_allocator(True, ps, g)))
        # the loss is a mean over each rank's tokens, so every gradient (expert ones included, whose
        # reduction group is only the expert-data-parallel ranks) is the sum over ranks / dp
        for _buf in self.buffers:
            _buf.grad_div = float(pc.dp)
        self.step_count = 0
        self.lr = cfg.lr
        self._hooks = []
        self._grad_scale = 1.0
        self._build_state()
        self._install_hooks()
        self.zero_grad()
        self.fused_step: Optional[Callable] = None       # set by parallel.fused_optimizer.attach()

    def _scalar_8bit(self) -> bool:
        """8-bit AdamW state: for every parameter (``optimizer == "adam8bit"``) or for what Muon leaves over."""
        c = self.cfg
        return c.optimizer == "adam8bit" or (c.optimizer == "muon" and c.muon_scalar_optimizer == "adam8bit")

    def _buffer_allocator(self, is_expert: bool, params, grad_dtype) -> Optional[Callable]:
        """Hook for subclasses that place the flat buffers in special memory."""
        return None

    # ---- state ------------------------------------------------------------
    def _build_state(self):
        self.state = []
        for buf in self.buffers:
            for b in buf.buckets:
                lo, hi = buf.shard_range(b)
                master = buf.param_buffer[lo:hi].float().clone()
                wd_mask = torch.zeros(hi - lo, dtype=torch.bool, device=master.device)
                muon_segments, muon_cross = [], []
                for p in b.params:
                    off = buf.offsets[p]
                    s, e = max(off, lo), min(off + p.numel(), hi)
                    if s >= e:
                        continue
                    decay = p.dim() >= 2 and not getattr(p, "no_weight_decay", False)
                    if decay:
                        wd_mask[s - lo:e - lo] = True
                    if self.cfg.optimizer == "muon" and _muon_eligible(p):
                        # a 3-D expert stack is E separate matrices; each matrix is one Muon unit
                        mats = p.shape[0] if p.dim() == 3 else 1
                        shape = tuple(p.shape[-2:])
                        per = p.numel() // mats
                        for i in range(mats):
                            ms, me = off + i * per, off + (i + 1) * per
                            if me <= lo or ms >= hi:
                                continue
                            if ms >= lo and me <= hi:
                                muon_segments.append((ms - lo, me - lo, shape))
                            else:     # cut by a shard boundary: this rank holds [cs, ce) of the matrix
                                cs, ce = max(ms, lo), min(me, hi)
                                muon_cross.append({"local": (cs - lo, ce - lo), "bucket": (ms - b.start, me - b.start),
                                                   "inner": (cs - ms, ce - ms), "shape": shape})
                use8 = self._scalar_8bit()
                need_m = not use8 or ((muon_segments or muon_cross) and
                                      (muon_cross or not self.cfg.muon_quantized_momentum))
                a8 = None
                if use8:
                    from ..optim.adam8bit import Adam8bitState
                    a8 = Adam8bitState.zeros(hi - lo, master.device)
                self.state.append({
                    "buf": buf, "bucket": b, "lo": lo, "hi": hi, "master": master,
                    "m": torch.zeros_like(master) if need_m else None, "v": None if use8 else torch.zeros_like(master),
                    "a8": a8,
                    "wd_mask": wd_mask, "muon": muon_segments, "muon_cross": muon_cross,
                    "muon_gather": self.cfg.optimizer == "muon" and _bucket_has_cut_matrix(buf, b),
                })

    def close(self) -> None:
        """Detach from the parameters: the gradient hooks live in the tensors' autograd metadata, where the cycle
        parameter -> hook -> optimizer -> flat buffer -> parameter is invisible to the garbage collector, so a dropped
        optimizer (and the model with it) would otherwise stay allocated."""
        for h in self._hooks:
            h.remove()
        self._hooks = []
        for buf in getattr(self, "buffers", []):
            for p in buf.params:
                for name in ("main_grad", "grad_added_to_main_grad"):
                    if hasattr(p, name):
                        try:
                            delattr(p, name)
                        except AttributeError:
                            pass

    def _install_hooks(self):
        for buf in self.buffers:
            for p in buf.params:
                def hook(param, buf=buf):
                    if getattr(param, "grad_added_to_main_grad", False):
                        param.grad_added_to_main_grad = False      # the wgrad GEMM accumulated in place
                        param.grad = None
                    elif param.grad is not None:
                        param.main_grad.add_(param.grad.view_as(param.main_grad))
                        param.grad = None
                    if not self._last_microbatch:
                        return
                    b = buf.bucket_of[param]
                    b.pending -= 1
                    if b.pending == 0 and not b.reduced:
                        self._on_bucket_ready(buf, b)
                self._hooks.append(p.register_post_accumulate_grad_hook(hook))
                # GEMM epilogues may add weight gradients directly into the flat buffer (CUDA, 2-D/3-D bf16 weights)
                p.fuse_wgrad_accumulation = bool(p.is_cuda and p.dim() >= 2 and p.dtype == torch.bfloat16)
        self._last_microbatch = True

    def _on_bucket_ready(self, buf: ParamGroupBuffer, b: Bucket) -> None:
        """Called from inside backward (last micro-batch) when every gradient of bucket ``b`` has been produced: with
        ``overlap_grad_reduce`` the bucket's reduction starts now, under the rest of the backward pass."""
        if self.overlap:
            buf.reduce_bucket(b, async_op=True, scale=self._grad_scale / buf.grad_div)

    def set_microbatch(self, is_last: bool, grad_scale: float = 1.0):
        """Call before each backward: gradient reduction only fires on the last micro-batch."""
        self._last_microbatch = is_last
        self._grad_scale = grad_scale
        if not is_last:
            return
        for buf in self.buffers:
            for b in buf.buckets:
                b.pending = len(b.params)
                b.reduced = False

    def zero_grad(self):
        for buf in self.buffers:
            buf.zero_grad()

    # ---- step -------------------------------------------------------------
    def finish_grad_sync(self):
        for buf in self.buffers:
            for b in buf.buckets:
                if not b.reduced:      # no overlap, or a bucket holding parameters that got no gradient
                    buf.reduce_bucket(b, async_op=False, scale=self._grad_scale / buf.grad_div)
            buf.finish()

    def _shard_grads(self):
        for st in self.state:
            yield st, st["buf"].grad_buffer[st["lo"]:st["hi"]]

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm over all shards.  Replicated copies across TP are counted once."""
        pc = self.pc
        dev = self.state[0]["master"].device if self.state else torch.device("cpu")
        total = torch.zeros((), dtype=torch.float32, device=dev)
        dense_sq = torch.zeros_like(total)
        expert_sq = torch.zeros_like(total)
        for st, g in self._shard_grads():
            sq = self._sumsq_tp_aware(st, g)
            if st["buf"].is_expert:
                expert_sq += sq
            else:
                dense_sq += sq
        if dist.is_initialized() and pc.world_size > 1:
            if self.distributed and pc.dp > 1:
                dist.all_reduce(dense_sq, group=pc.dp_group)
            if pc.ep > 1 or (self.distributed and pc.edp > 1):
                # experts: sum over the whole data-parallel group (distinct experts on EP
                # ranks; shards on EDP ranks when the optimizer is distributed)
                if not self.distributed and pc.edp > 1:
                    expert_sq = expert_sq / pc.edp
                dist.all_reduce(expert_sq, group=pc.dp_group)
            total = dense_sq + expert_sq
            if pc.tp > 1:
                dist.all_reduce(total, group=pc.tp_group)
            if pc.pp > 1:
                dist.all_reduce(total, group=pc.pp_group)
        else:
            total = dense_sq + expert_sq
        return total.sqrt()

    def _sumsq_tp_aware(self, st, g) -> torch.Tensor:
        """Sum of squares of a shard; tensors replicated over TP contribute 1/tp so the later
        TP all-reduce counts them once."""
        tp = self.pc.tp
        if tp == 1 and g.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous():
            from ..ops import cuda as cu           # one pass over the shard, no fp32 copy
            out = torch.zeros((), dtype=torch.float32, device=g.device)
            cu.sumsq(g, out)
            return out
        gf = g.float()
        if tp == 1:
            return (gf * gf).sum()
        buf, lo, hi = st["buf"], st["lo"], st["hi"]
        tot = torch.zeros((), dtype=torch.float32, device=g.device)
        for p in st["bucket"].params:
            off = buf.offsets[p]
            s, e = max(off, lo), min(off + p.numel(), hi)
            if s >= e:
                continue
            seg = gf[s - lo:e - lo]
            w = 1.0 if getattr(p, "tensor_model_parallel", False) else 1.0 / tp
            tot += w * (seg * seg).sum()
        return tot

    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> Dict[str, float]:
        cfg = self.cfg
        lr = self.lr if lr is None else lr
        self.finish_grad_sync()
        gnorm = self.grad_norm()
        clip = torch.ones_like(gnorm)
        if cfg.clip_grad > 0:
            clip = torch.clamp(cfg.clip_grad / (gnorm + 1e-6), max=1.0)
        self.step_count += 1
        t = self.step_count
        bc1 = 1.0 - cfg.beta1 ** t
        bc2 = 1.0 - cfg.beta2 ** t
        from ..optim import adamw as adamw_ops
        for st, g in self._shard_grads():
            buf = st["buf"]
            out = buf.param_buffer[st["lo"]:st["hi"]]
            skip = st["muon"]
            if st["muon"] or st["muon_gather"]:
                from ..optim import muon as muon_ops
                muon_ops.muon_update_segments(st, g, clip, lr, cfg)
                if st["muon_gather"]:          # same decision on every rank of the group: the gather is a collective
                    muon_ops.muon_update_cut_matrices(st, g, clip, lr, cfg)
                    skip = list(st["muon"]) + [(c["local"][0], c["local"][1], c["shape"]) for c in st["muon_cross"]]
            if st["a8"] is not None:
                from ..optim.adam8bit import adam8bit_update
                active = None
                if skip:
                    active = torch.ones(st["hi"] - st["lo"], dtype=torch.uint8, device=g.device)
                    for s0, e0, _ in skip:
                        active[s0:e0] = 0
                adam8bit_update(st["master"], st["a8"], g, out, st["wd_mask"], clip, lr, cfg.beta1, cfg.beta2, cfg.eps,
                                cfg.weight_decay, bc1, bc2, active=active)
                continue
            adamw_ops.adamw_shard_update(st["master"], st["m"], st["v"], g, out, st["wd_mask"], clip,
                                         lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, bc1, bc2,
                                         skip_segments=skip)
        for buf in self.buffers:
            buf.gather_params()
        return {"grad_norm": gnorm, "clip_coef": clip}

    # ---- checkpoint -------------------------------------------------------
    @torch.no_grad()
    def reset_master_from_params(self) -> None:
        """Re-seed the fp32 master shards from the (just loaded) low-precision parameters and clear
        the moments; used when a checkpoint was written under a different parallel layout."""
        for s in self.state:
            s["master"].copy_(s["buf"].param_buffer[s["lo"]:s["hi"]].float())
            for k in ("m", "v"):
                if s[k] is not None:
                    s[k].zero_()
            if s["a8"] is not None:
                for t in (s["a8"].m8, s["a8"].v8, s["a8"].am_m, s["a8"].am_v):
                    t.zero_()

    def state_dict(self) -> dict:
        return {
            "step": self.step_count, "lr": self.lr,
            "shards": [self._shard_state(s) for s in self.state],
        }

    @staticmethod
    def _shard_state(s) -> dict:
        d = {"lo": s["lo"], "hi": s["hi"], "master": s["master"].cpu()}
        for k in ("m", "v"):
            if s[k] is not None:
                d[k] = s[k].cpu()
        if s["a8"] is not None:
            a = s["a8"]
            d["a8"] = {"m8": a.m8.cpu(), "v8": a.v8.cpu(), "am_m": a.am_m.cpu(), "am_v": a.am_v.cpu()}
        return d

    def load_state_dict(self, sd: dict) -> None:
        self.step_count, self.lr = sd["step"], sd.get("lr", self.lr)
        if len(sd["shards"]) != len(self.state):
            raise ValueError("optimizer shard layout differs from the checkpoint")
        for s, t in zip(self.state, sd["shards"]):
            if (s["lo"], s["hi"]) != (t["lo"], t["hi"]):
                raise ValueError("optimizer shard ranges differ from the checkpoint")
            for k in ("master", "m", "v"):
                if s[k] is not None and k in t:
                    s[k].copy_(t[k].to(s[k].device))
            if s["a8"] is not None and "a8" in t:
                for k, v in t["a8"].items():
                    getattr(s["a8"], k).copy_(v.to(s["master"].device))
            s["buf"].param_buffer[s["lo"]:s["hi"]].copy_(s["master"].to(s["buf"].dtype))
        for buf in self.buffers:
            buf.gather_params()


_ = (math, Iterable)
