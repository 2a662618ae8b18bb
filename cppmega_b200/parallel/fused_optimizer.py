"""ZeRO-1 step with the collectives fused into the optimizer kernels over peer memory.

Per step and per shard, two kernels replace reduce-scatter + cast/scale + update + all-gather:

1. ``reduce_shard``: pulls this rank's slice of every rank's gradient buffer with peer loads, sums
   and scales it into fp32 and accumulates the squared norm;
2. ``adamw_push``: AdamW on the fp32 master slice, then stores the new bf16 values into every rank's
   parameter buffer with peer stores.

The reduction overlaps the backward pass bucket by bucket: when the last gradient of a bucket has been produced
(inside backward) this rank raises that bucket's ``GRAD`` flag on every peer and queues, on a second stream, a bounded
wait for the same flag of all peers followed by ``reduce_shard`` of its slice of the bucket - the counterpart of
``--overlap-grad-reduce`` (cppmega/recipes/nam56r_nemo_recipe.py:236-240), with peer loads instead of NCCL.  ``step()``
joins the second stream, all-reduces the squared norm (NCCL, 4 bytes) and runs ``adamw_push``.  The ``PARAM`` flag (my
pushes are complete - peers may run the next forward and may overwrite their gradient buffers) closes the step.  All
waits are bounded device-side waits.

Buffers whose reduction group has one rank (e.g. experts when EP spans the whole data-parallel
group) use the local fused AdamW kernel.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .dist_optimizer import DistributedOptimizer, OptimizerConfig, ParamGroupBuffer
from .symm_mem import SymmetricHeap

FLAG_GRAD = 0                 # kept for layout compatibility: whole-buffer "gradients ready" (unused with per-bucket flags)
FLAG_PARAM = 1
FLAG_BUCKET_BASE = 8          # flag index of bucket 0 of a heap's buffers (each heap has its own flag words)


class FusedDistributedOptimizer(DistributedOptimizer):
    def __init__(self, model, cfg: OptimizerConfig, pc, **kw):
        self._heaps: Dict[bool, Optional[SymmetricHeap]] = {}
        self._pc_for_alloc = pc
        self._side = None                        # second stream for the per-bucket pulls
        self._sq = None                          # [dense, expert] squared-norm accumulators of the running step
        self._bucket_flag, self._bucket_state = {}, {}
        kw["overlap"] = False                      # gradients stay local until the fused pull
        kw["distributed"] = True
        super().__init__(model, cfg, pc, **kw)
        from ..ops import cuda as cu
        self.L = cu.lib()
        vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        self.L.cm_reduce_shard.argtypes = [vp, i32, i32, i64, i64, f32, vp, vp, i32, vp, vp]
        self.L.cm_reduce_shard.restype = i32
        self.L.cm_adamw_push.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i64, i64, f32, f32, f32, f32, f32, f32, f32, i32, vp, vp]
        self.L.cm_adamw_push.restype = i32
        for st in self.state:
            buf: ParamGroupBuffer = st["buf"]
            if buf.n > 1:
                st["red"] = torch.empty(st["hi"] - st["lo"], dtype=torch.float32, device=st["master"].device)
        self._param_wait_pending = False
        # flag index and state entry of every (buffer, bucket) that lives in a heap
        per_heap = {}
        for st in self.state:
            buf, b = st["buf"], st["bucket"]
            if getattr(buf, "heap", None) is None:
                continue
            k = per_heap.get(id(buf.heap), 0)
            per_heap[id(buf.heap)] = k + 1
            self._bucket_flag[(id(buf), b.index)] = FLAG_BUCKET_BASE + k
            self._bucket_state[(id(buf), b.index)] = st
        if cfg.optimizer == "muon" or any(st.get("muon") or st.get("muon_cross") for st in self.state):
            raise NotImplementedError("the fused optimizer path implements AdamW; use the NCCL path for Muon")

    def _buffer_allocator(self, is_expert: bool, params, grad_dtype):
        pc = self._pc_for_alloc
        n = pc.edp if is_expert else pc.dp
        if n <= 1:
            return None
        group = pc.edp_group if is_expert else pc.dp_group
        ranks = pc.edp_ranks if is_expert else pc.dp_ranks
        heap = self._heaps.get(is_expert)
        if heap is None:
            total = 0
            for p in params:
                total += (p.numel() + 64) * (p.element_size() + torch.empty((), dtype=grad_dtype).element_size())
            # + per-bucket padding (128 * n elements each) and allocator alignment
            total += 64 << 20
            # dense buffers of other dtypes (fp32 per-head params) share the heap: reserve for them too
            total = int(total * 1.05)
            heap = SymmetricHeap(group, ranks, total, params[0].device)
            self._heaps[is_expert] = heap

        def alloc(buf: ParamGroupBuffer, numel: int, dtype: torch.dtype):
            buf.heap = heap
            return heap.alloc(numel, dtype)

        return alloc

    def _heaps_in_use(self):
        return [h for h in self._heaps.values() if h is not None]

    # gradients are reduced by the fused pull, not by NCCL
    def finish_grad_sync(self):
        for buf in self.buffers:
            if getattr(buf, "heap", None) is None:
                for b in buf.buckets:
                    if not b.reduced:
                        buf.reduce_bucket(b, async_op=False, scale=self._grad_scale / buf.grad_div)
                buf.finish()
            else:
                for b in buf.buckets:        # buckets whose hook never fired (parameters without a gradient this step)
                    if not b.reduced:
                        self._on_bucket_ready(buf, b)
        if self._side is not None:
            torch.cuda.current_stream().wait_stream(self._side)

    def zero_grad(self):
        # peers may still be pulling last step's gradients or pushing parameters: wait for their
        # PARAM flag before touching either buffer
        if getattr(self, "_param_wait_pending", False):
            for h in self._heaps_in_use():
                h.wait(FLAG_PARAM, self.step_count)
            self._param_wait_pending = False
        super().zero_grad()
        if getattr(self, "state", None):
            dev = self.state[0]["master"].device
            self._sq = torch.zeros(2, dtype=torch.float32, device=dev)       # [dense, expert] squared gradient norms of this step

    def _side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.state[0]["master"].device)
        return self._side

    def _on_bucket_ready(self, buf, b) -> None:
        """Inside backward: publish this bucket's gradients to the peers and start pulling its shard on the second stream."""
        key = (id(buf), b.index)
        st = self._bucket_state.get(key)
        if st is None:                       # a buffer without peers: scaled in finish_grad_sync
            return
        from ..ops import cuda as cu
        from ..ops import functional as F_
        step = self.step_count + 1
        flag = self._bucket_flag[key]
        heap = buf.heap
        heap.signal(flag, step)                                   # after the kernels that wrote these gradients (this stream)
        ev = torch.cuda.Event()
        ev.record()
        side = self._side_stream()
        side.wait_event(ev)                                       # this rank's own gradients are read by the pull as well
        dev = st["master"].device
        with torch.cuda.stream(side):
            heap.wait(flag, step)
            sq = self._sq[1:2] if buf.is_expert else self._sq[0:1]
            gk = 0 if buf.grad_buffer.dtype == torch.float32 else 1
            arr = heap.peer_ptr_array(buf.grad_buffer)
            rc = self.L.cm_reduce_shard(arr, buf.n, buf.rank, st["lo"], st["hi"] - st["lo"],
                                        float(self._grad_scale / buf.grad_div), st["red"].data_ptr(), sq.data_ptr(), gk,
                                        cu.err_word(dev).data_ptr(), cu.stream_ptr())
            if rc:
                raise RuntimeError(f"cm_reduce_shard failed ({rc})")
            F_.count_launch("reduce_shard")
        b.reduced = True

    @torch.no_grad()
    def step(self, lr: Optional[float] = None):
        from ..ops import cuda as cu
        from ..optim import adamw as adamw_ops
        cfg, pc = self.cfg, self.pc
        lr = self.lr if lr is None else lr
        self.finish_grad_sync()
        step = self.step_count + 1
        heaps = self._heaps_in_use()
        dev = self.state[0]["master"].device
        s = cu.stream_ptr()
        if pc.tp > 1:
            dense_sq, expert_sq = self._tensor_parallel_fixup()
        else:
            dense_sq, expert_sq = self._sq[0].clone(), self._sq[1].clone()   # filled by the per-bucket pulls
            for st in self.state:
                buf: ParamGroupBuffer = st["buf"]
                if "red" not in st:
                    g = buf.grad_buffer[st["lo"]:st["hi"]]
                    if buf.is_expert:
                        expert_sq += self._sumsq_tp_aware(st, g)
                    else:
                        dense_sq += self._sumsq_tp_aware(st, g)
        gnorm = self._finish_norm(dense_sq, expert_sq)
        clip = torch.ones_like(gnorm)
        if cfg.clip_grad > 0:
            clip = torch.clamp(cfg.clip_grad / (gnorm + 1e-6), max=1.0)
        self.step_count = step
        bc1 = 1.0 - cfg.beta1 ** step
        bc2 = 1.0 - cfg.beta2 ** step
        clip_t = clip.reshape(1).float().contiguous()
        for st in self.state:
            buf = st["buf"]
            if "red" in st:
                ok = 0 if buf.param_buffer.dtype == torch.float32 else 1
                arr = buf.heap.peer_ptr_array(buf.param_buffer)
                rc = self.L.cm_adamw_push(st["master"].data_ptr(), st["m"].data_ptr(), st["v"].data_ptr(),
                                          st["red"].data_ptr(), st["wd_mask"].data_ptr(), clip_t.data_ptr(), arr, buf.n,
                                          st["lo"], st["hi"] - st["lo"], float(lr), cfg.beta1, cfg.beta2, cfg.eps,
                                          cfg.weight_decay, bc1, bc2, ok, cu.err_word(dev).data_ptr(), s)
                if rc:
                    raise RuntimeError(f"cm_adamw_push failed ({rc})")
                from ..ops import functional as F_
                F_.count_launch("adamw_push")
            else:
                g = buf.grad_buffer[st["lo"]:st["hi"]]
                out = buf.param_buffer[st["lo"]:st["hi"]]
                adamw_ops.adamw_shard_update(st["master"], st["m"], st["v"], g, out, st["wd_mask"], clip, lr,
                                             cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, bc1, bc2,
                                             gate=cu.err_word(dev))
        for h in heaps:
            h.signal(FLAG_PARAM, step)
        self._param_wait_pending = bool(heaps)
        return {"grad_norm": gnorm, "clip_coef": clip}

    handles_sequence_parallel_grads = True       # the trainer must not all-reduce ``main_grad`` (peers pull from it)

    def _tensor_parallel_fixup(self):
        """TP > 1 with sequence parallelism, after the data-parallel reduction of every shard.  (1) Gradients of
        parameters that every TP rank holds whole but computes from its own sequence shard (norm weights, routers,
        experts) are partial sums: their segments of the reduced shards are all-reduced over the TP group, coalesced
        into one flat buffer.  (2) The squared norm is recomputed from the final values, counting tensors replicated
        over TP ``1 / tp`` so that the TP all-reduce of the norm counts them once.  Returns (dense, expert) sums."""
        pc = self.pc
        tp = pc.tp
        dev = self.state[0]["master"].device
        partial, replicated = [], []               # (shard view, is_expert)
        whole = []
        for st in self.state:
            buf, lo, hi = st["buf"], st["lo"], st["hi"]
            src = st["red"] if "red" in st else buf.grad_buffer[lo:hi]
            whole.append((src, buf.is_expert))
            for p in st["bucket"].params:
                off = buf.offsets[p]
                a, b = max(off, lo), min(off + p.numel(), hi)
                if a >= b:
                    continue
                seg = src[a - lo:b - lo]
                if getattr(p, "sequence_parallel_grad", False):
                    partial.append(seg)
                if not getattr(p, "tensor_model_parallel", False):
                    replicated.append((seg, buf.is_expert))
        if partial:
            flat = torch.cat([x.reshape(-1).float() for x in partial])
            dist.all_reduce(flat, group=pc.tp_group)
            o = 0
            for x in partial:
                x.copy_(flat[o:o + x.numel()])
                o += x.numel()
        sq = torch.zeros(2, dtype=torch.float32, device=dev)
        for src, is_expert in whole:
            xf = src.float()
            sq[1 if is_expert else 0] += (xf * xf).sum()
        for seg, is_expert in replicated:
            xf = seg.float()
            sq[1 if is_expert else 0] -= (1.0 - 1.0 / tp) * (xf * xf).sum()
        return sq[0].clone(), sq[1].clone()

    def _finish_norm(self, dense_sq, expert_sq):
        """Same reduction tree as ``DistributedOptimizer.grad_norm`` on already-sharded sums."""
        pc = self.pc
        if pc.dp > 1:
            dist.all_reduce(dense_sq, group=pc.dp_group)
            dist.all_reduce(expert_sq, group=pc.dp_group)
        total = dense_sq + expert_sq
        if pc.tp > 1:
            dist.all_reduce(total, group=pc.tp_group)
        if pc.pp > 1:
            dist.all_reduce(total, group=pc.pp_group)
        return total.sqrt()

    def close(self):
        super().close()
        for h in self._heaps_in_use():
            h.close()
        self._heaps = {}


def fused_optimizer_supported(pc, device: torch.device) -> bool:
    from .symm_mem import peer_access_available
    return (device.type == "cuda" and pc.world_size > 1 and pc.dp > 1
            and pc.config.distributed_optimizer and pc.config.fused_collectives and peer_access_available(pc))
