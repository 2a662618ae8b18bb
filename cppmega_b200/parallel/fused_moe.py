"""Expert-parallel MoE layer body over peer memory: dispatch fused with the permutation, grouped
tcgen05 expert GEMMs on the receiving rank, combine fused with un-permutation and weighting.

Forward on every rank of the EP group (same call order everywhere):

1. ``plan``: all ranks exchange per-expert token counts (one tiny all-gather) and derive, without
   a host sync, the final row of every routed copy inside the owner's 128-row-aligned expert
   segments;
2. ``push_rows``: copies go straight to those rows of the owner's symmetric input buffer;
3. flag barrier, then the owner runs fc1 -> SwiGLU -> fc2 with the grouped GEMM kernels;
4. flag barrier, then ``pull_combine`` reads each token's k results from their owners and forms the
   weighted sum.

Backward mirrors it: weighted output gradients are pushed to the owners, the grouped dgrad / wgrad
kernels run there, input gradients are pulled back and summed over k; the routing-weight gradient
is a row-dot against the owners' saved outputs.

Symmetric buffers: per layer an input and an output row buffer (they must survive until that
layer's backward), plus two buffers shared by all layers for the backward traffic.  Capacity is
``capacity_factor`` times the mean load (the worst case, ``ep`` times, when the buffers are shared by all
layers); an overflow drops the copies that do not fit, never forms an address outside a buffer, and sets the
kernel error word.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as F_
from .symm_mem import SymmetricHeap

TILE = 128
FLAG_BASE = 16
FLAGS_PER_LAYER = 5          # dispatch, expert outputs, grad dispatch, grad outputs, count exchange


def _lib():
    from ..ops import cuda as cu
    L = cu.lib()
    if not getattr(L, "_moe_declared", False):
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        L.cm_moe_push_rows.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, vp, vp]
        L.cm_moe_pull_combine.argtypes = [vp, i32, vp, vp, vp, vp, i32, i32, i32, i64, vp, vp]
        L.cm_moe_pull_rowdot.argtypes = [vp, i32, vp, vp, vp, vp, i32, i32, i32, i64, vp, vp]
        L.cm_moe_zero_pad_rows.argtypes = [vp, vp, vp, i32, i32, i64, vp]
        L.cm_moe_count.argtypes = [vp, i64, i32, vp, vp, vp]
        L.cm_moe_plan.argtypes = [vp, i64, i32, i32, i32, i32, vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp]
        for n in ("cm_moe_push_rows", "cm_moe_pull_combine", "cm_moe_pull_rowdot", "cm_moe_zero_pad_rows", "cm_moe_count", "cm_moe_plan"):
            getattr(L, n).restype = i32
        L._moe_declared = True
    return L


class MoEPlan:
    """Device-side routing plan of one call (no host synchronisation)."""

    use_kernels = True        # False: build the plan from library ops (the definition the kernels are tested against)

    def __init__(self, ids: torch.Tensor, num_experts: int, ep: int, ep_rank: int, group, capacity_rows: int, gather=None):
        T, k = ids.shape
        E, El = num_experts, num_experts // ep
        dev = ids.device
        flat = ids.reshape(-1)
        if self.use_kernels and ids.is_cuda and ids.dtype == torch.int64 and E <= 32 and 0 < T * k <= 64 * 255 * 1024:
            self._build_on_device(flat.contiguous(), T, k, E, El, ep, ep_rank, group, capacity_rows, gather)
            return
        counts = torch.bincount(flat, minlength=E)
        if ep > 1 and gather is not None:
            allc = gather(counts)                                # [src rank, expert] through peer memory
        elif ep > 1:
            allc = torch.empty(ep * E, dtype=counts.dtype, device=dev)
            dist.all_gather_into_tensor(allc, counts.contiguous(), group=group)
            allc = allc.view(ep, E)                              # [src rank, expert]
        else:
            allc = counts.view(1, E)
        tot = allc.sum(0)                                        # rows per expert (all sources)
        padded = (tot + (TILE - 1)) // TILE * TILE
        pe = padded.view(ep, El)
        seg_end = torch.cumsum(pe, 1)
        seg_start = (seg_end - pe).reshape(E)                    # start row of each expert on its owner
        before_me = allc[:ep_rank].sum(0) if ep_rank > 0 else torch.zeros_like(tot)
        base = seg_start + before_me                             # first row of my copies of expert e
        sort_idx = torch.argsort(flat, stable=True)
        e_sorted = flat[sort_idx]
        un_end = torch.cumsum(counts, 0)
        un_start = un_end - counts
        pos = torch.arange(T * k, device=dev)
        row_sorted = base[e_sorted] + (pos - un_start[e_sorted])
        # per copy in (token, j) order
        dest_row = torch.empty(T * k, dtype=torch.int64, device=dev)
        dest_row[sort_idx] = row_sorted
        self.dest_row = dest_row
        self.dest_rank = torch.div(flat, El, rounding_mode="floor").to(torch.int32)
        self.token_of_copy = torch.div(pos, k, rounding_mode="floor").to(torch.int32)
        self.T, self.k = T, k
        # receiver side (my local experts)
        lo = ep_rank * El
        my_tot = tot[lo:lo + El]
        my_pad = padded[lo:lo + El]
        my_end = torch.cumsum(my_pad, 0)
        my_start = (my_end - my_pad).clamp(max=capacity_rows)
        my_end = my_end.clamp(max=capacity_rows)                 # an overflowing routing is clipped to the buffer (and reported by push)
        self.seg_start_local = my_start.to(torch.int32)
        self.tot_local = torch.minimum(my_tot, my_end - my_start).to(torch.int32)
        self.seg_offsets = torch.cat([torch.zeros(1, dtype=my_end.dtype, device=dev), my_end]).to(torch.int32)
        tiles = torch.arange(capacity_rows // TILE, device=dev) * TILE
        te = torch.searchsorted(my_end, tiles, right=True)
        self.tile_expert = torch.where(te < El, te, torch.full_like(te, -1)).to(torch.int32)
        self.rows_used = my_end[-1]
        self.counts_global = tot


def _build_on_device(self, flat, T, k, E, El, ep, ep_rank, group, capacity_rows, gather):
    """The plan from two kernels (`moe_count`, `moe_plan`) instead of the chain of library ops below."""
    from ..ops.cuda import stream_ptr
    L, dev, n = _lib(), flat.device, T * k
    counts = torch.zeros(E, dtype=torch.int64, device=dev)
    block_counts = torch.empty(64 * E, dtype=torch.int32, device=dev)          # per-chunk parts, same chunks in both kernels
    rc = L.cm_moe_count(flat.data_ptr(), n, E, counts.data_ptr(), block_counts.data_ptr(), stream_ptr())
    if rc:
        raise RuntimeError(f"cm_moe_count failed ({rc})")
    if ep > 1 and gather is not None:
        allc = gather(counts)
    elif ep > 1:
        allc = torch.empty(ep * E, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(allc, counts, group=group)
    else:
        allc = counts
    n_tiles = capacity_rows // TILE
    i32 = lambda m: torch.empty(m, dtype=torch.int32, device=dev)
    self.dest_row = torch.empty(n, dtype=torch.int64, device=dev)
    self.dest_rank, self.token_of_copy = i32(n), i32(n)
    self.seg_start_local, self.tot_local, self.seg_offsets, self.tile_expert = i32(El), i32(El), i32(El + 1), i32(n_tiles)
    self.counts_global = torch.empty(E, dtype=torch.int64, device=dev)
    rc = L.cm_moe_plan(flat.data_ptr(), n, k, E, ep, ep_rank, allc.data_ptr(), block_counts.data_ptr(), TILE, n_tiles, self.dest_row.data_ptr(),
                       self.dest_rank.data_ptr(), self.token_of_copy.data_ptr(), self.seg_start_local.data_ptr(),
                       self.tot_local.data_ptr(), self.seg_offsets.data_ptr(), self.tile_expert.data_ptr(),
                       self.counts_global.data_ptr(), stream_ptr())
    if rc:
        raise RuntimeError(f"cm_moe_plan failed ({rc})")
    F_.count_launch("moe_plan", 2)
    self.T, self.k = T, k
    self.rows_used = self.seg_offsets[-1]


MoEPlan._build_on_device = _build_on_device


class FusedMoEBuffers:
    """Symmetric buffers of one EP group; one instance shared by all MoE layers of the model."""

    def __init__(self, pc, hidden: int, tokens_per_rank: int, topk: int, num_layers: int, device,
                 capacity_factor: Optional[float] = None, per_layer: bool = True, num_local_experts: int = 16):
        """``capacity_factor``: receive rows per buffer as a multiple of the mean load ``tokens_per_rank * topk``.
        ``None`` picks the worst case (every copy of every rank lands here: ``ep`` times the mean, no routing can
        overflow) when the buffers are shared by all layers, and 2.0 when every layer keeps its own pair, where the
        worst case would not fit; an overflow there drops the copies, zeroes their contribution and sets the error word."""
        self.pc = pc
        self.hidden = hidden
        El = 1
        mean_rows = tokens_per_rank * topk
        if capacity_factor is None:
            capacity_factor = 2.0 if per_layer else float(pc.ep)
        capacity_factor = min(float(capacity_factor), float(pc.ep))
        self.capacity_factor = capacity_factor
        pad_rows = max(16, num_local_experts) * TILE          # every local expert segment may end in a partial tile
        self.capacity = int((mean_rows * capacity_factor + pad_rows + TILE - 1) // TILE * TILE)
        n_bufs = (2 * num_layers if per_layer else 2) + 2
        nbytes = n_bufs * (self.capacity * hidden * 2 + 4096) + num_layers * 4096 * 2
        self.heap = SymmetricHeap(pc.ep_group, pc.ep_ranks, nbytes, device)
        self.per_layer = per_layer
        self.layer_bufs: List = []
        n = num_layers if per_layer else 1
        for _ in range(n):
            self.layer_bufs.append((self.heap.alloc((self.capacity, hidden), torch.bfloat16),
                                    self.heap.alloc((self.capacity, hidden), torch.bfloat16)))
        self.grad_in_ = self.heap.alloc((self.capacity, hidden), torch.bfloat16)
        self.grad_out_ = self.heap.alloc((self.capacity, hidden), torch.bfloat16)
        self.num_layers = num_layers
        self.count_bufs = {}                  # (layer slot, expert count) -> [ep, E] int64 exchange buffer
        self.epoch = 0
        _ = El

    def gather_counts(self, layer_slot: int, epoch: int, counts: torch.Tensor) -> torch.Tensor:
        """[E] per-expert copy counts of this rank -> [ep, E] of all ranks, through peer stores and one flag barrier
        (flag 4 of the layer's group of five) instead of a library all-gather."""
        key = (layer_slot, counts.numel())
        buf = self.count_bufs.get(key)
        if buf is None:
            buf = self.count_bufs[key] = self.heap.alloc((self.heap.world, counts.numel()), torch.int64)
        return self.heap.all_gather_words(counts.to(torch.int64).contiguous(), buf, FLAG_BASE + FLAGS_PER_LAYER * layer_slot + 4, epoch)

    def capacity_for(self, ncopies: int) -> int:
        return self.capacity

    def bufs(self, layer_slot: int, cap: int):
        return self.layer_bufs[layer_slot if self.per_layer else 0]

    def grad_bufs(self, cap: int):
        return self.grad_in_, self.grad_out_

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


class _LocalHeap:
    """Stand-in for the symmetric heap when all experts live on this GPU: one "peer", no flags."""

    world = 1

    @staticmethod
    def peer_ptr_array(t: torch.Tensor):
        return (ctypes.c_void_p * 1)(t.data_ptr())

    @staticmethod
    def barrier(*_args) -> None:
        return None


class LocalMoEBuffers:
    """EP = 1: the same permute-fused kernels on ordinary (caching-allocator) buffers.  Row buffers are exact-size
    (every copy lands here, so T*k rows plus at most 127 padding rows per expert) and live as long as autograd needs
    them, which with layer recomputation is one layer at a time."""

    def __init__(self, pc, hidden: int, num_experts: int, device):
        self.pc, self.hidden, self.num_experts, self.device = pc, hidden, num_experts, device
        self.heap = _LocalHeap()
        self.epoch = 0

    def capacity_for(self, ncopies: int) -> int:
        return (ncopies + self.num_experts * (TILE - 1) + TILE - 1) // TILE * TILE

    def _row_buf(self, cap: int):
        return torch.empty(cap, self.hidden, dtype=torch.bfloat16, device=self.device)

    def bufs(self, layer_slot: int, cap: int):
        return self._row_buf(cap), self._row_buf(cap)

    def grad_bufs(self, cap: int):
        return self._row_buf(cap), self._row_buf(cap)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


def _push(heap: SymmetricHeap, src, plan: MoEPlan, dst_buf, scale=None):
    from ..ops.cuda import err_word, stream_ptr
    rc = _lib().cm_moe_push_rows(src.data_ptr(), plan.token_of_copy.data_ptr(), plan.dest_rank.data_ptr(),
                                 plan.dest_row.data_ptr(), None if scale is None else scale.data_ptr(),
                                 heap.peer_ptr_array(dst_buf), heap.world, plan.T * plan.k, src.shape[1],
                                 dst_buf.shape[0], err_word(src.device).data_ptr(), stream_ptr())
    if rc:
        raise RuntimeError(f"cm_moe_push_rows failed ({rc})")
    F_.count_launch("moe_push_rows")


def _pull_combine(heap: SymmetricHeap, src_buf, plan: MoEPlan, weights, H, dtype):
    from ..ops.cuda import err_word, stream_ptr
    out = torch.empty(plan.T, H, dtype=dtype, device=src_buf.device)
    rc = _lib().cm_moe_pull_combine(heap.peer_ptr_array(src_buf), heap.world, plan.dest_rank.data_ptr(),
                                    plan.dest_row.data_ptr(), None if weights is None else weights.data_ptr(),
                                    out.data_ptr(), plan.T, plan.k, H, src_buf.shape[0],
                                    err_word(src_buf.device).data_ptr(), stream_ptr())
    if rc:
        raise RuntimeError(f"cm_moe_pull_combine failed ({rc})")
    F_.count_launch("moe_pull_combine")
    return out


def _pull_rowdot(heap: SymmetricHeap, src_buf, plan: MoEPlan, dy):
    from ..ops.cuda import err_word, stream_ptr
    out = torch.empty(plan.T, plan.k, dtype=torch.float32, device=dy.device)
    rc = _lib().cm_moe_pull_rowdot(heap.peer_ptr_array(src_buf), heap.world, plan.dest_rank.data_ptr(),
                                   plan.dest_row.data_ptr(), dy.data_ptr(), out.data_ptr(), plan.T, plan.k, dy.shape[1],
                                   src_buf.shape[0], err_word(dy.device).data_ptr(), stream_ptr())
    if rc:
        raise RuntimeError(f"cm_moe_pull_rowdot failed ({rc})")
    F_.count_launch("moe_pull_rowdot")
    return out


def _zero_pad(buf, plan: MoEPlan, capacity: int):
    from ..ops.cuda import stream_ptr
    rc = _lib().cm_moe_zero_pad_rows(buf.data_ptr(), plan.seg_start_local.data_ptr(), plan.tot_local.data_ptr(),
                                     plan.tot_local.numel(), buf.shape[1], capacity, stream_ptr())
    if rc:
        raise RuntimeError(f"cm_moe_zero_pad_rows failed ({rc})")


def _grouped(x, w, tile_expert, rows, b_mn, out=None):
    """out[r] = x[r] . W[e(r)]^T (b_mn False) or x[r] . W[e(r)] (b_mn True, W [E, red, out])."""
    from ..ops.cuda import lib, err_word, stream_ptr, _check
    E = w.shape[0]
    if b_mn:
        red, n_out = w.shape[1], w.shape[2]
    else:
        n_out, red = w.shape[1], w.shape[2]
    if out is None:
        out = torch.empty(rows, n_out, dtype=x.dtype, device=x.device)
    _check(lib().cm_grouped_gemm_rows_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), rows, n_out, red, E, int(b_mn),
                                           tile_expert.data_ptr(), err_word(x.device).data_ptr(), stream_ptr()),
           "cm_grouped_gemm_rows_bf16")
    F_.count_launch("grouped_gemm")
    return out


def _grouped_wgrad(dy, x, seg_offsets, E, w=None):
    """dW[e] = dy_e^T x_e per expert segment; accumulated into ``w.main_grad`` when the optimizer allows it."""
    from ..ops.cuda import lib, err_word, stream_ptr, _check, wgrad_into_main_grad
    rows, N = dy.shape
    K = x.shape[1]

    def run(out, acc):
        out = torch.empty(E, N, K, dtype=dy.dtype, device=dy.device) if out is None else out
        _check(lib().cm_grouped_gemm_k_bf16(dy.data_ptr(), x.data_ptr(), out.data_ptr(), rows, N, K, E, seg_offsets.data_ptr(),
                                            int(out.dtype == torch.float32), int(acc), err_word(dy.device).data_ptr(),
                                            stream_ptr()), "cm_grouped_gemm_k_bf16")
        F_.count_launch("grouped_gemm")
        return out
    return run(None, False) if w is None else wgrad_into_main_grad(w, run)


def _fp8_mode(w1, w2) -> Optional[str]:
    """``None`` (bf16 experts), ``"mxfp8"`` or ``"tensorwise"``: the recipe in force where the layer's forward runs.  The
    block-scaled expert GEMMs want every expert's rows / columns to start on a 128 boundary of the stacked weights."""
    rec = F_.precision_recipe()
    if rec == "bf16":
        return None
    ok = (w1.dtype == torch.bfloat16 and w1.shape[1] % 128 == 0 and w1.shape[2] % 128 == 0
          and w2.shape[1] % 128 == 0 and w2.shape[2] % 128 == 0)
    return rec if ok else None


def _experts_fwd_mx(xin, w1, w2, tile_expert, yout, tensorwise: bool):
    """h = xin W1^T, yout = swiglu(h) W2^T on the block-scaled grouped GEMM; returns h."""
    from ..ops.cuda import mxfp8 as mx, swiglu
    E = w1.shape[0]
    tw = True if tensorwise else None
    h = mx.grouped_rows_mxfp8(mx.quantize_rowwise(xin, True, tw), mx.quantize_expert_weights(w1, False, tensorwise), tile_expert, E,
                              w1.shape[1], False)
    a = swiglu(h)
    mx.grouped_rows_mxfp8(mx.quantize_rowwise(a, True, tw), mx.quantize_expert_weights(w2, False, tensorwise), tile_expert, E,
                          w2.shape[1], False, out=yout)
    return h


def _experts_bwd_mx(grad_in, h, xin, w1, w2, plan, grad_out, tensorwise: bool):
    """Expert backward in FP8: every operand is quantised along the axis its product reduces over; a tensor that
    feeds both a dgrad (along features) and a wgrad (along tokens) is read once for both copies."""
    from ..ops.cuda import lib, mxfp8 as mx, stream_ptr, swiglu, wgrad_into_main_grad, _check
    E, cap = w1.shape[0], grad_in.shape[0]
    tw = (lambda t: mx.tensor_amax(t)) if tensorwise else (lambda t: None)
    a = swiglu(h)
    g_row, g_col = mx.quantize_both(grad_in, True, tw(grad_in))                         # [cap, H] and [H, cap]
    da = mx.grouped_rows_mxfp8(g_row, mx.quantize_expert_weights(w2, True, tensorwise), plan.tile_expert, E, w2.shape[2], True)     # [cap, F]
    a_col = mx.quantize_colwise(a, True, tw(a))                                         # [F, cap]
    dw2 = wgrad_into_main_grad(w2, lambda out, acc: mx.grouped_wgrad_mxfp8(g_col, a_col, plan.seg_offsets, E, out, acc))
    dh = torch.empty_like(h)
    _check(lib().cm_swiglu_bwd(h.data_ptr(), da.data_ptr(), dh.data_ptr(), cap, w2.shape[2], stream_ptr()), "cm_swiglu_bwd")
    F_.count_launch("swiglu_bwd")
    dh_row, dh_col = mx.quantize_both(dh, True, tw(dh))                                 # [cap, 2F] and [2F, cap]
    mx.grouped_rows_mxfp8(dh_row, mx.quantize_expert_weights(w1, True, tensorwise), plan.tile_expert, E, w1.shape[2], True, out=grad_out)
    x_col = mx.quantize_colwise(xin, True, tw(xin))                                     # [H, cap]
    dw1 = wgrad_into_main_grad(w1, lambda out, acc: mx.grouped_wgrad_mxfp8(dh_col, x_col, plan.seg_offsets, E, out, acc))
    return dw1, dw2


class _FusedMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, w1, w2, ids, bufs: FusedMoEBuffers, layer_slot: int):
        from ..ops.cuda import swiglu
        pc, heap = bufs.pc, bufs.heap
        cap = bufs.capacity_for(ids.numel())
        H = x.shape[1]
        ep0 = bufs.next_epoch()
        gather = (lambda c: bufs.gather_counts(layer_slot, ep0, c)) if hasattr(bufs, "gather_counts") else None
        plan = MoEPlan(ids, w1.shape[0] * pc.ep, pc.ep, pc.ep_rank, pc.ep_group, cap, gather)
        xin, yout = bufs.bufs(layer_slot, cap)
        f0 = FLAG_BASE + FLAGS_PER_LAYER * layer_slot
        x = x.contiguous()
        _push(heap, x, plan, xin)
        heap.barrier(f0 + 0, ep0)
        _zero_pad(xin, plan, cap)
        with torch.no_grad():
            fp8 = _fp8_mode(w1, w2)
            if fp8 is not None:
                h = _experts_fwd_mx(xin, w1, w2, plan.tile_expert, yout, fp8 == "tensorwise")
            else:
                h = _grouped(xin, w1, plan.tile_expert, cap, False)
                a = swiglu(h)
                _grouped(a, w2, plan.tile_expert, cap, False, out=yout)
        heap.barrier(f0 + 1, ep0)
        p32 = probs.float().contiguous()
        y = _pull_combine(heap, yout, plan, p32.reshape(-1), H, x.dtype)
        # xin / yout go through save_for_backward as well: activation checkpointing only drops what it sees there
        ctx.save_for_backward(h, w1, w2, p32, xin, yout)
        ctx.plan, ctx.bufs, ctx.slot, ctx.cap = plan, bufs, layer_slot, cap
        ctx.x_dtype, ctx.p_dtype = x.dtype, probs.dtype
        ctx.fp8 = fp8                              # the backward runs under the recipe of its forward, whatever is set then
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.cuda import lib, stream_ptr, _check
        h, w1, w2, p32, xin, yout = ctx.saved_tensors
        plan, bufs = ctx.plan, ctx.bufs
        pc, heap, cap = bufs.pc, bufs.heap, ctx.cap
        grad_in, grad_out = bufs.grad_bufs(cap)
        H = dy.shape[1]
        dy = dy.contiguous()
        epb = bufs.next_epoch()
        f0 = FLAG_BASE + FLAGS_PER_LAYER * ctx.slot
        dprobs = _pull_rowdot(heap, yout, plan, dy)
        _push(heap, dy, plan, grad_in, scale=p32.reshape(-1))
        heap.barrier(f0 + 2, epb)
        _zero_pad(grad_in, plan, cap)      # padding rows feed the wgrad products: 0 * stale NaN would poison them
        E = w1.shape[0]
        Fh = w2.shape[2]
        # recompute a = swiglu(h); expert backward on the padded layout
        from ..ops.cuda import swiglu as _sw
        if ctx.fp8 is not None:
            with torch.no_grad():
                dw1, dw2 = _experts_bwd_mx(grad_in, h, xin, w1, w2, plan, grad_out, ctx.fp8 == "tensorwise")
            heap.barrier(f0 + 3, epb)
            dx = _pull_combine(heap, grad_out, plan, None, H, ctx.x_dtype)
            return dx, dprobs.to(ctx.p_dtype), dw1, dw2, None, None, None
        with torch.no_grad():
            a = _sw(h)
            da = _grouped(grad_in, w2, plan.tile_expert, cap, True)                  # [cap, F]
            dw2 = _grouped_wgrad(grad_in, a, plan.seg_offsets, E, w2)                   # [E, H, F]
            dh = torch.empty_like(h)
            _check(lib().cm_swiglu_bwd(h.data_ptr(), da.data_ptr(), dh.data_ptr(), cap, Fh, stream_ptr()), "cm_swiglu_bwd")
            F_.count_launch("swiglu_bwd")
            _grouped(dh, w1, plan.tile_expert, cap, True, out=grad_out)               # [cap, H]
            dw1 = _grouped_wgrad(dh, xin, plan.seg_offsets, E, w1)                        # [E, 2F, H]
        heap.barrier(f0 + 3, epb)
        dx = _pull_combine(heap, grad_out, plan, None, H, ctx.x_dtype)
        return dx, dprobs.to(ctx.p_dtype), dw1, dw2, None, None, None


class FusedMoEDispatcher:
    """Callable installed as ``MoELayer.fused_dispatcher``."""

    def __init__(self, bufs: FusedMoEBuffers, layer_slot: int):
        self.bufs, self.slot = bufs, layer_slot

    def __call__(self, flat, probs, ids, experts):
        return _FusedMoEFn.apply(flat, probs, experts.weight1, experts.weight2, ids, self.bufs, self.slot)


def attach(model, pc, device, tokens_per_rank: int, per_layer: bool = True, capacity_factor: Optional[float] = None,
           overlap_shared_expert: bool = True) -> Optional[FusedMoEBuffers]:
    """Install the fused dispatcher on every MoE layer of ``model`` (EP > 1, bf16, peer access)."""
    layers = model.moe_layers()
    if not layers:
        return None
    hidden = model.cfg.hidden_size
    if pc.ep <= 1:
        local = LocalMoEBuffers(pc, hidden, model.cfg.moe.num_experts, device)
        for slot, m in enumerate(layers):
            m.fused_dispatcher = FusedMoEDispatcher(local, slot)
        return local
    if capacity_factor is None:
        capacity_factor = model.cfg.moe.capacity_factor
    bufs = FusedMoEBuffers(pc, hidden, tokens_per_rank, model.cfg.moe.topk, len(layers), device,
                           capacity_factor=capacity_factor, per_layer=per_layer,
                           num_local_experts=model.cfg.moe.num_experts // pc.ep)
    for slot, m in enumerate(layers):
        m.fused_dispatcher = FusedMoEDispatcher(bufs, slot)
        # the routed path is mostly NVLink transfers and flag waits: the shared expert's GEMMs run beside it on a second stream
        m.overlap_shared_expert = overlap_shared_expert
    return bufs
