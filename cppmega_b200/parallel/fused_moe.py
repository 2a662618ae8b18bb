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

With EP > 1 and enough tokens the call is split into two token chunks with their own plans, buffer halves and
flags: a second ("transport") stream carries plan + push of chunk 1 while the expert GEMMs of chunk 0 run, and the
combine of chunk 0 while the GEMMs of chunk 1 run (backward likewise), so about half of the NVLink time sits under
tensor-core work.  Cross-GPU order is carried by the flags (signalled on the stream that produced the data, awaited
with a bounded wait on the stream that consumes it), same-GPU order between the two streams by events.

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
FLAGS_PER_CHUNK = 5          # dispatch, expert outputs, grad dispatch, grad outputs, count exchange
MAX_CHUNKS = 2               # token chunks per call whose transfers and expert GEMMs overlap (two streams)
FLAGS_PER_LAYER = FLAGS_PER_CHUNK * MAX_CHUNKS
MIN_CHUNK_COPIES = 8192      # below this many routed copies per chunk the pipeline is not worth its launches


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
        pad_rows = MAX_CHUNKS * max(16, num_local_experts) * TILE      # every local expert segment of every chunk may end in a partial tile
        self.capacity = int((mean_rows * capacity_factor + pad_rows + MAX_CHUNKS * TILE - 1) // (MAX_CHUNKS * TILE) * (MAX_CHUNKS * TILE))
        n_bufs = (2 * num_layers if per_layer else 2) + 2
        nbytes = n_bufs * (self.capacity * hidden * 2 + 4096) + num_layers * 4096 * 2 * MAX_CHUNKS
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
        self.count_bufs = {}                  # (layer slot, chunk, expert count) -> [ep, E] int64 exchange buffer
        self.epoch = 0
        self.chunks = MAX_CHUNKS              # 1: everything on the calling stream, one plan per call
        self._comm = None
        _ = El

    def chunks_for(self, tokens: int, topk: int) -> int:
        n = max(1, min(int(self.chunks), MAX_CHUNKS))
        while n > 1 and (tokens % n or (tokens // n) * topk < MIN_CHUNK_COPIES):
            n -= 1
        return n

    def comm_stream(self):
        if self._comm is None:
            self._comm = torch.cuda.Stream(device=self.heap.device)
        return self._comm

    def gather_counts(self, layer_slot: int, chunk: int, epoch: int, counts: torch.Tensor) -> torch.Tensor:
        """[E] per-expert copy counts of this rank -> [ep, E] of all ranks, through peer stores and one flag barrier
        (flag 4 of the chunk's group of five) instead of a library all-gather."""
        key = (layer_slot, chunk, counts.numel())
        buf = self.count_bufs.get(key)
        if buf is None:
            buf = self.count_bufs[key] = self.heap.alloc((self.heap.world, counts.numel()), torch.int64)
        return self.heap.all_gather_words(counts.to(torch.int64).contiguous(), buf, _flag0(layer_slot, chunk) + 4, epoch)

    def capacity_for(self, ncopies: int) -> int:
        return self.capacity

    def bufs(self, layer_slot: int, cap: int):
        return self.layer_bufs[layer_slot if self.per_layer else 0]

    def grad_bufs(self, cap: int):
        return self.grad_in_, self.grad_out_

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


def set_transport_blocks_per_sm(n: int) -> int:
    """Blocks of 256 threads per SM that a push / pull launch may take (1..8); returns the previous value.  8 is fastest
    for a transfer that runs alone; the two-stream pipeline wants fewer, so that a transfer leaves room on every SM for
    the expert GEMM CTA of the other chunk."""
    L = _lib()
    L.cm_moe_set_transport_blocks_per_sm.argtypes = [ctypes.c_int]
    L.cm_moe_set_transport_blocks_per_sm.restype = ctypes.c_int
    return int(L.cm_moe_set_transport_blocks_per_sm(int(n)))


def _flag0(layer_slot: int, chunk: int) -> int:
    return FLAG_BASE + FLAGS_PER_LAYER * layer_slot + FLAGS_PER_CHUNK * chunk


class _LocalHeap:
    """Stand-in for the symmetric heap when all experts live on this GPU: one "peer", no flags."""

    world = 1

    @staticmethod
    def signal(*_args) -> None:
        return None

    @staticmethod
    def wait(*_args) -> None:
        return None

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

    def chunks_for(self, tokens: int, topk: int) -> int:
        return 1

    def comm_stream(self):
        return torch.cuda.current_stream()

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


def _pull_combine(heap: SymmetricHeap, src_buf, plan: MoEPlan, weights, H, dtype, out=None):
    from ..ops.cuda import err_word, stream_ptr
    if out is None:
        out = torch.empty(plan.T, H, dtype=dtype, device=src_buf.device)
    rc = _lib().cm_moe_pull_combine(heap.peer_ptr_array(src_buf), heap.world, plan.dest_rank.data_ptr(),
                                    plan.dest_row.data_ptr(), None if weights is None else weights.data_ptr(),
                                    out.data_ptr(), plan.T, plan.k, H, src_buf.shape[0],
                                    err_word(src_buf.device).data_ptr(), stream_ptr())
    if rc:
        raise RuntimeError(f"cm_moe_pull_combine failed ({rc})")
    F_.count_launch("moe_pull_combine")
    return out


def _pull_rowdot(heap: SymmetricHeap, src_buf, plan: MoEPlan, dy, out=None):
    from ..ops.cuda import err_word, stream_ptr
    if out is None:
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


class _ChunkState:
    """What one token chunk of a call keeps between its pipeline stages and for the backward pass."""
    __slots__ = ("index", "tok", "f0", "plan", "xin", "yout", "h", "event")


class _FusedMoEFn(torch.autograd.Function):
    """Stages per chunk c (T = transport stream, M = the calling stream):

        forward    T: plan, push rows, signal DISPATCH[c]      M: wait DISPATCH[c], fc1 / SwiGLU / fc2, signal OUT[c]
                   T: wait OUT[c], pull + combine into y[c]
        backward   T: row-dot of dy with the owners' outputs (d probs), push weighted dy, signal GDISPATCH[c]
                   M: wait GDISPATCH[c], expert dgrad / wgrad, signal GOUT[c]      T: wait GOUT[c], pull + sum into dx[c]

    All T stages of a call are queued in chunk order, so T works on chunk c+1 while M works on chunk c.  Every T section
    starts by waiting for an event of M, hence later transport work can never overtake earlier work of the calling
    stream on a tensor both touch; M waits for T's last stage before the call returns."""

    @staticmethod
    def _chunks(bufs, layer_slot, ids, cap_total, n):
        T = ids.shape[0]
        Tc = T // n
        cap_c = (cap_total // n) // TILE * TILE
        xin_all, yout_all = bufs.bufs(layer_slot, cap_total)
        out = []
        for c in range(n):
            ch = _ChunkState()
            ch.index, ch.tok, ch.f0 = c, slice(c * Tc, (c + 1) * Tc), _flag0(layer_slot, c)
            ch.xin, ch.yout = xin_all[c * cap_c:(c + 1) * cap_c], yout_all[c * cap_c:(c + 1) * cap_c]
            ch.plan = ch.h = ch.event = None
            out.append(ch)
        return out, cap_c, xin_all, yout_all

    @staticmethod
    def forward(ctx, x, probs, w1, w2, ids, bufs: FusedMoEBuffers, layer_slot: int):
        from ..ops.cuda import swiglu_rows
        pc, heap = bufs.pc, bufs.heap
        T, H = x.shape
        cap_total = bufs.capacity_for(ids.numel())
        n = bufs.chunks_for(T, ids.shape[1])
        ep0 = bufs.next_epoch()
        chunks, cap_c, xin_all, yout_all = _FusedMoEFn._chunks(bufs, layer_slot, ids, cap_total, n)
        x = x.contiguous()
        p32 = probs.float().contiguous()
        y = torch.empty(T, H, dtype=x.dtype, device=x.device)
        fp8 = _fp8_mode(w1, w2)
        main = torch.cuda.current_stream()
        comm = bufs.comm_stream() if n > 1 else main
        has_gather = hasattr(bufs, "gather_counts")
        comm.wait_event(main.record_event())
        with torch.cuda.stream(comm):
            for ch in chunks:
                gather = (lambda cnt, c=ch.index: bufs.gather_counts(layer_slot, c, ep0, cnt)) if has_gather else None
                ch.plan = MoEPlan(ids[ch.tok], w1.shape[0] * pc.ep, pc.ep, pc.ep_rank, pc.ep_group, cap_c, gather)
                _push(heap, x[ch.tok], ch.plan, ch.xin)
                heap.signal(ch.f0 + 0, ep0)
                ch.event = comm.record_event()
        for ch in chunks:
            main.wait_event(ch.event)
            heap.wait(ch.f0 + 0, ep0)                      # every rank's rows of this chunk have landed here
            _zero_pad(ch.xin, ch.plan, cap_c)
            with torch.no_grad():
                if fp8 is not None:
                    ch.h = _experts_fwd_mx(ch.xin, w1, w2, ch.plan.tile_expert, ch.yout, fp8 == "tensorwise")
                else:
                    ch.h = _grouped(ch.xin, w1, ch.plan.tile_expert, cap_c, False)
                    a = swiglu_rows(ch.h, ch.plan.seg_offsets[-1:])      # only the rows in use of the worst-case buffer
                    _grouped(a, w2, ch.plan.tile_expert, cap_c, False, out=ch.yout)
            heap.signal(ch.f0 + 1, ep0)
            ch.event = main.record_event()
        with torch.cuda.stream(comm):
            for ch in chunks:
                comm.wait_event(ch.event)
                heap.wait(ch.f0 + 1, ep0)                  # every owner's outputs of this chunk are complete
                _pull_combine(heap, ch.yout, ch.plan, p32[ch.tok].reshape(-1), H, x.dtype, out=y[ch.tok])
            done = comm.record_event()
        main.wait_event(done)
        # xin / yout go through save_for_backward as well: activation checkpointing only drops what it sees there
        ctx.save_for_backward(w1, w2, p32, xin_all, yout_all, *[ch.h for ch in chunks])
        for ch in chunks:
            ch.h = ch.event = None
        ctx.chunks, ctx.bufs, ctx.slot, ctx.cap_c, ctx.cap_total = chunks, bufs, layer_slot, cap_c, cap_total
        ctx.x_dtype, ctx.p_dtype = x.dtype, probs.dtype
        ctx.fp8 = fp8                              # the backward runs under the recipe of its forward, whatever is set then
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.cuda import swiglu_bwd_rows, swiglu_rows
        w1, w2, p32, xin_all, yout_all, *hs = ctx.saved_tensors
        chunks, bufs, cap_c = ctx.chunks, ctx.bufs, ctx.cap_c
        heap = bufs.heap
        n = len(chunks)
        grad_in_all, grad_out_all = bufs.grad_bufs(ctx.cap_total)
        T, H = dy.shape
        dy = dy.contiguous()
        epb = bufs.next_epoch()
        E, Fh = w1.shape[0], w2.shape[2]
        dprobs = torch.empty(T, p32.shape[1], dtype=torch.float32, device=dy.device)
        dx = torch.empty(T, H, dtype=ctx.x_dtype, device=dy.device)
        main = torch.cuda.current_stream()
        comm = bufs.comm_stream() if n > 1 else main
        gin = [grad_in_all[c * cap_c:(c + 1) * cap_c] for c in range(n)]
        gout = [grad_out_all[c * cap_c:(c + 1) * cap_c] for c in range(n)]
        events = [None] * n
        comm.wait_event(main.record_event())
        with torch.cuda.stream(comm):
            for ch in chunks:
                c = ch.index
                _pull_rowdot(heap, ch.yout, ch.plan, dy[ch.tok], out=dprobs[ch.tok])
                _push(heap, dy[ch.tok], ch.plan, gin[c], scale=p32[ch.tok].reshape(-1))
                heap.signal(ch.f0 + 2, epb)
                events[c] = comm.record_event()
        dw1 = dw2 = None
        for ch in chunks:
            c, plan, h, xin = ch.index, ch.plan, hs[ch.index], ch.xin
            main.wait_event(events[c])
            heap.wait(ch.f0 + 2, epb)
            _zero_pad(gin[c], plan, cap_c)      # padding rows feed the wgrad products: 0 * stale NaN would poison them
            with torch.no_grad():
                if ctx.fp8 is not None:
                    g1, g2 = _experts_bwd_mx(gin[c], h, xin, w1, w2, plan, gout[c], ctx.fp8 == "tensorwise")
                else:
                    used = plan.seg_offsets[-1:]                                     # rows in use (device int32)
                    a = swiglu_rows(h, used)                                         # recompute a = swiglu(h)
                    da = _grouped(gin[c], w2, plan.tile_expert, cap_c, True)         # [cap, F]
                    g2 = _grouped_wgrad(gin[c], a, plan.seg_offsets, E, w2)          # [E, H, F]
                    dh = swiglu_bwd_rows(h, da, used)
                    _grouped(dh, w1, plan.tile_expert, cap_c, True, out=gout[c])     # [cap, H]
                    g1 = _grouped_wgrad(dh, xin, plan.seg_offsets, E, w1)            # [E, 2F, H]
            fused_acc = getattr(w1, "grad_added_to_main_grad", False)                # the GEMM epilogue accumulated in place
            dw1 = g1 if (dw1 is None or fused_acc) else dw1 + g1
            dw2 = g2 if (dw2 is None or getattr(w2, "grad_added_to_main_grad", False)) else dw2 + g2
            heap.signal(ch.f0 + 3, epb)
            events[c] = main.record_event()
        with torch.cuda.stream(comm):
            for ch in chunks:
                comm.wait_event(events[ch.index])
                heap.wait(ch.f0 + 3, epb)
                _pull_combine(heap, gout[ch.index], ch.plan, None, H, ctx.x_dtype, out=dx[ch.tok])
            done = comm.record_event()
        main.wait_event(done)
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
