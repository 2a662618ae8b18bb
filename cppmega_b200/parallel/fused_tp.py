"""Tensor-parallel linears with the sequence-parallel collectives fused into the GEMMs, over peer memory.

Two implementations of each, selected by ``FusedTP.mode`` (``"auto"``, the default, takes the staged all-gather and the
direct reduce-scatter, the faster form of each in ``tools/tp_bench.py``):

``"staged"`` - every activation shard crosses NVLink exactly once.

* ``ag_gemm``  (column-parallel forward, row-parallel dgrad):  ``y = gather_seq(x) . op(W)``.  On a second stream a copy
  kernel stores this rank's shard into slot ``me`` of every peer's gathered buffer and raises one flag per source;
  meanwhile the main stream multiplies the local shard, then each remote shard as its flag arrives (bounded waits), all
  from local memory.
* ``gemm_rs``  (row-parallel forward, column-parallel dgrad):  ``y_shard = reduce_scatter_seq(x . op(W))``.  One GEMM per
  destination shard (remote owners first) whose epilogue stores straight into the owner's staging slot, so the peer
  stores of one shard drain under the main loop of the next; after a flag barrier the owner sums its ``tp`` slots.
* weight gradients: ``dW (+)= gather_seq(a)^T b``: one launch of the token-gathering GEMM over the local slots (a
  row-parallel backward gathers ``dy`` once for dgrad and wgrad).

``"direct"`` - nothing is staged at the consumer: the GEMM's TMA producer reads each 128-row block of the gathered
operand from the peer that holds it (``ag_gemm``, ``ag_wgrad``), and one GEMM's epilogue scatters all output tiles to
their owners (``gemm_rs``).  A remote tile crosses the link once per column of output tiles that uses it, so this mode
wins only when the weight is narrow; it is kept for comparison (``tools/tp_bench.py`` times both against NCCL).

All need ``(S / tp) % 128 == 0`` (row blocks must not straddle ranks), bf16, and peer access; otherwise the NCCL
mappings in :mod:`cppmega_b200.parallel.tensor_parallel` are used.  This is the replacement for the reference's
Megatron column/row linears with ``--sequence-parallel`` (cppmega/megatron/cppmega_mamba3_tp_mixer.py:217-229,363-375)
and its TP communication overlap flags (cppmega/recipes/nam56r_nemo_recipe.py:429-443).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import functional as F_
from .symm_mem import SymmetricHeap

FLAG_AG, FLAG_AG_DONE, FLAG_RS, FLAG_RS_DONE, FLAG_GATH, FLAG_GATH_DONE = 0, 1, 2, 3, 4, 5      # this heap belongs to the TP group alone


def _lib():
    from ..ops import cuda as cu
    L = cu.lib()
    if not getattr(L, "_tp_declared", False):
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        L.cm_gemm_bf16_peer_a.argtypes = [vp, i32, i32, i32, vp, vp, i32, i32, i64, i64, i32, vp, vp]
        L.cm_gemm_bf16_peer_c.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i32, vp, vp]
        L.cm_sum_slots.argtypes = [vp, vp, i32, i64, vp]
        L.cm_gemm_bf16_peer_k.argtypes = [vp, i32, i32, i32, i32, vp, vp, i32, i32, i64, i64, i32, i32, vp, vp]
        for n in ("cm_gemm_bf16_peer_a", "cm_gemm_bf16_peer_c", "cm_sum_slots", "cm_gemm_bf16_peer_k"):
            getattr(L, n).restype = i32
        L._tp_declared = True
    return L


class FusedTP:
    """Symmetric buffers of one TP group, shared by all layers (one transfer in flight at a time per kind)."""

    def __init__(self, pc, device, max_local_rows: int, max_width: int):
        self.pc, self.device = pc, device
        self.tp = pc.tp
        self.max_elems = max_local_rows * max_width
        nbytes = self.max_elems * 2 * (1 + 2 * self.tp) + 16384
        self.heap = SymmetricHeap(pc.tp_group, pc.tp_ranks, nbytes, device)
        self.xbuf = self.heap.alloc((self.max_elems,), torch.bfloat16)                 # all-gather source ("direct" mode)
        self.stage = self.heap.alloc((self.tp * self.max_elems,), torch.bfloat16)      # reduce-scatter slots
        self.gath = self.heap.alloc((self.tp * self.max_elems,), torch.bfloat16)       # gathered shards, slot p = rank p's
        self.ag_epoch = 0
        self.rs_epoch = 0
        self.g_epoch = 0
        # "staged": every shard crosses NVLink once (pushed into the consumers' memory by a copy kernel on a second
        # stream, one flag per source) and the GEMMs read local memory, starting with this rank's own shard.
        # "direct": the GEMM's TMA loads read the peers' memory tile by tile (each remote tile crosses the link once
        # per column of output tiles that needs it); kept for comparison.
        self.mode = "auto"
        self._copy_stream = None

    def _mode(self, kind: str) -> str:
        """``kind``: "ag" (all-gather -> GEMM and the gathered weight gradients) or "rs" (GEMM -> reduce-scatter).
        "auto" takes the faster form of each, measured at TP 2 on the NAM56R projections: the staged all-gather
        (0.71 of the roofline against 0.10 for remote tile reads, which cross NVLink once per output-tile column), and
        the one-launch GEMM whose epilogue scatters to the owners (its per-shard form pays a wave of tail tiles per
        launch: 0.38 against 0.54)."""
        if self.mode == "auto":
            return "staged" if kind == "ag" else "direct"
        return self.mode

    def supported(self, batch: int, rows_per_seg: int, width_in: int, width_out: int) -> bool:
        return (rows_per_seg % 128 == 0 and batch * rows_per_seg * max(width_in, width_out) <= self.max_elems
                and width_in % 8 == 0 and width_out % 8 == 0)

    # ---- all-gather -> GEMM ------------------------------------------------------------------
    def stage_shard(self, x_local: torch.Tensor) -> torch.Tensor:
        """Copy this rank's [B, S/tp, W] shard into the symmetric buffer and meet the group; returns the staged view
        [B * S/tp, W].  Every ``stage_shard`` is closed by one ``release`` after the last kernel that reads the peers."""
        B, Sl, W = x_local.shape
        self.ag_epoch += 1
        src = self.xbuf[:B * Sl * W].view(B * Sl, W)
        self.heap.wait(FLAG_AG_DONE, self.ag_epoch - 1)          # every rank has finished reading the previous contents
        src.copy_(x_local.reshape(B * Sl, W))
        self.heap.barrier(FLAG_AG, self.ag_epoch)                # all shards are in place
        return src

    def release(self) -> None:
        self.heap.signal(FLAG_AG_DONE, self.ag_epoch)

    # ---- staged all-gather: push once, compute from local memory -----------------------------
    def _side(self):
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        return self._copy_stream

    def push_shard(self, x_local: torch.Tensor):
        """Start the all-gather of this rank's [B, S/tp, W] shard: on the second stream it is copied into slot ``me`` of
        every rank's gathered buffer (peer stores from this package's copy kernel), then flag ``FLAG_GATH`` is raised
        everywhere.  Returns ``slots``: per rank p the [B * S/tp, W] view of the LOCAL slot p; slot p may be read after
        ``wait_slot(p)``.  Close with :meth:`release_gathered` after the last kernel that reads the slots."""
        from ..ops.cuda import fast_copy_
        B, Sl, W = x_local.shape
        n = B * Sl * W
        self.g_epoch += 1
        me = self.heap.me
        slots = [self.gath[p * self.max_elems:p * self.max_elems + n].view(B * Sl, W) for p in range(self.tp)]
        x2 = x_local.reshape(B * Sl, W)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        # peers must have finished reading what the previous gather left in their slot `me`
        self.heap.wait(FLAG_GATH_DONE, self.g_epoch - 1)
        ev = torch.cuda.Event()
        ev.record()
        side = self._side()
        side.wait_event(ev)
        with torch.cuda.stream(side):
            for q in range(1, self.tp):
                p = (me + q) % self.tp
                fast_copy_(self.heap.peer_tensor(slots[me], p), x2)
            self.heap.signal(FLAG_GATH, self.g_epoch)
        x2.record_stream(side)
        return slots, x2

    def wait_slot(self, p: int) -> None:
        self.heap.wait_one(FLAG_GATH, p, self.g_epoch)

    def release_gathered(self) -> None:
        self.heap.signal(FLAG_GATH_DONE, self.g_epoch)

    def _ag_gemm_staged(self, x_local, w, b_mn: bool, keep: bool):
        from ..ops.cuda import gemm
        B, Sl, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        slots, x2 = self.push_shard(x_local)
        out = torch.empty(B, self.tp * Sl, N, dtype=torch.bfloat16, device=x_local.device)
        me = self.heap.me
        for q in range(self.tp):
            p = (me + q) % self.tp                       # own shard first: its product hides the transfers
            if q:
                self.wait_slot(p)
            src = x2 if q == 0 else slots[p]
            for b in range(B):
                gemm(src[b * Sl:(b + 1) * Sl], w, b_mn=b_mn, out=out[b, p * Sl:(p + 1) * Sl])
        if not keep:
            self.release_gathered()
        F_.count_launch("tp_ag_gemm")
        return out, (slots, x2)

    def _wgrad_staged(self, gathered, batch: int, local: torch.Tensor, peer_is_a: bool, out, accumulate: bool, out_shape):
        """``out [M, N] (+)= A^T B`` over all tokens with one operand gathered: one launch of the token-gathering
        kernel whose per-rank operand pointers are this rank's LOCAL slots (and its own shard), so it reads no peer."""
        from ..ops.cuda import err_word, stream_ptr
        slots, x2 = gathered
        M, N = out_shape
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=local.device)
            accumulate = False
        assert local.stride(1) == 1 and out.is_contiguous() and out.dtype in (torch.bfloat16, torch.float32)
        me = self.heap.me
        self.heap.wait(FLAG_GATH, self.g_epoch)                  # all shards have landed (usually long ago)
        ptrs = (ctypes.c_void_p * self.tp)(*[(x2 if p == me else slots[p]).data_ptr() for p in range(self.tp)])
        rc = _lib().cm_gemm_bf16_peer_k(ptrs, self.tp, x2.shape[0] // batch, batch, int(peer_is_a),
                                        local.data_ptr(), out.data_ptr(), M, N, local.stride(0), N,
                                        int(out.dtype == torch.float32), int(accumulate), err_word(self.device).data_ptr(),
                                        stream_ptr())
        if rc:
            raise RuntimeError(f"cm_gemm_bf16_peer_k failed ({rc})")
        F_.count_launch("tp_ag_wgrad")
        return out

    def _gemm_rs_staged(self, x: torch.Tensor, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """Per destination shard: this rank's partial product is stored by the GEMM epilogue straight into slot ``me`` of
        the owner's staging area (plain peer stores that drain under the next shard's main loop); the owner sums."""
        from ..ops.cuda import gemm, stream_ptr
        B, S, K = x.shape
        Sl = S // self.tp
        N = w.shape[1] if b_mn else w.shape[0]
        self.rs_epoch += 1
        me = self.heap.me
        n_local = B * Sl * N
        stage = self.stage[:self.tp * n_local]
        my_slot = stage[me * n_local:(me + 1) * n_local].view(B, Sl, N)
        self.heap.wait(FLAG_RS_DONE, self.rs_epoch - 1)          # owners have consumed the previous slots
        for q in range(1, self.tp + 1):
            p = (me + q) % self.tp                       # remote owners first, this rank's own shard last
            dst = self.heap.peer_tensor(my_slot, p)
            for b in range(B):
                gemm(x[b, p * Sl:(p + 1) * Sl], w, b_mn=b_mn, out=dst[b])
        self.heap.barrier(FLAG_RS, self.rs_epoch)                # every rank's partial tiles have landed here
        out = torch.empty(B, Sl, N, dtype=torch.bfloat16, device=x.device)
        rc = _lib().cm_sum_slots(stage.data_ptr(), out.data_ptr(), self.tp, n_local, stream_ptr())
        if rc:
            raise RuntimeError(f"cm_sum_slots failed ({rc})")
        self.heap.signal(FLAG_RS_DONE, self.rs_epoch)
        F_.count_launch("tp_gemm_rs")
        return out

    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool, keep_staged: bool = False) -> torch.Tensor:
        """x_local [B, S/tp, K] bf16 -> [B, S, N];  w is [N, K] (b_mn False) or [K, N] (b_mn True)."""
        from ..ops.cuda import err_word, stream_ptr
        if self._mode("ag") == "staged":
            out, self._last_gathered = self._ag_gemm_staged(x_local, w, b_mn, keep_staged)
            return out
        B, Sl, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        src = self.stage_shard(x_local)
        out = torch.empty(B, self.tp * Sl, N, dtype=torch.bfloat16, device=x_local.device)
        rc = _lib().cm_gemm_bf16_peer_a(self.heap.peer_ptr_array(src), self.tp, Sl, B, w.data_ptr(), out.data_ptr(), N, K,
                                        w.stride(0), N, int(b_mn), err_word(self.device).data_ptr(), stream_ptr())
        if rc:
            raise RuntimeError(f"cm_gemm_bf16_peer_a failed ({rc})")
        if not keep_staged:
            self.release()
        F_.count_launch("tp_ag_gemm")
        return out

    def ag_wgrad(self, staged: torch.Tensor, batch: int, local: torch.Tensor, peer_is_a: bool, out: Optional[torch.Tensor],
                 accumulate: bool, out_shape) -> torch.Tensor:
        """``out [M, N] (+)= A^T B`` over all tokens, where the staged operand ([B * S/tp, W] per rank) is A when
        ``peer_is_a`` (then ``local`` is B [B * S, N]) and B otherwise (``local`` is A [B * S, M])."""
        from ..ops.cuda import err_word, stream_ptr
        M, N = out_shape
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=local.device)
            accumulate = False
        assert local.stride(1) == 1 and out.is_contiguous() and out.dtype in (torch.bfloat16, torch.float32)
        rc = _lib().cm_gemm_bf16_peer_k(self.heap.peer_ptr_array(staged), self.tp, staged.shape[0] // batch, batch, int(peer_is_a),
                                        local.data_ptr(), out.data_ptr(), M, N, local.stride(0), N,
                                        int(out.dtype == torch.float32), int(accumulate), err_word(self.device).data_ptr(),
                                        stream_ptr())
        if rc:
            raise RuntimeError(f"cm_gemm_bf16_peer_k failed ({rc})")
        F_.count_launch("tp_ag_wgrad")
        return out

    # ---- GEMM -> reduce-scatter --------------------------------------------------------------
    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """x [B, S, K] bf16 (K = this rank's slice of the reduction) -> [B, S/tp, N] summed over the TP group."""
        from ..ops.cuda import err_word, stream_ptr
        if self._mode("rs") == "staged":
            return self._gemm_rs_staged(x if x.is_contiguous() else x.contiguous(), w, b_mn)
        B, S, K = x.shape
        Sl = S // self.tp
        N = w.shape[1] if b_mn else w.shape[0]
        self.rs_epoch += 1
        x2 = x.reshape(B * S, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        n_local = B * Sl * N
        stage = self.stage[:self.tp * n_local]
        self.heap.wait(FLAG_RS_DONE, self.rs_epoch - 1)          # owners have consumed the previous slots
        rc = _lib().cm_gemm_bf16_peer_c(x2.data_ptr(), w.data_ptr(), self.heap.peer_ptr_array(stage), self.tp, self.heap.me,
                                        Sl, B, N, K, x2.stride(0), w.stride(0), int(b_mn),
                                        err_word(self.device).data_ptr(), stream_ptr())
        if rc:
            raise RuntimeError(f"cm_gemm_bf16_peer_c failed ({rc})")
        self.heap.barrier(FLAG_RS, self.rs_epoch)                # every rank's partial tiles have landed here
        out = torch.empty(B, Sl, N, dtype=torch.bfloat16, device=x.device)
        rc = _lib().cm_sum_slots(stage.data_ptr(), out.data_ptr(), self.tp, n_local, stream_ptr())
        if rc:
            raise RuntimeError(f"cm_sum_slots failed ({rc})")
        self.heap.signal(FLAG_RS_DONE, self.rs_epoch)
        F_.count_launch("tp_gemm_rs")
        return out


_STATE: Optional[FusedTP] = None


def install(pc, device, max_local_rows: int, max_width: int) -> Optional[FusedTP]:
    """Create the TP buffers (collective over the TP group).  Returns None when the topology does not allow it."""
    global _STATE
    from .symm_mem import peer_access_available
    if pc.tp <= 1 or not pc.sequence_parallel or not peer_access_available(pc):
        _STATE = None
        return None
    _STATE = FusedTP(pc, device, max_local_rows, max_width)
    return _STATE


def uninstall() -> None:
    global _STATE
    _STATE = None


def current() -> Optional[FusedTP]:
    return _STATE


class ColumnLinearSPFn(torch.autograd.Function):
    """y = gather_seq(x) W^T with W [N_local, K]."""

    @staticmethod
    def forward(ctx, x_local, w, tp: FusedTP):
        ctx.tp = tp
        ctx.save_for_backward(x_local, w)
        return tp.ag_gemm(x_local, w, b_mn=False)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.cuda import wgrad_into_main_grad
        x_local, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = tp.gemm_rs(dy, w, b_mn=True)                                   # [B,S,N_l] . W[N_l,K] -> scatter
        if ctx.needs_input_grad[1]:
            dy2 = dy.reshape(-1, dy.shape[-1])                                   # [T, N_l]: the local operand A
            if tp._mode("ag") == "staged":
                gathered = tp.push_shard(x_local)                                # gather(x) again: operand B, from local slots
                dw = wgrad_into_main_grad(w, lambda out, acc: tp._wgrad_staged(gathered, x_local.shape[0], dy2, False, out, acc,
                                                                               tuple(w.shape)))
                tp.release_gathered()
            else:
                staged = tp.stage_shard(x_local)                                 # gather(x) is operand B, read from the peers
                dw = wgrad_into_main_grad(w, lambda out, acc: tp.ag_wgrad(staged, x_local.shape[0], dy2, False, out, acc, tuple(w.shape)))
                tp.release()
        return dx, dw, None


class RowLinearSPFn(torch.autograd.Function):
    """y_shard = reduce_scatter_seq(x W^T) with W [N, K_local]."""

    @staticmethod
    def forward(ctx, x, w, tp: FusedTP):
        ctx.tp = tp
        ctx.save_for_backward(x, w)
        return tp.gemm_rs(x, w, b_mn=False)

    @staticmethod
    def backward(ctx, dy_local):
        from ..ops.cuda import wgrad_into_main_grad
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy_local = dy_local.contiguous()
        dx = dw = None
        need_dw = ctx.needs_input_grad[1]
        staged = None
        if tp._mode("ag") == "staged":
            gathered = None
            if ctx.needs_input_grad[0]:
                dx = tp.ag_gemm(dy_local, w, b_mn=True, keep_staged=need_dw)    # gather(dy)[B,S,N] . W[N,K_l]
                gathered = tp._last_gathered
            if need_dw:
                if gathered is None:
                    gathered = tp.push_shard(dy_local)
                x2 = x.reshape(-1, x.shape[-1])
                if not x2.is_contiguous():
                    x2 = x2.contiguous()
                dw = wgrad_into_main_grad(w, lambda out, acc: tp._wgrad_staged(gathered, dy_local.shape[0], x2, True, out, acc,
                                                                               tuple(w.shape)))
                tp.release_gathered()                                            # one gather of dy served dgrad and wgrad
            return dx, dw, None
        if ctx.needs_input_grad[0]:
            dx = tp.ag_gemm(dy_local, w, b_mn=True, keep_staged=need_dw)        # gather(dy)[B,S,N] . W[N,K_l]
            if need_dw:
                staged = tp.xbuf[:dy_local.numel()].view(-1, dy_local.shape[-1])
        if need_dw:
            if staged is None:
                staged = tp.stage_shard(dy_local)
            x2 = x.reshape(-1, x.shape[-1])                                      # [T, K_l]: the local operand B
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            dw = wgrad_into_main_grad(w, lambda out, acc: tp.ag_wgrad(staged, dy_local.shape[0], x2, True, out, acc, tuple(w.shape)))
            tp.release()                                                         # one staging of dy served dgrad and wgrad
        return dx, dw, None


def column_linear(x_local: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
    tp = _STATE
    if (tp is None or x_local.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x_local.dim() != 3
            or not tp.supported(x_local.shape[0], x_local.shape[1], x_local.shape[2], w.shape[0])):
        return None
    return ColumnLinearSPFn.apply(x_local.contiguous(), w, tp)


def row_linear(x: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
    tp = _STATE
    if (tp is None or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 3 or x.shape[1] % tp.tp
            or not tp.supported(x.shape[0], x.shape[1] // tp.tp, x.shape[2], w.shape[0])):
        return None
    return RowLinearSPFn.apply(x, w, tp)
