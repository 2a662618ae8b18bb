"""Pipeline parallelism: stage layout and the 1F1B schedule over point-to-point send/recv.

Pipeline transfers stay on the library's p2p primitives (NCCL on GPUs, gloo on CPU), batched per
step so that matching sends and receives are posted together; activations are
``[micro_batch, seq(/tp under SP), hidden]`` in the model dtype, the message the reference's
schedules exchange (split rule of cppmega/recipes/run_profiles.py:308-321).
The last stage owns the MTP heads and therefore a second copy of the input embedding; the two
copies are kept identical by summing their gradients over the (first, last) stage pair.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .state import ParallelContext


def stage_layer_numbers(depth: int, pp: int, stage: int, vpp: int = 1, chunk: int = 0) -> List[int]:
    """1-indexed layers of virtual chunk ``chunk`` on pipeline stage ``stage``.  Layers are cut into
    ``pp*vpp`` near-equal consecutive chunks (earlier chunks take the remainder); chunk ``c`` of the
    model lives on stage ``c % pp`` as its ``c // pp``-th virtual chunk."""
    chunks = pp * vpp
    if chunks > depth:
        raise ValueError(f"cannot split {depth} layers into {chunks} chunks")
    base, rem = divmod(depth, chunks)
    sizes = [base + (1 if c < rem else 0) for c in range(chunks)]
    c = chunk * pp + stage
    start = sum(sizes[:c])
    return list(range(start + 1, start + sizes[c] + 1))


def schedule_1f1b(pp: int, stage: int, num_microbatches: int) -> List[tuple]:
    """Ordered list of ("F", i) / ("B", i) actions of one stage under non-interleaved 1F1B."""
    warm = min(pp - stage - 1, num_microbatches)
    steady = num_microbatches - warm
    acts: List[tuple] = [("F", i) for i in range(warm)]
    for i in range(steady):
        acts.append(("F", warm + i))
        acts.append(("B", i))
    acts += [("B", steady + i) for i in range(warm)]
    return acts


def _p2p(ops, wait: bool = True):
    """Post a batch of sends / receives as one group; ``wait=False`` returns the requests un-waited (sends: the stream
    that produced the tensor carries on; the caller keeps the tensor and the requests until :meth:`PipelineComm.drain`)."""
    if not ops:
        return []
    reqs = dist.batch_isend_irecv(ops)
    if wait:
        for r in reqs:
            r.wait()
    return reqs


class PipelineComm:
    def __init__(self, pc: ParallelContext, shape: Sequence[int], dtype: torch.dtype, device):
        self.pc, self.shape, self.dtype, self.device = pc, tuple(shape), dtype, device
        self.prev = pc.pp_ranks[pc.pp_rank - 1] if pc.pp_rank > 0 else None
        self.next = pc.pp_ranks[pc.pp_rank + 1] if pc.pp_rank < pc.pp - 1 else None
        self._pending = []                     # (requests, tensor) of sends that nobody has waited for yet

    def _buf(self):
        return torch.empty(self.shape, dtype=self.dtype, device=self.device)

    def recv_forward(self) -> Optional[torch.Tensor]:
        if self.prev is None:
            return None
        t = self._buf()
        _p2p([dist.P2POp(dist.irecv, t, self.prev)])
        return t.requires_grad_()

    def send_forward(self, t: torch.Tensor) -> None:
        """Pure sends do not hold the compute stream: the request is waited for at the end of the schedule."""
        if self.next is not None:
            t = t.detach().contiguous()
            self._pending.append((_p2p([dist.P2POp(dist.isend, t, self.next)], wait=False), t))

    def recv_backward(self) -> Optional[torch.Tensor]:
        if self.next is None:
            return None
        t = self._buf()
        _p2p([dist.P2POp(dist.irecv, t, self.next)])
        return t

    def send_backward(self, g: Optional[torch.Tensor]) -> None:
        if self.prev is not None and g is not None:
            g = g.contiguous()
            self._pending.append((_p2p([dist.P2POp(dist.isend, g, self.prev)], wait=False), g))

    def drain(self) -> None:
        for reqs, _t in self._pending:
            for r in reqs:
                r.wait()
        self._pending = []

    def send_forward_recv_backward(self, t: torch.Tensor) -> Optional[torch.Tensor]:
        if self.next is None:
            return None
        g = self._buf()
        _p2p([dist.P2POp(dist.isend, t.detach().contiguous(), self.next), dist.P2POp(dist.irecv, g, self.next)])
        return g

    def send_backward_recv_forward(self, g: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if self.prev is None:
            return None
        t = self._buf()
        _p2p([dist.P2POp(dist.isend, g.contiguous(), self.prev), dist.P2POp(dist.irecv, t, self.prev)])
        return t.requires_grad_()


def run_pipeline_schedule(trainer, microbatches: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    """Forward/backward of all micro-batches of one optimizer step under 1F1B."""
    pc: ParallelContext = trainer.pc
    model = trainer.model
    M = len(microbatches)
    mbs = [trainer._to_device(mb) for mb in microbatches]
    B, S = mbs[0]["input_ids"].shape
    s_local = S // pc.tp if pc.sequence_parallel else S
    comm = PipelineComm(pc, (B, s_local, trainer.model_cfg.hidden_size), trainer.cfg.torch_dtype(), trainer.device)
    inputs: List[Optional[torch.Tensor]] = [None] * M
    outputs: List[Optional[torch.Tensor]] = [None] * M
    stats = {"loss": None, "lm_loss": None, "mtp": None}
    acts = schedule_1f1b(pc.pp, pc.pp_rank, M)
    n_bwd_done = 0
    pending_recv_fwd: Optional[torch.Tensor] = None
    have_pending = False

    def forward(i, x_in):
        mb = mbs[i]
        if pc.is_first_pp:
            out = model(mb["input_ids"], mb["labels"] if pc.is_last_pp else None, mb.get("loss_mask"),
                        structure_inputs=mb.get("structure_inputs"))
        else:
            out = model(mb["input_ids"], mb["labels"] if pc.is_last_pp else None, mb.get("loss_mask"),
                        hidden_in=x_in, structure_inputs=mb.get("structure_inputs"))
        inputs[i] = x_in
        if pc.is_last_pp:
            outputs[i] = out["loss"] / M
            l = out["loss"].detach()
            stats["loss"] = l if stats["loss"] is None else stats["loss"] + l
            stats["lm_loss"] = out["lm_loss"] if stats["lm_loss"] is None else stats["lm_loss"] + out["lm_loss"]
            if out["mtp_losses"]:
                stats["mtp"] = out["mtp_losses"] if stats["mtp"] is None else [a + b for a, b in zip(stats["mtp"], out["mtp_losses"])]
            return None
        outputs[i] = out
        return out

    def backward(i, g_out):
        nonlocal n_bwd_done
        n_bwd_done += 1
        trainer.optimizer.set_microbatch(is_last=(n_bwd_done == M), grad_scale=1.0)
        out = outputs[i]
        if pc.is_last_pp:
            out.backward()
        else:
            torch.autograd.backward(out, grad_tensors=g_out)
        x_in = inputs[i]
        outputs[i] = inputs[i] = None
        return None if x_in is None else x_in.grad

    k = 0
    while k < len(acts):
        kind, i = acts[k]
        nxt = acts[k + 1] if k + 1 < len(acts) else None
        if kind == "F":
            x_in = pending_recv_fwd if have_pending else comm.recv_forward()
            pending_recv_fwd, have_pending = None, False
            out = forward(i, x_in)
            if nxt is not None and nxt[0] == "B" and not pc.is_last_pp:
                g = comm.send_forward_recv_backward(out)           # steady state: fused exchange
                gin = backward(nxt[1], g)
                k += 2
                after = acts[k] if k < len(acts) else None
                if after is not None and after[0] == "F" and not pc.is_first_pp:
                    pending_recv_fwd, have_pending = comm.send_backward_recv_forward(gin), True
                else:
                    comm.send_backward(gin)
                continue
            if out is not None:
                comm.send_forward(out)
            k += 1
        else:
            g = comm.recv_backward()
            gin = backward(i, g)
            after = acts[k + 1] if k + 1 < len(acts) else None
            if after is not None and after[0] == "F" and not pc.is_first_pp:
                pending_recv_fwd, have_pending = comm.send_backward_recv_forward(gin), True
            else:
                comm.send_backward(gin)
            k += 1

    comm.drain()
    sync_embedding_copies(model, pc)
    dev = trainer.device
    zero = torch.zeros((), device=dev)
    res = {"loss": (stats["loss"] / M) if stats["loss"] is not None else zero,
           "lm_loss": (stats["lm_loss"] / M) if stats["lm_loss"] is not None else zero}
    if stats["mtp"] is not None:
        res["mtp_losses"] = [m / M for m in stats["mtp"]]
    return res


def sync_embedding_copies(model, pc: ParallelContext) -> None:
    """Sum the gradients of the embedding copies held by the first stage (input) and the last
    stage (MTP heads) so both stay bit-identical after the update."""
    if pc.pp == 1 or not hasattr(model, "embedding"):
        return
    if not (pc.is_first_pp or pc.is_last_pp):
        return
    if not getattr(model.cfg.mtp, "num_layers", 0) or model.cfg.mtp.fastmtp and False:
        return
    grp = pc.embd_group
    if grp is None:
        return
    for p in model.embedding.parameters():
        g = getattr(p, "main_grad", None)
        if g is not None:
            dist.all_reduce(g, group=grp)


# ---------------------------------------------------------------------------------------------------------
# Several model chunks per rank: interleaved 1F1B (virtual pipeline) and the V-shaped DualPipeV placement
# ---------------------------------------------------------------------------------------------------------

class ChunkedModel(torch.nn.Module):
    """The model chunks held by one pipeline rank.  ``chunk_ids[i]`` is the position of ``chunks[i]`` in the global
    chain of ``total_chunks`` chunks; chunk 0 owns the embedding, the last chunk the output layer and the MTP heads.
    When one rank holds both ends (V placement) they share one embedding module, so no gradient sync is needed."""

    def __init__(self, chunks, chunk_ids, total_chunks: int):
        super().__init__()
        self.chunks = torch.nn.ModuleList(chunks)
        self.chunk_ids = list(chunk_ids)
        self.total_chunks = total_chunks
        self.cfg = chunks[0].cfg
        first = [c for c, i in zip(chunks, chunk_ids) if i == 0]
        last = [c for c, i in zip(chunks, chunk_ids) if i == total_chunks - 1]
        self.shared_embedding = False
        if first and last and first[0] is not last[0] and hasattr(last[0], "embedding"):
            last[0].embedding = first[0].embedding
            self.shared_embedding = True

    def chunk(self, chunk_id: int):
        return self.chunks[self.chunk_ids.index(chunk_id)]

    def moe_layers(self):
        out = []
        for c in self.chunks:
            out += c.moe_layers()
        return out

    def update_router_biases(self):
        for c in self.chunks:
            c.update_router_biases()

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, *a, **k):
        raise RuntimeError("a chunked model runs through run_chunked_schedule")


def build_chunked_model(cfg, pc: ParallelContext, schedule: str, **model_kwargs) -> ChunkedModel:
    """Model chunks of this rank for ``schedule`` = ``interleaved`` (chunk v*pp + stage) or ``dualpipev``
    (chunks stage and 2*pp-1-stage)."""
    from ..models.nam56r import NAM56RModel
    from . import schedules as sch
    if schedule == "interleaved":
        total = pc.pp * max(pc.config.vpp, 1)
        mine = [v * pc.pp + pc.pp_rank for v in range(max(pc.config.vpp, 1))]
    elif schedule == "dualpipev":
        if pc.ep > 1:
            raise ValueError("DualPipeV requires expert parallel size 1")
        total = 2 * pc.pp
        mine = [pc.pp_rank, 2 * pc.pp - 1 - pc.pp_rank]
    else:
        raise ValueError(f"unknown chunked schedule {schedule!r}")
    layers = sch.split_layers(cfg.depth, total)
    chunks = [NAM56RModel(cfg, pc, layer_numbers=layers[c], pre_process=(c == 0), post_process=(c == total - 1),
                          **model_kwargs) for c in mine]
    return ChunkedModel(chunks, mine, total)


def schedule_actions(schedule: str, pp: int, vpp: int, num_microbatches: int):
    """Action lists of every pipeline rank and the chunk -> rank map."""
    from . import schedules as sch
    if schedule == "interleaved":
        per_rank = [sch.interleaved_1f1b(pp, vpp, st, num_microbatches) for st in range(pp)]
        owner = lambda c: sch.chunk_owner_interleaved(c, pp)
        total = pp * vpp
    else:
        per_rank = sch.dualpipev(pp, num_microbatches)
        owner = lambda c: sch.chunk_owner_v(c, pp)
        total = 2 * pp
    sch.validate(per_rank, total, num_microbatches, owner)
    return per_rank, owner, total


def run_chunked_schedule(trainer, microbatches: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    """Execute one optimizer step of an interleaved or V-shaped schedule.

    Every rank knows every rank's action list, hence the exact order in which each peer will send to it: receives are
    posted in that order (point-to-point channels are FIFO per pair) when their tensor is first needed, sends are posted
    as results appear and not waited for until the step ends, and a chunk hand-over inside one rank (the turn of the V)
    is a plain tensor hand-off."""
    pc: ParallelContext = trainer.pc
    model: ChunkedModel = trainer.model
    M = len(microbatches)
    mbs = [trainer._to_device(mb) for mb in microbatches]
    B, S = mbs[0]["input_ids"].shape
    s_local = S // pc.tp if pc.sequence_parallel else S
    shape = (B, s_local, trainer.model_cfg.hidden_size)
    dtype, dev = trainer.cfg.torch_dtype(), trainer.device
    per_rank, owner, total = schedule_actions(trainer.cfg.pipeline_schedule, pc.pp, max(pc.config.vpp, 1), M)
    me = pc.pp_rank

    def message_of(action):
        """(key, destination stage) of the tensor an action produces for another chunk, or None."""
        kind, c, mb = action
        if kind == "F" and c < total - 1:
            return ("F", c, mb), owner(c + 1)
        if kind == "B" and c > 0:
            return ("B", c, mb), owner(c - 1)
        return None

    # Expected messages per source, in the source's own send order (a channel is FIFO).  A receive is posted when its
    # tensor is first needed, together with any earlier message of the same channel that has not been posted yet.
    # Posting everything up front is valid on a buffered transport, but an NCCL receive is a kernel that occupies its
    # stream until the matching send arrives: receives queued ahead of this rank's own compute and sends in launch order
    # can starve them (the interleaved and V-shaped schedules stopped that way on two GPUs).
    expected: Dict[int, List[tuple]] = {}
    channel_of: Dict[tuple, int] = {}
    for src in range(pc.pp):
        if src == me:
            continue
        keys = []
        for action in per_rank[src]:
            msg = message_of(action)
            if msg is not None and msg[1] == me:
                keys.append(msg[0])
                channel_of[msg[0]] = src
        expected[src] = keys
    posted: Dict[int, int] = {src: 0 for src in expected}
    recv_buf: Dict[tuple, torch.Tensor] = {}
    recv_req: Dict[tuple, object] = {}
    handoff: Dict[tuple, torch.Tensor] = {}
    send_reqs = []

    def fetch(key):
        if key in handoff:
            return handoff.pop(key)
        src = channel_of[key]
        while key not in recv_req:
            k = expected[src][posted[src]]
            posted[src] += 1
            buf = torch.empty(shape, dtype=dtype, device=dev)
            recv_buf[k] = buf
            recv_req[k] = dist.irecv(buf, src=pc.pp_ranks[src], group=pc.pp_directed.get((src, me)))
        recv_req.pop(key).wait()
        return recv_buf.pop(key)

    def deliver(action, tensor):
        msg = message_of(action)
        if msg is None:
            return
        key, dst = msg
        if dst == me:
            handoff[key] = tensor
        else:
            t = tensor.contiguous()
            send_reqs.append((dist.isend(t, dst=pc.pp_ranks[dst], group=pc.pp_directed.get((me, dst))), t))

    inputs: Dict[tuple, Optional[torch.Tensor]] = {}
    outputs: Dict[tuple, torch.Tensor] = {}
    stats = {"loss": None, "lm_loss": None, "mtp": None}
    my_actions = per_rank[me]
    n_bwd_total = sum(1 for a in my_actions if a[0] == "B")
    n_bwd = 0
    for action in my_actions:
        kind, c, mb = action
        chunk = model.chunk(c)
        batch = mbs[mb]
        if kind == "F":
            x_in = None
            if c > 0:
                x_in = fetch(("F", c - 1, mb)).detach().requires_grad_()
            labels = batch["labels"] if c == total - 1 else None
            out = chunk(batch["input_ids"], labels, batch.get("loss_mask"), hidden_in=x_in,
                        structure_inputs=batch.get("structure_inputs"))
            inputs[(c, mb)] = x_in
            if c == total - 1:
                outputs[(c, mb)] = out["loss"] / M
                l = out["loss"].detach()
                stats["loss"] = l if stats["loss"] is None else stats["loss"] + l
                stats["lm_loss"] = out["lm_loss"] if stats["lm_loss"] is None else stats["lm_loss"] + out["lm_loss"]
                if out["mtp_losses"]:
                    stats["mtp"] = (out["mtp_losses"] if stats["mtp"] is None
                                    else [a + b for a, b in zip(stats["mtp"], out["mtp_losses"])])
            else:
                outputs[(c, mb)] = out
                deliver(action, out.detach())
        else:
            n_bwd += 1
            trainer.optimizer.set_microbatch(is_last=(n_bwd == n_bwd_total), grad_scale=1.0)
            out = outputs.pop((c, mb))
            if c == total - 1:
                out.backward()
            else:
                torch.autograd.backward(out, grad_tensors=fetch(("B", c + 1, mb)))
            x_in = inputs.pop((c, mb))
            if x_in is not None:
                deliver(action, x_in.grad)
    for req, _t in send_reqs:
        req.wait()
    if not model.shared_embedding:
        for ch in model.chunks:
            if hasattr(ch, "embedding"):
                sync_embedding_copies(ch, pc)
                break
    zero = torch.zeros((), device=dev)
    res = {"loss": (stats["loss"] / M) if stats["loss"] is not None else zero,
           "lm_loss": (stats["lm_loss"] / M) if stats["lm_loss"] is not None else zero}
    if stats["mtp"] is not None:
        res["mtp_losses"] = [m / M for m in stats["mtp"]]
    return res
