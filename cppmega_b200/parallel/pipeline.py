"""Pipeline parallelism: stage layout and the 1F1B schedule over point-to-point send/recv.

Pipeline transfers stay on the library's p2p primitives (NCCL on GPUs, gloo on CPU), batched per
step so that matching sends and receives are posted together; activations are
``[micro_batch, seq(/tp under SP), hidden]`` in the model dtype, the message the reference's
schedules exchange (SURVEY collective C13; split rule of cppmega/recipes/run_profiles.py:308-321).
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


def _p2p(ops):
    if not ops:
        return
    for r in dist.batch_isend_irecv(ops):
        r.wait()


class PipelineComm:
    def __init__(self, pc: ParallelContext, shape: Sequence[int], dtype: torch.dtype, device):
        self.pc, self.shape, self.dtype, self.device = pc, tuple(shape), dtype, device
        self.prev = pc.pp_ranks[pc.pp_rank - 1] if pc.pp_rank > 0 else None
        self.next = pc.pp_ranks[pc.pp_rank + 1] if pc.pp_rank < pc.pp - 1 else None

    def _buf(self):
        return torch.empty(self.shape, dtype=self.dtype, device=self.device)

    def recv_forward(self) -> Optional[torch.Tensor]:
        if self.prev is None:
            return None
        t = self._buf()
        _p2p([dist.P2POp(dist.irecv, t, self.prev)])
        return t.requires_grad_()

    def send_forward(self, t: torch.Tensor) -> None:
        if self.next is not None:
            _p2p([dist.P2POp(dist.isend, t.detach().contiguous(), self.next)])

    def recv_backward(self) -> Optional[torch.Tensor]:
        if self.next is None:
            return None
        t = self._buf()
        _p2p([dist.P2POp(dist.irecv, t, self.next)])
        return t

    def send_backward(self, g: Optional[torch.Tensor]) -> None:
        if self.prev is not None and g is not None:
            _p2p([dist.P2POp(dist.isend, g.contiguous(), self.prev)])

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
