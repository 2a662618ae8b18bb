"""Pipeline schedule generators and the MoE communication-overlap plan.

Everything here is pure scheduling logic (lists of actions and dependency graphs) so that it can be checked
exhaustively on a CPU; the executors consume these lists.

* :func:`interleaved_1f1b` - per-stage action order for PP x VPP (virtual chunks), the launcher topology of the
  reference (PP=2, VPP=2; cppmega/recipes/run_profiles.py:308-321 for the layer split).
* :func:`dualpipev` - the V-shaped bidirectional schedule: ``2*pp`` model chunks, rank ``r`` holds chunks ``r`` and
  ``2*pp-1-r`` (rank 0: chunks 0 and 3 of a 2-rank pipe, rank 1: chunks 1 and 2), forward of one micro-batch
  overlapped with backward of another on the same rank (cppmega/megatron/dualpipev_schedule.py:114-377).  As in the
  reference it is restricted to EP = 1: with EP > 1 the expert all-to-alls of the two directions would interleave
  differently on different ranks.
* :func:`validate` - simulates a set of per-rank action lists and proves that every dependency (forward of chunk
  c needs forward of chunk c-1 of the same micro-batch, backward needs the forward and the backward of chunk c+1)
  is met without deadlock; returns the makespan in unit steps and the peak number of live activations per rank.
* :class:`LayerOverlapPlan` - the combined-1F1B expert-parallel overlap plan for a hybrid stack: sequence mixers
  (Mamba, M2RNN, DSA/MLA) are opaque compute nodes, MoE layers are split into router / dispatch / experts / combine
  nodes assigned to a compute and a communication stream so that the dispatch/combine of micro-batch *i* overlap
  compute of micro-batch *i+1* (cppmega/megatron/hybrid_schedule_plan.py:51-105 node types, :112-240 plan).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

Action = Tuple[str, int, int]          # ("F" | "B", chunk, micro-batch)


# ---------------------------------------------------------------------------
# chunk placement
# ---------------------------------------------------------------------------

def chunk_owner_interleaved(chunk: int, pp: int) -> int:
    return chunk % pp


def chunk_owner_v(chunk: int, pp: int) -> int:
    """V placement: chunks 0..pp-1 go down the ranks, chunks pp..2pp-1 come back up."""
    return chunk if chunk < pp else 2 * pp - 1 - chunk


def split_layers(depth: int, chunks: int) -> List[List[int]]:
    """1-indexed layers per chunk, near-equal consecutive pieces (earlier chunks take the remainder)."""
    if chunks > depth:
        raise ValueError(f"cannot split {depth} layers into {chunks} chunks")
    base, rem = divmod(depth, chunks)
    out, start = [], 1
    for c in range(chunks):
        n = base + (1 if c < rem else 0)
        out.append(list(range(start, start + n)))
        start += n
    return out


# ---------------------------------------------------------------------------
# interleaved 1F1B
# ---------------------------------------------------------------------------

def interleaved_1f1b(pp: int, vpp: int, stage: int, num_microbatches: int) -> List[Action]:
    """Megatron-style interleaved schedule for one stage.  Micro-batches advance in groups of ``pp``; virtual
    chunk ``v`` of this stage is model chunk ``v*pp + stage``.  ``num_microbatches`` must be a multiple of ``pp``
    when ``vpp > 1``."""
    if vpp == 1:
        warm = min(pp - stage - 1, num_microbatches)
        acts: List[Action] = [("F", stage, i) for i in range(warm)]
        for i in range(num_microbatches - warm):
            acts += [("F", stage, warm + i), ("B", stage, i)]
        acts += [("B", stage, num_microbatches - warm + i) for i in range(warm)]
        return acts
    if num_microbatches % pp:
        raise ValueError("interleaved schedule needs num_microbatches divisible by the pipeline size")
    total = num_microbatches * vpp

    def fwd_item(k: int) -> Tuple[int, int]:       # k-th forward of this stage -> (virtual chunk, micro-batch)
        group, within = divmod(k, pp * vpp)
        v, j = divmod(within, pp)
        return v, group * pp + j

    def bwd_item(k: int) -> Tuple[int, int]:
        group, within = divmod(k, pp * vpp)
        v, j = divmod(within, pp)
        return vpp - 1 - v, group * pp + j

    warm = min((pp - stage - 1) * 2 + (vpp - 1) * pp, total)
    acts = []
    for k in range(warm):
        v, mb = fwd_item(k)
        acts.append(("F", v * pp + stage, mb))
    for k in range(total - warm):
        v, mb = fwd_item(warm + k)
        acts.append(("F", v * pp + stage, mb))
        v, mb = bwd_item(k)
        acts.append(("B", v * pp + stage, mb))
    for k in range(total - warm, total):
        v, mb = bwd_item(k)
        acts.append(("B", v * pp + stage, mb))
    return acts


# ---------------------------------------------------------------------------
# DualPipeV
# ---------------------------------------------------------------------------

def dualpipev(pp: int, num_microbatches: int, ep: int = 1) -> List[List[Action]]:
    """Per-rank action lists of the V schedule (``2*pp`` chunks).  Built greedily: at every unit step each rank
    runs the ready action that is furthest along (backward before forward, later chunk first), holding at most
    ``2*pp`` forward activations.  The result is checked by :func:`validate` before it is returned."""
    if ep != 1:
        raise ValueError("DualPipeV requires expert parallel size 1: the two directions would order the expert "
                         "all-to-alls differently on different ranks")
    if num_microbatches < 2 * pp:
        raise ValueError(f"DualPipeV needs at least {2 * pp} micro-batches for {pp} ranks")
    chunks = 2 * pp
    done_f: Dict[Tuple[int, int], int] = {}
    done_b: Dict[Tuple[int, int], int] = {}
    acts: List[List[Action]] = [[] for _ in range(pp)]
    live = [0] * pp
    cap = 2 * pp
    step = 0
    total = 2 * chunks * num_microbatches
    count = 0
    while count < total:
        step += 1
        if step > 8 * total + 64:
            raise RuntimeError("DualPipeV generation did not converge")
        chosen: List[Optional[Action]] = [None] * pp
        for r in range(pp):
            mine = [c for c in range(chunks) if chunk_owner_v(c, pp) == r]
            best = None
            for c in sorted(mine, reverse=True):                      # backward first, later chunk first
                for mb in range(num_microbatches):
                    if (c, mb) in done_b or (c, mb) not in done_f or done_f[(c, mb)] >= step:
                        continue
                    if c < chunks - 1 and ((c + 1, mb) not in done_b or done_b[(c + 1, mb)] >= step):
                        continue
                    best = ("B", c, mb)
                    break
                if best:
                    break
            if best is None and live[r] < cap:
                for c in sorted(mine, reverse=True):
                    for mb in range(num_microbatches):
                        if (c, mb) in done_f:
                            continue
                        if c > 0 and ((c - 1, mb) not in done_f or done_f[(c - 1, mb)] >= step):
                            continue
                        best = ("F", c, mb)
                        break
                    if best:
                        break
            chosen[r] = best
        for r, a in enumerate(chosen):
            if a is None:
                continue
            kind, c, mb = a
            if kind == "F":
                done_f[(c, mb)] = step
                live[r] += 1
            else:
                done_b[(c, mb)] = step
                live[r] -= 1
            acts[r].append(a)
            count += 1
    validate(acts, chunks, num_microbatches, lambda c: chunk_owner_v(c, pp))
    return acts


# ---------------------------------------------------------------------------
# validation by simulation
# ---------------------------------------------------------------------------

@dataclass
class ScheduleReport:
    makespan: int
    peak_live: List[int]
    bubble_fraction: float


def validate(per_rank: Sequence[Sequence[Action]], chunks: int, num_microbatches: int, owner) -> ScheduleReport:
    """Simulate in unit steps (forward and backward of a chunk cost one step each; a result is visible to other
    ranks from the next step).  Raises ``ValueError`` on a missing / duplicated action, a wrong owner or a
    deadlock."""
    n = len(per_rank)
    seen = set()
    for r, acts in enumerate(per_rank):
        for a in acts:
            kind, c, mb = a
            if owner(c) != r:
                raise ValueError(f"rank {r} schedules chunk {c} owned by rank {owner(c)}")
            if a in seen:
                raise ValueError(f"duplicate action {a}")
            seen.add(a)
    want = {(k, c, mb) for k in "FB" for c in range(chunks) for mb in range(num_microbatches)}
    if seen != want:
        raise ValueError(f"schedule misses {sorted(want - seen)[:4]} / has extra {sorted(seen - want)[:4]}")
    pos = [0] * n
    done: Dict[Action, int] = {}
    live = [0] * n
    peak = [0] * n
    step = 0
    remaining = len(want)
    while remaining:
        step += 1
        progressed = False
        fired: List[Tuple[int, Action]] = []
        for r in range(n):
            if pos[r] >= len(per_rank[r]):
                continue
            kind, c, mb = a = per_rank[r][pos[r]]
            if kind == "F":
                ok = c == 0 or done.get(("F", c - 1, mb), step) < step
            else:
                ok = done.get(("F", c, mb), step) < step and (c == chunks - 1 or done.get(("B", c + 1, mb), step) < step)
            if ok:
                fired.append((r, a))
        for r, a in fired:
            done[a] = step
            pos[r] += 1
            live[r] += 1 if a[0] == "F" else -1
            peak[r] = max(peak[r], live[r])
            remaining -= 1
            progressed = True
        if not progressed:
            stuck = {r: per_rank[r][pos[r]] for r in range(n) if pos[r] < len(per_rank[r])}
            raise ValueError(f"deadlock at step {step}: waiting on {stuck}")
    work = len(want) / n
    return ScheduleReport(step, peak, 1.0 - work / step)


# ---------------------------------------------------------------------------
# MoE communication-overlap plan
# ---------------------------------------------------------------------------

@dataclass
class PlanNode:
    name: str
    layer: int
    kind: str                  # "opaque" | "router" | "dispatch" | "experts" | "combine" | "pre" | "post"
    stream: str                # "comp" | "comm"
    deps: List[int] = field(default_factory=list)


@dataclass
class LayerOverlapPlan:
    """Forward node graph of one model chunk for one micro-batch."""

    nodes: List[PlanNode]

    @classmethod
    def from_layer_kinds(cls, kinds: Sequence[str], first_layer: int = 1, pre: bool = False, post: bool = False,
                         overlap: bool = True) -> "LayerOverlapPlan":
        """``kinds``: one of ``M`` (Mamba), ``R`` (M2RNN), ``A`` (attention), ``E`` (MoE) per layer."""
        nodes: List[PlanNode] = []

        def add(name, layer, kind, stream, deps):
            nodes.append(PlanNode(name, layer, kind, stream, list(deps)))
            return len(nodes) - 1

        last = []
        if pre:
            last = [add("embedding", 0, "pre", "comp", [])]
        for i, k in enumerate(kinds):
            L = first_layer + i
            if k != "E":
                last = [add(f"L{L}.{k}", L, "opaque", "comp", last)]
                continue
            comm = "comm" if overlap else "comp"
            r = add(f"L{L}.router", L, "router", "comp", last)
            d = add(f"L{L}.dispatch", L, "dispatch", comm, [r])
            s = add(f"L{L}.shared", L, "opaque", "comp", [r])           # shared expert overlaps the dispatch
            e = add(f"L{L}.experts", L, "experts", "comp", [d])
            c = add(f"L{L}.combine", L, "combine", comm, [e])
            last = [c, s]
        if post:
            add("loss", first_layer + len(kinds), "post", "comp", last)
        return cls(nodes)

    def stream_order(self) -> Dict[str, List[int]]:
        order: Dict[str, List[int]] = {"comp": [], "comm": []}
        for i, n in enumerate(self.nodes):
            order[n.stream].append(i)
        return order

    def critical_path(self, cost: Dict[str, float]) -> float:
        """Length of the longest dependency + stream-order chain, with ``cost[kind]`` per node."""
        finish: List[float] = [0.0] * len(self.nodes)
        stream_free = {"comp": 0.0, "comm": 0.0}
        for i, n in enumerate(self.nodes):
            start = max([stream_free[n.stream]] + [finish[d] for d in n.deps])
            finish[i] = start + cost.get(n.kind, 0.0)
            stream_free[n.stream] = finish[i]
        return max(finish) if finish else 0.0


def interleave_microbatches(plan: LayerOverlapPlan, cost: Dict[str, float], num_microbatches: int = 2) -> float:
    """Makespan of ``num_microbatches`` copies of ``plan`` issued round-robin node by node on two streams: the
    combined-1F1B idea that one micro-batch's all-to-all hides behind another's compute."""
    n = len(plan.nodes)
    finish = [[0.0] * n for _ in range(num_microbatches)]
    stream_free = {"comp": 0.0, "comm": 0.0}
    for i, node in enumerate(plan.nodes):
        for mb in range(num_microbatches):
            start = max([stream_free[node.stream]] + [finish[mb][d] for d in node.deps])
            finish[mb][i] = start + cost.get(node.kind, 0.0)
            stream_free[node.stream] = finish[mb][i]
    return max(max(f) for f in finish) if n else 0.0
