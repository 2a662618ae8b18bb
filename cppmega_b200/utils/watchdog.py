"""Failure detection on the host: a per-step timeout watchdog and a store-based rank heartbeat.

The reference has no elasticity and diagnoses failures after the fact (NaN checks disabled,
scripts/remote_smoke_h200_dsa_9_4_m.sh:732; bisect scripts).  Here:

* :class:`StepWatchdog` - a daemon thread that raises the alarm (callback, default: dump stacks and
  ``os._exit(86)``) when ``beat()`` has not been called for ``timeout_s``.  A hung collective or a stuck
  kernel wait therefore ends the process instead of blocking the job.
* :class:`RankHeartbeat` - every rank writes ``hb/<rank> = step, time`` into a ``torch.distributed`` store;
  ``dead_ranks()`` lists ranks whose heartbeat is older than the limit, so the survivors learn about a lost
  peer on the host before their next launch and can stop at a step boundary and resume from the last
  checkpoint.

Nothing here touches the GPU; the tests run on CPU with gloo ranks and a rank that stops on purpose.
"""
from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time
from typing import Callable, Dict, List, Optional


class StepWatchdog:
    def __init__(self, timeout_s: float, rank: int = 0, on_timeout: Optional[Callable[[float, int], None]] = None,
                 poll_s: float = 0.5):
        self.timeout_s, self.rank, self.poll_s = float(timeout_s), rank, poll_s
        self.on_timeout = on_timeout or self._default_action
        self._last = time.monotonic()
        self._step = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.fired = False

    def _default_action(self, idle_s: float, step: int) -> None:
        sys.stderr.write(f"[watchdog] rank {self.rank}: no progress for {idle_s:.1f}s after step {step}; aborting\n")
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        sys.stderr.flush()
        os._exit(86)

    def start(self) -> "StepWatchdog":
        self._last = time.monotonic()
        self._thread = threading.Thread(target=self._run, daemon=True, name="cppmega-watchdog")
        self._thread.start()
        return self

    def beat(self, step: int) -> None:
        self._step = step
        self._last = time.monotonic()

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            idle = time.monotonic() - self._last
            if idle > self.timeout_s:
                self.fired = True
                self.on_timeout(idle, self._step)
                return

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.poll_s + 1)


class RankHeartbeat:
    def __init__(self, store, rank: int, world: int, limit_s: float = 30.0, clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world, self.limit_s, self.clock = store, rank, world, limit_s, clock

    def beat(self, step: int) -> None:
        self.store.set(f"hb/{self.rank}", f"{step},{self.clock():.3f}")

    def snapshot(self) -> Dict[int, Optional[tuple]]:
        out: Dict[int, Optional[tuple]] = {}
        for r in range(self.world):
            try:
                if hasattr(self.store, "check") and not self.store.check([f"hb/{r}"]):
                    out[r] = None
                    continue
                raw = self.store.get(f"hb/{r}")
                s = raw.decode() if isinstance(raw, bytes) else str(raw)
                step, t = s.split(",")
                out[r] = (int(step), float(t))
            except Exception:
                out[r] = None
        return out

    def dead_ranks(self) -> List[int]:
        now = self.clock()
        dead = []
        for r, v in self.snapshot().items():
            if r == self.rank:
                continue
            if v is None or now - v[1] > self.limit_s:
                dead.append(r)
        return dead

    def lagging_ranks(self, max_lag_steps: int = 1) -> List[int]:
        snap = self.snapshot()
        mine = snap.get(self.rank)
        if mine is None:
            return []
        return [r for r, v in snap.items() if v is not None and mine[0] - v[0] > max_lag_steps]


class DictStore:
    """In-process stand-in for a distributed store (tests, single-process runs)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k: str, v) -> None:
        with self._lock:
            self._d[k] = v.encode() if isinstance(v, str) else bytes(v)

    def get(self, k: str) -> bytes:
        with self._lock:
            return self._d[k]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)

    def delete_key(self, k: str) -> bool:
        with self._lock:
            return self._d.pop(k, None) is not None
