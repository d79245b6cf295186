"""Failure detection for multi-rank jobs: host-side heartbeats and collective time-outs.

The reference has no failure handling beyond a final rendezvous and checkpoint rotation (train.py:237,
280-281).  Here every device-side wait is bounded and reports through a status word (`ops/csrc/common.cuh`),
and on the host:

  * `Heartbeat`: each rank writes a monotonically increasing counter to a `torch.distributed` store from a
    daemon thread; `dead_ranks()` lists peers whose counter stopped for longer than `timeout_s`.  Ranks poll it
    between steps, i.e. with no kernel or collective of their own in flight, and raise `RankFailure` before
    launching work that would wait on a dead peer.
  * `guarded_collective`: runs a collective under the process group's time-out and converts the backend error
    into `RankFailure`.
  * `skip_step_on_nonfinite`: NaN/Inf gradients make the optimizer skip the step instead of poisoning weights.
Recovery is restart-from-checkpoint (`train.py --resume`); `parallel/checkpoint.py` only ever publishes complete
checkpoints.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


class RankFailure(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, period_s: float = 0.5, timeout_s: float = 5.0,
                 prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.period, self.timeout, self.prefix = period_s, timeout_s, prefix
        self._stop = threading.Event()
        self._beat = 0
        self._last_seen = {}
        self._thread = threading.Thread(target=self._run, daemon=True)

    def start(self) -> "Heartbeat":
        self._tick()
        self._thread.start()
        return self

    def _tick(self):
        self._beat += 1
        self.store.set(f"{self.prefix}/{self.rank}", str(self._beat))

    def _run(self):
        while not self._stop.wait(self.period):
            try:
                self._tick()
            except Exception:
                return

    def stop(self):
        self._stop.set()

    def dead_ranks(self) -> List[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = int(self.store.get(f"{self.prefix}/{r}").decode())
            except Exception:
                val = -1
            last = self._last_seen.get(r)
            if last is None or last[0] != val:
                self._last_seen[r] = (val, now)
            elif now - last[1] > self.timeout:
                dead.append(r)
        return dead

    def check(self) -> None:
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(f"rank(s) {dead} stopped sending heartbeats for more than {self.timeout}s")


def guarded_collective(fn: Callable, *args, **kwargs):
    """Run a collective; a backend time-out or abort surfaces as RankFailure."""
    try:
        return fn(*args, **kwargs)
    except (RuntimeError, dist.DistBackendError) as e:  # type: ignore[attr-defined]
        raise RankFailure(f"collective failed: {e}") from e


def skip_step_on_nonfinite(optimizer, loss: Optional[torch.Tensor] = None) -> bool:
    """Returns True (and clears gradients) if the loss or the gradient norm is not finite."""
    bad = loss is not None and not torch.isfinite(loss.detach()).all()
    flat = getattr(optimizer, "flat_grads", None)
    if not bad and flat is not None:
        bad = not torch.isfinite(flat.float().sum())
    if bad:
        optimizer.zero_grad()
        if flat is not None:
            flat.zero_()
    return bool(bad)
