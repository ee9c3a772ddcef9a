"""Host-side failure detection: a per-rank heartbeat in the job's key-value store.

Every rank publishes `hb/<rank> = (iteration, wall-clock)` before each step and a daemon thread
checks that no peer's heartbeat is older than `timeout_s`.  When one is, the watchdog records
which rank went quiet; the training loop calls `raise_if_failed()` between steps — before its
next launch — so a rank never enters a collective that a dead peer will not join.  Nothing here
touches the GPU: a stalled or vanished rank is detected on the host, and the process-group
timeout (`ADANA_PG_TIMEOUT_S`) is the backstop for a collective that was already issued.

The reference has no in-process failure detection (its resilience is job-level: periodic
`latest` checkpoints + `--auto_resume`, src/optim/base.py:136-157, src/main.py:457-468); this
adds the missing early exit so that the restart logic can take over.
"""
from __future__ import annotations

import os
import threading
import time
from datetime import timedelta
from typing import Optional


class PeerFailure(RuntimeError):
    pass


class HeartbeatWatchdog:
    def __init__(self, store, rank: int, world: int, timeout_s: float, period_s: Optional[float] = None,
                 clock=time.time):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = float(timeout_s)
        self.period_s = period_s if period_s is not None else max(0.05, min(1.0, self.timeout_s / 4))
        self.clock = clock
        self.failed: Optional[str] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last_beat = None

    @classmethod
    def from_env(cls, timeout_s: float):
        """Builds a second TCPStore client on the rendezvous address (MASTER_ADDR/MASTER_PORT+1 is
        not required: keys are namespaced, the job's own store is reused through a prefix)."""
        import torch.distributed as dist

        store = dist.PrefixStore("adana_hb", dist.distributed_c10d._get_default_store())
        return cls(store, dist.get_rank(), dist.get_world_size(), timeout_s)

    # ---- publisher ---------------------------------------------------------------------------------
    def beat(self, iteration: int):
        self._last_beat = self.clock()
        self.store.set(f"hb/{self.rank}", f"{iteration}:{self._last_beat:.3f}")

    # ---- checker -----------------------------------------------------------------------------------
    def check_once(self) -> Optional[str]:
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                raw = self.store.get(f"hb/{r}")
            except Exception:
                continue  # not published yet: the start-up grace period is handled by the caller
            raw = raw.decode() if isinstance(raw, (bytes, bytearray)) else str(raw)
            try:
                it, ts = raw.split(":")
                age = now - float(ts)
            except ValueError:
                continue
            if age > self.timeout_s:
                return f"rank {r} sent no heartbeat for {age:.1f}s (last at iteration {it})"
        return None

    def _run(self):
        while not self._stop.wait(self.period_s):
            try:
                msg = self.check_once()
            except Exception as e:  # store went away: the master rank died
                msg = f"heartbeat store unreachable: {e!r}"
            if msg is not None:
                self.failed = msg
                return

    def start(self):
        self._thread = threading.Thread(target=self._run, daemon=True, name="adana-heartbeat")
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.period_s + 1)

    def raise_if_failed(self):
        if self.failed is not None:
            raise PeerFailure(self.failed)
