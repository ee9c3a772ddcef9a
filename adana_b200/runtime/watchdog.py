"""Host-side failure detection: a per-rank heartbeat in the job's key-value store.

Every rank publishes `hb/<rank> = iteration:sequence:phase`.  The sequence number is advanced by a daemon
thread every `period_s`, so it keeps moving through phases in which the training thread publishes nothing
(an evaluation that only the master runs, a long checkpoint write, a compile warm-up).  The same thread
watches the peers: a peer has failed when its value has not CHANGED for `timeout_s` on this process's own
monotonic clock (no wall clocks are compared, so clock skew between nodes does not count as silence), or,
with `step_deadline_s`, when its iteration has not advanced for that long while it reports the `train`
phase (a main thread stuck in a collective while the process is alive).  The verdict is re-evaluated on
every check: a peer whose heartbeat moves again is healthy again.  The training loop calls
`raise_if_failed()` between steps — before its next launch — so a rank never enters a collective that a
dead peer will not join.  Nothing here
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
                 clock=time.monotonic, step_deadline_s: float = 0.0):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = float(timeout_s)
        self.step_deadline_s = float(step_deadline_s)
        self.period_s = period_s if period_s is not None else max(0.05, min(1.0, self.timeout_s / 4))
        self.clock = clock
        self.failed: Optional[str] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._iteration, self._seq, self._phase = 0, 0, "train"
        self._lock = threading.Lock()
        self._seen = {}       # peer -> [last raw value, local time it last changed, last iteration, time it advanced]

    @classmethod
    def from_env(cls, timeout_s: float, step_deadline_s: float = 0.0):
        """Uses the job's own rendezvous store through a key prefix (no second server or port)."""
        import torch.distributed as dist

        store = dist.PrefixStore("adana_hb", dist.distributed_c10d._get_default_store())
        return cls(store, dist.get_rank(), dist.get_world_size(), timeout_s, step_deadline_s=step_deadline_s)

    # ---- publisher ---------------------------------------------------------------------------------
    def _publish(self):
        with self._lock:
            self._seq += 1
            value = f"{self._iteration}:{self._seq}:{self._phase}"
        self.store.set(f"hb/{self.rank}", value)

    def beat(self, iteration: int, phase: str = "train"):
        """Called by the training thread: the iteration it is about to run (and the phase it is in)."""
        with self._lock:
            self._iteration, self._phase = int(iteration), phase
        self._publish()

    def phase(self, name: str):
        """Context manager for a phase other ranks may not share (evaluation, checkpoint): the step deadline does
        not run while it is open."""
        wd = self

        class _Phase:
            def __enter__(self_inner):
                wd.beat(wd._iteration, name)

            def __exit__(self_inner, *exc):
                wd.beat(wd._iteration, "train")
                return False

        return _Phase()

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
            parts = raw.split(":")
            try:
                it = int(parts[0])
            except ValueError:
                continue
            phase = parts[2] if len(parts) > 2 else "train"
            seen = self._seen.get(r)
            if seen is None:
                self._seen[r] = [raw, now, it, now]
                continue
            if raw != seen[0]:
                seen[0], seen[1] = raw, now
            if it != seen[2] or phase != "train":
                seen[2], seen[3] = it, now
            if now - seen[1] > self.timeout_s:
                return f"rank {r} sent no heartbeat for {now - seen[1]:.1f}s (last at iteration {it})"
            if self.step_deadline_s > 0 and now - seen[3] > self.step_deadline_s:
                return f"rank {r} is alive but stayed at iteration {it} for {now - seen[3]:.1f}s"
        return None

    def _run(self):
        while not self._stop.wait(self.period_s):
            try:
                self._publish()
                self.failed = self.check_once()     # re-evaluated every time: a peer that moves again is healthy
            except Exception as e:  # store went away: the master rank died
                self.failed = f"heartbeat store unreachable: {e!r}"
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
