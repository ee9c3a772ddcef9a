"""Host-side model of the peer-memory flag barrier (csrc/comm_p2p.cu::p2p_barrier_kernel) and an exhaustive
interleaving checker for it.

Protocol: barrier number k (k = 1, 2, ... — sequence numbers only grow) on rank r is a kernel of `world`
threads; thread t stores k into slot r of rank t's flag array (release, system scope) and then spins until slot t
of its OWN array holds a value >= k (acquire).  The next barrier on a rank starts only after the previous
kernel has ended (stream order).  Claims checked over every interleaving of the individual stores and loads:

  safety    when rank r leaves barrier k, every rank has entered barrier k (made all its round-k stores to r) —
            so everything a rank wrote before entering is ordered before what r does after leaving;
  liveness  no reachable state is stuck: some rank can always move until all ranks have finished all rounds
            (a rank that never enters is the failure case, handled by the kernel's time limit, not modelled).

`check(world, rounds, reset_flags=True)` models a broken variant (flags cleared after each barrier) and is used by
the tests to show that the checker does find violations.
"""
from __future__ import annotations

from collections import deque
from typing import Optional, Tuple


def check(world: int = 3, rounds: int = 2, reset_flags: bool = False) -> Tuple[bool, Optional[str], int]:
    """Breadth-first search over all interleavings.  Returns (ok, first problem found, states explored)."""
    full = (1 << world) - 1
    # state: per rank (round k in 1..rounds+1, stores-done mask, waits-passed mask); flags[t][r] = value rank r wrote to rank t
    init = (tuple((1, 0, 0) for _ in range(world)), tuple(tuple(0 for _ in range(world)) for _ in range(world)))
    seen = {init}
    todo = deque([init])
    while todo:
        ranks, flags = todo.popleft()
        moved = False
        for r, (k, stores, waits) in enumerate(ranks):
            if k > rounds:
                continue
            for t in range(world):
                if not (stores >> t) & 1:
                    # thread t of rank r stores k into flags[t][r]
                    nf = [list(row) for row in flags]
                    nf[t][r] = k
                    nr = list(ranks)
                    nr[r] = (k, stores | (1 << t), waits)
                    nxt = (tuple(nr), tuple(tuple(row) for row in nf))
                    moved = True
                    if nxt not in seen:
                        seen.add(nxt)
                        todo.append(nxt)
                elif not (waits >> t) & 1 and flags[r][t] >= k:
                    # thread t of rank r sees slot t of its own array at >= k and stops spinning
                    nw = waits | (1 << t)
                    nr = list(ranks)
                    nf = flags
                    if nw == full and stores == full:
                        # rank r leaves barrier k: every rank must have entered barrier k towards r
                        for u, (ku, su, _) in enumerate(ranks):
                            entered = ku > k or (ku == k and (su >> r) & 1)
                            if not entered:
                                return False, f"rank {r} left barrier {k} before rank {u} entered it", len(seen)
                        if reset_flags:
                            nf = [list(row) for row in flags]
                            nf[r] = [0] * world          # the broken variant clears its own slots
                            nf = tuple(tuple(row) for row in nf)
                        nr[r] = (k + 1, 0, 0)
                    else:
                        nr[r] = (k, stores, nw)
                    nxt = (tuple(nr), nf)
                    moved = True
                    if nxt not in seen:
                        seen.add(nxt)
                        todo.append(nxt)
        if not moved and any(k <= rounds for k, _, _ in ranks):
            return False, f"stuck: ranks {ranks}, flags {flags}", len(seen)
    return True, None, len(seen)
