"""Host-side models of two device protocols, each with an exhaustive interleaving checker: the peer-memory flag
barrier (csrc/comm_p2p.cu::p2p_barrier_kernel, `check`) and the ticket / chunk-counter copy protocol of the staged
gather GEMM (csrc/gemm_tcgen05.cu, `check_staged_gather`).

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


def check_staged_gather(ctas: int = 2, resident: int = 1, units: int = 4, units_per_chunk: int = 2,
                        static_assignment: bool = False) -> Tuple[bool, Optional[str], int]:
    """Model of the staged gather GEMM's copy protocol (csrc/gemm_tcgen05.cu: stage_copy_loop / stage_wait).

    Each CTA has one copier warp and one producer.  A copier repeatedly takes the next unit from a shared ticket
    counter, copies it and bumps the counter of the unit's chunk; a producer walks over all chunks in order and
    passes chunk c only when its counter has reached `units_per_chunk`.  A CTA leaves when both are done.  Only
    `resident` CTAs run at first (the grid may be larger than what fits, or another kernel may hold SMs): a waiting
    CTA starts when a running one leaves.  Checked over every interleaving:

      safety    a producer never passes a chunk with a unit not yet copied;
      liveness  no reachable state is stuck before every CTA has left.

    `static_assignment=True` models the variant in which unit u belongs to the copier of CTA u % ctas: a resident
    producer then waits for a unit owned by a CTA that cannot start, and the checker must report it."""
    n_chunks = (units + units_per_chunk - 1) // units_per_chunk
    # per CTA: (running, copier_holding_unit or -1, copier_done, producer_next_chunk, static_next_unit)
    init_ctas = tuple((i < resident, -1, False, 0, i) for i in range(ctas))
    init = (0, tuple(0 for _ in range(n_chunks)), frozenset(), init_ctas)   # ticket, chunk counters, copied units, CTAs
    seen = {init}
    todo = deque([init])
    while todo:
        ticket, counters, copied, cs = todo.popleft()
        succ = []
        for i, (run, hold, cdone, pnext, snext) in enumerate(cs):
            if not run:
                continue
            if not cdone:
                if hold < 0:      # take a unit
                    if static_assignment:
                        u, nt, ns = (snext, ticket, snext + ctas)
                    else:
                        u, nt, ns = (ticket, ticket + 1, snext)
                    c2 = list(cs)
                    c2[i] = (run, u, False, pnext, ns) if u < units else (run, -1, True, pnext, ns)
                    succ.append((nt, counters, copied, tuple(c2)))
                else:             # finish the copy of the unit held and count it
                    cn = list(counters)
                    cn[hold // units_per_chunk] += 1
                    c2 = list(cs)
                    c2[i] = (run, -1, False, pnext, snext)
                    succ.append((ticket, tuple(cn), copied | {hold}, tuple(c2)))
            if pnext < n_chunks:
                need = min(units_per_chunk, units - pnext * units_per_chunk)
                if counters[pnext] >= need:
                    for u in range(pnext * units_per_chunk, pnext * units_per_chunk + need):
                        if u not in copied:
                            return False, f"producer of CTA {i} passed chunk {pnext} before unit {u} was copied", len(seen)
                    c2 = list(cs)
                    c2[i] = (run, hold, cdone, pnext + 1, snext)
                    succ.append((ticket, counters, copied, tuple(c2)))
            if cdone and pnext == n_chunks:      # the CTA leaves; a waiting one takes its SM
                c2 = list(cs)
                c2[i] = (False, -1, True, n_chunks, snext)
                for j, (rj, hj, dj, pj, sj) in enumerate(c2):
                    if not rj and not (dj and pj == n_chunks):
                        c2[j] = (True, hj, dj, pj, sj)
                        break
                succ.append((ticket, counters, copied, tuple(c2)))
        all_left = all((not run) and cdone and pnext == n_chunks for run, _, cdone, pnext, _ in cs)
        if not succ and not all_left:
            return False, f"stuck: ticket {ticket}, counters {counters}, CTAs {cs}", len(seen)
        for nxt in succ:
            if nxt not in seen:
                seen.add(nxt)
                todo.append(nxt)
    return True, None, len(seen)
