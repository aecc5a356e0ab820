"""Exhaustive host-side check of the two synchronisation protocols the kernels rely on, on small instances.

The kernels cannot be run under a race detector, so the protocols themselves are modelled: every role is a little state machine
whose steps are the atomic operations it performs on shared words (an mbarrier phase, a flag word, a buffer slot), and
`explore` walks EVERY interleaving of those steps (breadth first over the reachable states), checking an invariant in each
state and that no state other than "all roles finished" is stuck.

  * `ring_model`: the shared-memory ring between the TMA producer and the MMA consumer of the GEMM / attention kernels:
    per stage one `full` and one `empty` barrier with phase parity; the producer waits `empty[s]` with the inverted parity
    (so that the first pass through the ring does not wait), the consumer waits `full[s]`.
  * `epoch_flag_model`: the cross-GPU barrier of `parallel/symm.py`: rank r writes the new epoch into word [slot][r] of EVERY
    rank's flag array, then waits until all words of its own array have reached that epoch; buffers written before the signal
    may be read by peers after their wait, and may be overwritten again only after the next barrier.
"""
from __future__ import annotations

from collections import deque


def explore(initial, roles, invariant, done):
  """`initial`: hashable state; `roles`: list of functions state -> list of successor states (empty when the role is blocked or
  finished); `invariant(state)` returns an error string or None; `done(state)`: every role finished. Returns (#states, error)."""
  seen, todo = {initial}, deque([initial])
  while todo:
    st = todo.popleft()
    err = invariant(st)
    if err:
      return len(seen), err
    nxt = [s for role in roles for s in role(st)]
    if not nxt and not done(st):
      return len(seen), f"deadlock in state {st}"
    for s in nxt:
      if s not in seen:
        seen.add(s)
        todo.append(s)
  return len(seen), None


# ------------------------------------------------------------------------------------------------- shared-memory ring
def ring_model(stages: int, items: int, producer_parity_inverted: bool = True):
  """State: (p_i, c_i, p_pc, c_pc, full phases, empty phases, slot contents). Item k lives in stage k % stages; a role's wait
  on a barrier with parity q passes when the barrier's completed-phase bit differs from ... the mbarrier rule: `try_wait(q)`
  succeeds once the phase with parity q has completed, i.e. when the current phase bit != q."""
  # barrier state: current phase bit (starts 0); an arrival (count 1) flips it
  init = (0, 0, 0, 0, (0,) * stages, (0,) * stages, (-1,) * stages)

  def producer(st):
    p, c, ppc, cpc, full, empty, slots = st
    if p >= items:
      return []
    s, rnd = p % stages, p // stages
    if ppc == 0:                                     # wait empty[s] with parity (round ^ 1) (or round, in the broken variant)
      q = (rnd & 1) ^ (1 if producer_parity_inverted else 0)
      return [(p, c, 1, cpc, full, empty, slots)] if empty[s] != q else []
    if ppc == 1:                                     # write the slot
      return [(p, c, 2, cpc, full, empty, slots[:s] + (p,) + slots[s + 1:])]
    return [(p + 1, c, 0, cpc, full[:s] + (full[s] ^ 1,) + full[s + 1:], empty, slots)]       # arrive full[s]

  def consumer(st):
    p, c, ppc, cpc, full, empty, slots = st
    if c >= items:
      return []
    s, rnd = c % stages, c // stages
    if cpc == 0:                                     # wait full[s] with parity round
      return [(p, c, ppc, 1, full, empty, slots)] if full[s] != (rnd & 1) else []
    if cpc == 1:                                     # read the slot: it must hold item c
      return [(p, c, ppc, 2, full, empty, slots if slots[s] == c else slots[:s] + (-2,) + slots[s + 1:])]
    return [(p, c + 1, ppc, 0, full, empty[:s] + (empty[s] ^ 1,) + empty[s + 1:], slots)]     # arrive empty[s]

  def invariant(st):
    return "the consumer read a stage that did not hold its item" if -2 in st[6] else None

  return init, [producer, consumer], invariant, (lambda st: st[0] >= items and st[1] >= items)


# ------------------------------------------------------------------------------------------------- cross-GPU epoch flags
def epoch_flag_model(ranks: int, rounds: int, wait_before_overwrite: bool = True):
  """Every round a rank (1) writes its buffer with the round number, (2) signals: stores epoch = round + 1 into word [r] of every
  rank's flags, one peer at a time, (3) waits for its own words, (4) reads every peer's buffer and requires the round's value,
  (5) (if `wait_before_overwrite`) passes a second barrier before the next round overwrites the buffer. Without (5) a fast rank
  overwrites data a slow peer has not read yet: the model finds that interleaving."""
  R = ranks
  # state: per rank (round, pc, sub) ; flags[R][R] for barrier A, flags2[R][R] for barrier B ; bufs[R] ; bad
  zero = tuple(tuple(0 for _ in range(R)) for _ in range(R))
  init = (tuple((0, 0, 0) for _ in range(R)), zero, zero, tuple(-1 for _ in range(R)), 0)

  def set2(m, i, j, v):
    row = m[i][:j] + (v,) + m[i][j + 1:]
    return m[:i] + (row,) + m[i + 1:]

  def role(r):
    def step(st):
      procs, fa, fb, bufs, bad = st
      rnd, pc, sub = procs[r]
      if rnd >= rounds:
        return []
      def upd(nr, npc, nsub, fa=fa, fb=fb, bufs=bufs, bad=bad):
        return [(procs[:r] + ((nr, npc, nsub),) + procs[r + 1:], fa, fb, bufs, bad)]
      e = rnd + 1
      if pc == 0:                                    # write own buffer
        return upd(rnd, 1, 0, bufs=bufs[:r] + (rnd,) + bufs[r + 1:])
      if pc == 1:                                    # signal A: one store per peer
        nfa = set2(fa, sub, r, e)
        return upd(rnd, 1, sub + 1, fa=nfa) if sub + 1 < R else upd(rnd, 2, 0, fa=nfa)
      if pc == 2:                                    # wait A
        return upd(rnd, 3, 0) if all(v >= e for v in fa[r]) else []
      if pc == 3:                                    # read peer `sub`
        nb = bad or (1 if bufs[sub] != rnd else 0)
        if sub + 1 < R:
          return upd(rnd, 3, sub + 1, bad=nb)
        return upd(rnd, 4, 0, bad=nb) if wait_before_overwrite else upd(rnd + 1, 0, 0, bad=nb)
      if pc == 4:                                    # signal B
        nfb = set2(fb, sub, r, e)
        return upd(rnd, 4, sub + 1, fb=nfb) if sub + 1 < R else upd(rnd, 5, 0, fb=nfb)
      return upd(rnd + 1, 0, 0) if all(v >= e for v in fb[r]) else []      # wait B
    return step

  def invariant(st):
    return "a rank read a peer buffer that did not hold the data of the current exchange" if st[4] else None

  return init, [role(r) for r in range(R)], invariant, (lambda st: all(p[0] >= rounds for p in st[0]))
