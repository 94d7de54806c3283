"""The tagged-word exchange of the tensor-/expert-parallel kernels as a small event model on
CPU: why two alternating halves of the staging buffer are enough and one is not.

Protocol (include/b200w4.h, "exchanges inside the kernels"): every rank repeats
  SEND:   e = own count + 1; store (tag e, value) into half e & 1 of EVERY rank's buffer;
  GATHER: e = own count + 1; wait until every rank's entry of half e & 1 carries tag e,
          read the values, count = e.
Stores travel to a peer in order but with arbitrary delay (nothing flushes them); a rank may
therefore run ahead of its peers.  The model delivers stores and advances ranks in random
order and checks that every gather reads exactly the values of its own exchange."""
import random

import pytest


class Violation(Exception):
    pass


def run_exchanges(world, exchanges, halves, seed):
    rng = random.Random(seed)
    # stage[p][half][src] = (tag, value); channels[(src, dst)] = in-order stores in flight
    stage = [[[(0, None)] * world for _ in range(halves)] for _ in range(world)]
    channels = {(s, d): [] for s in range(world) for d in range(world)}
    count = [0] * world
    sent = [0] * world                      # exchanges whose SEND a rank has issued
    while min(count) < exchanges:
        moves = [("deliver", k) for k, q in channels.items() if q]
        for r in range(world):
            if count[r] >= exchanges:
                continue
            e = count[r] + 1
            if sent[r] < e:
                moves.append(("send", r))
            else:
                tags = [stage[r][e % halves][s][0] for s in range(world)]
                if any(t > e for t in tags):
                    # a peer's later exchange already overwrote an entry this gather still
                    # needs: the value is lost and the wait can never end
                    raise Violation((r, e, tags))
                if all(t == e for t in tags):
                    moves.append(("gather", r))
        assert moves, "deadlock without a violation"
        kind, arg = rng.choice(moves)
        if kind == "deliver":
            src, dst = arg
            tag, value = channels[arg].pop(0)
            stage[dst][tag % halves][src] = (tag, value)
        elif kind == "send":
            e = count[arg] + 1
            for dst in range(world):
                channels[(arg, dst)].append((e, (arg, e)))
            sent[arg] = e
        else:
            e = count[arg] + 1
            for s in range(world):
                if stage[arg][e % halves][s] != (e, (s, e)):
                    raise Violation((arg, e, s))
            count[arg] = e
    return count


@pytest.mark.parametrize("world", [2, 3, 8])
def test_two_halves_are_enough(world):
    for seed in range(300):
        assert run_exchanges(world, 6, halves=2, seed=seed) == [6] * world


def test_one_half_is_not():
    """With a single half a rank that runs one exchange ahead overwrites entries its peer has
    not read yet; some schedule must show it."""
    bad = 0
    for seed in range(300):
        try:
            run_exchanges(2, 6, halves=1, seed=seed)
        except Violation:
            bad += 1
    assert bad > 0


# ---- the wait bound against host skew -------------------------------------------------------
# A gather kernel spins for at most `wait_limit` after it starts.  The ranks' host threads do
# not start an exchange at the same instant: one may still be loading a kernel's code (first
# launch) or growing a buffer when the others already wait for its stores.  The bound must
# therefore exceed the skew, and a rank that does give up must stay in step with the group.

def run_timed(world, start, exchanges, wait_limit, flight=1.0, kernel=1.0):
    """Discrete-event model.  Rank r issues exchange e at max(own previous gather's end,
    start[r] for e == 1): SEND lands on every rank `flight` later; its GATHER begins `kernel`
    after the send and ends when the last word of the half has landed, or gives up at
    begin + wait_limit.  Returns (gave_up[r][e], count[r])."""
    arrive = [[None] * world for _ in range(exchanges + 1)]   # arrive[e][src]: landing time
    t = list(start)
    gave_up = [[False] * (exchanges + 1) for _ in range(world)]
    count = [0] * world
    for e in range(1, exchanges + 1):
        begin = [0.0] * world
        for r in range(world):
            arrive[e][r] = t[r] + flight
            begin[r] = t[r] + kernel
        for r in range(world):
            last = max(arrive[e])
            if last - begin[r] > wait_limit:
                gave_up[r][e] = True
                t[r] = begin[r] + wait_limit
            else:
                t[r] = max(begin[r], last)
            count[r] = e  # the count advances either way: the group stays in step
    return gave_up, count


def test_eight_ranks_one_starts_late():
    """Seven ranks start together, the eighth 80 time units later (its first launch of the
    exchange's kernels loads their code).  A bound of 50 -- the first design -- makes the seven
    give up on exchange 1; a bound above the skew does not, and in both cases every rank
    finishes every exchange with the same count, so later exchanges pair up again."""
    world, exchanges = 8, 5
    start = [0.0] * 7 + [80.0]
    gave_up, count = run_timed(world, start, exchanges, wait_limit=50.0)
    assert all(gave_up[r][1] for r in range(7)) and not gave_up[7][1]
    assert count == [exchanges] * world
    assert not any(gave_up[r][e] for r in range(world) for e in range(2, exchanges + 1))
    gave_up, count = run_timed(world, start, exchanges, wait_limit=2000.0)
    assert not any(any(g) for g in gave_up)
    assert count == [exchanges] * world


def test_warm_start_removes_the_skew():
    """With every kernel of the exchange launched once on a private one-rank group before the
    ranks meet at a barrier, the remaining skew is the barrier's own (a few units): even the
    short bound holds."""
    gave_up, _ = run_timed(8, [0.0, 1.5, 0.3, 2.0, 0.1, 0.9, 1.1, 0.4], 5, wait_limit=50.0)
    assert not any(any(g) for g in gave_up)
