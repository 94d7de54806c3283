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
