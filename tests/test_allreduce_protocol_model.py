"""Host-side model of the counter protocol of the range-wise gradient all-reduce
(``vmoe_b200/csrc/allreduce_p2p.cu``): W ranks, R ranges, monotone counters whose target in
step ``epoch`` is ``epoch * W``. Every rank is two coroutines (its compute stream and its
communication stream) that yield wherever the device code waits or where another rank's
kernel could run in between; a seeded random scheduler
interleaves them. The model checks that the result is the sum over ranks in every step and
that no rank ever reads a peer's data too early or overwrites data a peer still needs. Dropping
any one of the three waits makes the model fail, which shows that it can see such bugs.
"""
import random

import pytest

READY, REDUCED, DONE = 0, 1, 2


class Violation(AssertionError):
  pass


class Cluster:
  """Buffers are lists of (value, tag) cells; the tag says what the cell holds:
  ('grad', epoch), ('sum', epoch)."""

  def __init__(self, world, ranges, cells_per_slice):
    self.world, self.ranges, self.cps = world, ranges, cells_per_slice
    self.range_len = world * cells_per_slice
    self.buf = [[(0, ("init", 0))] * (ranges * self.range_len) for _ in range(world)]
    self.flags = [[[0] * ranges for _ in range(3)] for _ in range(world)]

  def slice_of(self, rng, owner):
    base = rng * self.range_len + owner * self.cps
    return range(base, base + self.cps)


def compute_stream(c, rank, epochs, grads, st):
  """The backward pass and the optimizer of one rank: writes the gradients range by range
  (last range first), then waits for the communication stream and checks the sums."""
  w = c.world
  for epoch in range(1, epochs + 1):
    for rng in reversed(range(c.ranges)):
      for i in range(rng * c.range_len, (rng + 1) * c.range_len):
        c.buf[rank][i] = (grads(rank, epoch, i), ("grad", epoch))
      st["written"][rng] = epoch  # the marker fired: the side stream may reduce this range
      yield
    while st["comm_done"] < epoch:  # stream wait queued by finish()
      yield
    for i in range(c.ranges * c.range_len):
      value, tag = c.buf[rank][i]
      want = sum(grads(q, epoch, i) for q in range(w))
      if tag != ("sum", epoch) or value != want:
        raise Violation(f"rank {rank} cell {i} holds {value} {tag}, wanted {want} in step {epoch}")
    yield


def comm_stream(c, rank, epochs, st, skip=None):
  """The side stream of one rank: reduce and gather kernels per range, then the wait on the
  done counters. ``skip`` names a wait to leave out."""
  w = c.world
  for epoch in range(1, epochs + 1):
    target = epoch * w
    for rng in reversed(range(c.ranges)):
      while st["written"][rng] < epoch:  # side stream waits for the compute stream's event
        yield
      # ---- reduce kernel
      for p in range(w):
        c.flags[p][READY][rng] += 1
      if skip != "ready":
        while c.flags[rank][READY][rng] < target:
          yield
      for i in c.slice_of(rng, rank):
        acc = 0
        for q in range(w):
          value, tag = c.buf[q][i]
          if tag != ("grad", epoch):
            raise Violation(f"rank {rank} summed {tag} of rank {q} in step {epoch}")
          acc += value
          yield
        c.buf[rank][i] = (acc, ("sum", epoch))
      for p in range(w):
        c.flags[p][REDUCED][rng] += 1
      yield
      # ---- gather kernel
      if skip != "reduced":
        while c.flags[rank][REDUCED][rng] < target:
          yield
      for q in range(w):
        if q == rank:
          continue
        for i in c.slice_of(rng, q):
          value, tag = c.buf[q][i]
          if tag != ("sum", epoch):
            raise Violation(f"rank {rank} gathered {tag} of rank {q} in step {epoch}")
          c.buf[rank][i] = (value, tag)
          yield
      for p in range(w):
        c.flags[p][DONE][rng] += 1
      yield
    # ---- one wait on the done counters, queued before the optimizer
    for rng in range(c.ranges):
      if skip != "done":
        while c.flags[rank][DONE][rng] < target:
          yield
    st["comm_done"] = epoch
    yield


def programs(c, epochs, grads, skip=None):
  progs = {}
  for r in range(c.world):
    st = {"written": [0] * c.ranges, "comm_done": 0}
    progs[("compute", r)] = compute_stream(c, r, epochs, grads, st)
    progs[("comm", r)] = comm_stream(c, r, epochs, st, skip)
  return progs


def run(world, ranges, epochs, seed, skip=None, cells_per_slice=2, max_turns=200_000):
  rnd = random.Random(seed)
  c = Cluster(world, ranges, cells_per_slice)
  grads = lambda rank, epoch, i: (rank + 1) * 1000 + epoch * 37 + i
  progs = programs(c, epochs, grads, skip)
  turns = 0
  while progs:
    r = rnd.choice(sorted(progs))
    # Run a random burst so that ranks drift far apart as well as interleave finely.
    for _ in range(rnd.choice((1, 1, 2, 5, 40))):
      try:
        next(progs[r])
      except StopIteration:
        del progs[r]
        break
    turns += 1
    if turns > max_turns:
      raise Violation("the model did not finish: a wait can never be satisfied")


@pytest.mark.parametrize("world, ranges", [(2, 1), (2, 3), (3, 2), (4, 2), (8, 1)])
def test_protocol_is_correct_under_random_schedules(world, ranges):
  for seed in range(25):
    run(world, ranges, epochs=3, seed=seed)


@pytest.mark.parametrize("skip", ["ready", "reduced", "done"])
def test_model_detects_a_missing_wait(skip):
  failures = 0
  for seed in range(60):
    try:
      run(3, 2, epochs=3, seed=seed, skip=skip)
    except Violation:
      failures += 1
  assert failures > 0, f"leaving out the '{skip}' wait went unnoticed"


def test_counters_end_at_epoch_times_world():
  c = Cluster(4, 2, 2)
  alive = list(programs(c, 5, lambda rank, epoch, i: rank + epoch + i).values())
  while alive:
    for g in list(alive):
      try:
        next(g)
      except StopIteration:
        alive.remove(g)
  for r in range(4):
    for kind in (READY, REDUCED, DONE):
      assert c.flags[r][kind] == [5 * 4] * 2
