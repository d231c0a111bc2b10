"""Host-side model of the peer-memory protocol of the expert-parallel MoE layer
(``vmoe_b200/ops/moe_ops.py:_P2PMoeFn``, ``vmoe_b200/csrc/moe_p2p.cu``).

Every rank owns one expert and the buffers XE (rows pushed to its expert), YB (expert outputs
coming home), DYE and DXB (the same for the backward pass), with monotone counters: per-tile
arrival counters that gate the first GEMM (target ``epoch * rows``) and per-source completion
counters that gate the combine (target ``epoch``). Steps are separated by "free" counters
instead of a barrier: after its last read of XE / DYE in a backward pass (the weight
gradients) an owner bumps its entry of every rank's free counters, and a rank's next forward
pass pushes only once every owner has done so. Each rank is a coroutine on one in-order
stream; a seeded random scheduler interleaves the ranks. Cells carry a tag (what, step) so
that a read of stale or too-new data is seen. Leaving out the free wait or either other kind
of wait makes the model fail.
"""
import random

import pytest


class Violation(AssertionError):
  pass


class Layer:

  def __init__(self, world, rows):
    self.w, self.r = world, rows
    cell = (0, ("init", 0))
    # xe[owner][src][row], yb[home][expert][row]; the same shapes for the backward buffers.
    self.xe = [[[cell] * rows for _ in range(world)] for _ in range(world)]
    self.dye = [[[cell] * rows for _ in range(world)] for _ in range(world)]
    self.yb = [[[cell] * rows for _ in range(world)] for _ in range(world)]
    self.dxb = [[[cell] * rows for _ in range(world)] for _ in range(world)]
    self.fx = [[0] * world for _ in range(world)]    # [owner][tile = source]
    self.fdy = [[0] * world for _ in range(world)]
    self.fy = [[0] * world for _ in range(world)]    # [home][expert]
    self.fdx = [[0] * world for _ in range(world)]
    self.ffree = [[0] * world for _ in range(world)]  # [pusher][owner]


def _expect(cell, what, step, who):
  value, tag = cell
  if tag != (what, step):
    raise Violation(f"{who} read {tag}, wanted {(what, step)}")
  return value


def rank_program(c, q, steps, skip=None):
  w, r = c.w, c.r
  x_of = lambda step, src, owner, row: step * 1000 + src * 100 + owner * 10 + row
  for step in range(1, steps + 1):
    # ------------------------------------------------------------------ forward
    if skip != "free":
      for owner in range(w):
        while c.ffree[q][owner] < step - 1:
          yield
    # push my rows for every expert into its owner's XE, then bump the tile's counter
    for i in range(w):
      owner = (q + i) % w
      for row in range(r):
        c.xe[owner][q][row] = (x_of(step, q, owner, row), ("x", step))
        yield
      c.fx[owner][q] += r
    # GEMM1 gated per tile, GEMM2 storing each source's rows into that source's YB
    hid = {}
    for i in range(w):
      src = (q + i) % w
      if skip != "arrival":
        while c.fx[q][src] < step * r:
          yield
      for row in range(r):
        hid[src, row] = _expect(c.xe[q][src][row], "x", step, f"GEMM1 of rank {q}") + 1
        yield
    for i in range(w):
      src = (q + i) % w
      for row in range(r):
        c.yb[src][q][row] = (hid[src, row] * 2, ("y", step))
        yield
      c.fy[src][q] += 1
    # combine at home once every expert's rows are complete
    for e in range(w):
      if skip != "complete":
        while c.fy[q][e] < step:
          yield
      for row in range(r):
        got = _expect(c.yb[q][e][row], "y", step, f"combine of rank {q}")
        if got != (x_of(step, q, e, row) + 1) * 2:
          raise Violation(f"rank {q} combined a wrong value in step {step}")
      yield
    # ------------------------------------------------------------------ backward
    for i in range(w):
      owner = (q + i) % w
      for row in range(r):
        # the push also reads the expert outputs at home (gate gradients)
        _expect(c.yb[q][owner][row], "y", step, f"backward push of rank {q}")
        c.dye[owner][q][row] = (x_of(step, q, owner, row) + 7, ("dy", step))
        yield
      c.fdy[owner][q] += r
    dpre = {}
    for i in range(w):
      src = (q + i) % w
      if skip != "arrival":
        while c.fdy[q][src] < step * r:
          yield
      for row in range(r):
        dpre[src, row] = _expect(c.dye[q][src][row], "dy", step, f"dgrad GEMM of rank {q}") + 1
        yield
    for i in range(w):
      src = (q + i) % w
      for row in range(r):
        c.dxb[src][q][row] = (dpre[src, row] * 3, ("dx", step))
        yield
      c.fdx[src][q] += 1
    # weight gradients read the rows received in the forward pass once more
    for src in range(w):
      for row in range(r):
        _expect(c.xe[q][src][row], "x", step, f"wgrad of rank {q}")
        _expect(c.dye[q][src][row], "dy", step, f"wgrad of rank {q}")
      yield
    # ... for the last time: every pusher may overwrite what it sent to this owner
    for src in range(w):
      c.ffree[src][q] += 1
    for e in range(w):
      if skip != "complete":
        while c.fdx[q][e] < step:
          yield
      for row in range(r):
        got = _expect(c.dxb[q][e][row], "dx", step, f"backward combine of rank {q}")
        if got != (x_of(step, q, e, row) + 8) * 3:
          raise Violation(f"rank {q} combined a wrong gradient in step {step}")
      yield


def run(world, rows, steps, seed, skip=None, max_turns=400_000):
  rnd = random.Random(seed)
  c = Layer(world, rows)
  progs = {q: rank_program(c, q, steps, skip) for q in range(world)}
  turns = 0
  while progs:
    q = rnd.choice(sorted(progs))
    for _ in range(rnd.choice((1, 1, 3, 10, 80))):
      try:
        next(progs[q])
      except StopIteration:
        del progs[q]
        break
    turns += 1
    if turns > max_turns:
      raise Violation("the model did not finish: a wait can never be satisfied")
  return c


@pytest.mark.parametrize("world, rows", [(2, 2), (3, 2), (4, 1), (8, 1)])
def test_protocol_is_correct_under_random_schedules(world, rows):
  for seed in range(20):
    c = run(world, rows, steps=3, seed=seed)
    assert all(v == 3 * rows for row in c.fx for v in row)
    assert all(v == 3 for row in c.fy for v in row)
    assert all(v == 3 for row in c.ffree for v in row)


@pytest.mark.parametrize("skip", ["free", "arrival", "complete"])
def test_model_detects_a_missing_wait(skip):
  failures = 0
  for seed in range(80):
    try:
      run(3, 2, steps=3, seed=seed, skip=skip)
    except Violation:
      failures += 1
  assert failures > 0, f"leaving out the '{skip}' wait went unnoticed"
