"""Host-side failure detection between steps: heartbeats and a barrier with a deadline.

Ranks publish the step they have reached in the process group's key-value store. Before it
launches the next step a rank checks that every peer has published that step too (or has
announced that it left); a peer that stays behind past the deadline is reported with
``PeerFailure`` while no kernel or collective of the step is in flight yet, so the survivors
can checkpoint and stop instead of hanging in a collective. ``store_barrier`` is a named
barrier on the same store that raises ``BarrierTimeout`` with the ranks that never arrived.

Device-side waits are bounded separately: every kernel that waits on a flag, a peer or an
mbarrier gives up after a cycle limit and sets a bit in a status word
(``check_status`` turns a non-zero word into ``DeviceWaitTimeout``).

The reference has no counterpart: its only failure handling is restarting from the last
checkpoint (``vmoe/train/trainer.py:272-319``).
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class PeerFailure(RuntimeError):
  def __init__(self, ranks: Sequence[int], step: int, left: Sequence[int] = ()):
    self.ranks, self.step, self.left = list(ranks), step, list(left)
    what = f"ranks {self.ranks} did not reach step {step}"
    if self.left:
      what += f"; ranks {self.left} announced that they left"
    super().__init__(what)


class BarrierTimeout(RuntimeError):
  def __init__(self, name: str, missing: Sequence[int]):
    self.name, self.missing = name, list(missing)
    super().__init__(f"barrier {name!r}: ranks {self.missing} never arrived")


class DeviceWaitTimeout(RuntimeError):
  pass


STATUS_BITS = {1: "TMA producer wait", 2: "MMA wait", 4: "epilogue wait", 8: "ready-flag wait",
               16: "index out of range (access skipped)", 32: "peer signal wait"}


def check_status(status: torch.Tensor, what: str = "kernel") -> None:
  """Raises if a kernel recorded a timed-out wait in ``status``; clears the word."""
  value = int(status.item())
  if value:
    status.zero_()
    names = [name for bit, name in STATUS_BITS.items() if value & bit]
    raise DeviceWaitTimeout(f"{what}: device-side wait gave up ({', '.join(names)}; status={value})")


def _default_store():
  from torch.distributed import distributed_c10d
  return distributed_c10d._get_default_store()


class Heartbeat:
  """Step heartbeats of all ranks in a key-value store."""

  def __init__(self, store=None, rank: Optional[int] = None, world_size: Optional[int] = None,
               prefix: str = "vmoe_b200/heartbeat"):
    self.store = store if store is not None else _default_store()
    self.rank = dist.get_rank() if rank is None else rank
    self.world = dist.get_world_size() if world_size is None else world_size
    self.prefix = prefix

  def _key(self, rank: int) -> str:
    return f"{self.prefix}/{rank}"

  def beat(self, step: int) -> None:
    self.store.set(self._key(self.rank), str(int(step)))

  def leave(self) -> None:
    """Announces a planned exit (between steps, with nothing in flight)."""
    self.store.set(f"{self._key(self.rank)}/left", "1")

  def _step_of(self, rank: int) -> int:
    key = self._key(rank)
    if not self.store.check([key]):
      return -1
    return int(self.store.get(key).decode())

  def check(self, step: int, timeout_s: float = 10.0, poll_s: float = 0.05) -> None:
    """Returns when every peer has published ``step`` (or later); raises ``PeerFailure`` with
    the ranks that have not by the deadline or that announced they left."""
    deadline = time.monotonic() + timeout_s
    pending = [r for r in range(self.world) if r != self.rank]
    while True:
      # A peer that published this step counts for it even if it left afterwards.
      pending = [r for r in pending if self._step_of(r) < step]
      if not pending:
        return
      left = [r for r in pending if self.store.check([f"{self._key(r)}/left"])]
      if left:
        raise PeerFailure([r for r in pending if r not in left], step, left=left)
      if time.monotonic() >= deadline:
        raise PeerFailure(pending, step)
      time.sleep(poll_s)


_BARRIER_CALLS: dict = {}


def store_barrier(name: str, timeout_s: float = 60.0, store=None, rank: Optional[int] = None,
                  world_size: Optional[int] = None, poll_s: float = 0.02) -> None:
  """Named barrier through the key-value store; ``BarrierTimeout`` lists who is missing.

  A name may be used any number of times: every rank counts its own calls per (store, name)
  and the count is part of the key, so the n-th barrier of a name only sees the n-th arrivals
  (all ranks must call a given name equally often, as with any collective)."""
  store = store if store is not None else _default_store()
  rank = dist.get_rank() if rank is None else rank
  world = dist.get_world_size() if world_size is None else world_size
  gen_key = (id(store), name, rank)
  gen = _BARRIER_CALLS.get(gen_key, 0)
  _BARRIER_CALLS[gen_key] = gen + 1
  store.set(f"vmoe_b200/barrier/{name}/{gen}/{rank}", "1")
  deadline = time.monotonic() + timeout_s
  keys = [f"vmoe_b200/barrier/{name}/{gen}/{r}" for r in range(world)]
  while True:
    missing: List[int] = [r for r, k in enumerate(keys) if not store.check([k])]
    if not missing:
      return
    if time.monotonic() >= deadline:
      raise BarrierTimeout(name, missing)
    time.sleep(poll_s)
