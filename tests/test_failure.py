"""Host-side failure detection logic against a fake key-value store (single process)."""
import pytest
import torch

from vmoe_b200.parallel import failure


class FakeStore:
  def __init__(self):
    self.d = {}

  def set(self, k, v):
    self.d[k] = v.encode() if isinstance(v, str) else v

  def get(self, k):
    return self.d[k]

  def check(self, keys):
    return all(k in self.d for k in keys)


def test_heartbeat_passes_when_all_peers_reached_the_step():
  store = FakeStore()
  hbs = [failure.Heartbeat(store, rank=r, world_size=3) for r in range(3)]
  for hb in hbs:
    hb.beat(5)
  hbs[0].check(5, timeout_s=0.1)
  hbs[1].beat(6)
  hbs[1].check(5, timeout_s=0.1)  # a peer that is ahead is fine


def test_heartbeat_names_the_ranks_that_are_behind():
  store = FakeStore()
  hbs = [failure.Heartbeat(store, rank=r, world_size=3) for r in range(3)]
  hbs[0].beat(2)
  hbs[1].beat(2)
  hbs[2].beat(1)
  with pytest.raises(failure.PeerFailure) as e:
    hbs[0].check(2, timeout_s=0.1, poll_s=0.01)
  assert e.value.ranks == [2] and e.value.left == [] and e.value.step == 2


def test_heartbeat_reports_a_peer_that_left_without_waiting_for_the_deadline():
  store = FakeStore()
  hbs = [failure.Heartbeat(store, rank=r, world_size=2) for r in range(2)]
  hbs[0].beat(3)
  hbs[1].beat(2)
  hbs[1].leave()
  with pytest.raises(failure.PeerFailure) as e:
    hbs[0].check(3, timeout_s=30.0)
  assert e.value.left == [1]


def test_store_barrier_times_out_with_the_missing_ranks():
  store = FakeStore()
  failure.store_barrier("a", timeout_s=0.1, store=store, rank=0, world_size=1)
  with pytest.raises(failure.BarrierTimeout) as e:
    failure.store_barrier("b", timeout_s=0.05, store=store, rank=1, world_size=3, poll_s=0.01)
  assert e.value.missing == [0, 2]


def test_check_status_decodes_and_clears_the_word():
  status = torch.tensor([8 | 32], dtype=torch.int32)
  with pytest.raises(failure.DeviceWaitTimeout) as e:
    failure.check_status(status, "expert exchange")
  assert "ready-flag wait" in str(e.value) and "peer signal wait" in str(e.value)
  assert int(status.item()) == 0
  failure.check_status(status)  # zero: nothing to report


def test_store_barrier_can_reuse_a_name():
  """The second barrier of a name must wait for second arrivals, not see the first ones."""
  store = FakeStore()
  failure._BARRIER_CALLS.clear()
  # both ranks pass the first barrier (rank 1 arrives first, then rank 0 completes it)
  with pytest.raises(failure.BarrierTimeout):
    failure.store_barrier("epoch", timeout_s=0.02, store=store, rank=1, world_size=2, poll_s=0.01)
  failure.store_barrier("epoch", timeout_s=0.1, store=store, rank=0, world_size=2)
  # second use: only rank 0 arrives; the keys of the first use must not satisfy it
  with pytest.raises(failure.BarrierTimeout) as e:
    failure.store_barrier("epoch", timeout_s=0.05, store=store, rank=0, world_size=2, poll_s=0.01)
  assert e.value.missing == [1]


def test_canary_words_around_peer_written_regions():
  """Guard words of a (here: plain CPU) buffer: intact after writes inside the regions, reported
  by offset after a write that runs one element past a region or copies a neighbouring guard."""
  from vmoe_b200.parallel import symm
  buf = torch.zeros(4096, dtype=torch.uint8)
  offsets = [0, 1024 + symm.GUARD_BYTES, 4096 - symm.GUARD_BYTES]
  symm.write_guards(buf, offsets)
  buf[symm.GUARD_BYTES:offsets[1]] = 7           # the whole first region
  buf[offsets[1] + symm.GUARD_BYTES:offsets[2]] = 9
  assert symm.damaged_guards(buf, offsets) == []
  buf[offsets[1]] = 7                            # one byte too far
  assert symm.damaged_guards(buf, offsets) == [offsets[1]]
  symm.write_guards(buf, offsets)
  buf[offsets[2]:] = buf[:symm.GUARD_BYTES].clone()   # a guard copied over another
  assert symm.damaged_guards(buf, offsets) == [offsets[2]]
