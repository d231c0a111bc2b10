"""Mesh construction and regex placement without devices: world size and rank are passed in
(the reference mocks ``jax.devices`` for the same purpose,
``vmoe/partitioning_test.py:35-245``)."""
import logging

import numpy as np
import pytest
import torch

from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.parallel import partitioning
from vmoe_b200.parallel.partitioning import PartitionSpec


@pytest.mark.parametrize("world, partitions", [(1, 1), (2, 2), (4, 2), (8, 8), (8, 4), (16, 8),
                                               (32, 8)])
def test_every_rank_appears_once(world, partitions):
  seen = set()
  for rank in range(world):
    mesh = mesh_lib.get_auto_logical_mesh(partitions, world_size=world, rank=rank,
                                          create_groups=False)
    assert mesh.shape == {"expert": partitions, "replica": world // partitions}
    assert rank in mesh.expert_ranks and rank in mesh.replica_ranks
    assert len(mesh.expert_ranks) == partitions
    assert len(mesh.replica_ranks) == world // partitions
    layout = mesh.layout()
    assert layout[mesh.expert_rank][mesh.replica_rank] == rank
    seen.add((mesh.expert_rank, mesh.replica_rank))
  assert len(seen) == world


def test_expert_partitions_stay_inside_a_node():
  # 16 ranks on two nodes of eight GPUs, eight expert partitions: every expert group is a node.
  for rank in range(16):
    mesh = mesh_lib.get_auto_logical_mesh(8, world_size=16, rank=rank, create_groups=False)
    assert {r // 8 for r in mesh.expert_ranks} == {rank // 8}
    assert sorted(r % 8 for r in mesh.replica_ranks) == [rank % 8] * 2


def test_too_many_partitions_are_clipped(caplog):
  with caplog.at_level(logging.ERROR):
    mesh = mesh_lib.get_auto_logical_mesh(16, world_size=4, rank=1, create_groups=False)
  assert mesh.num_partitions == 4
  assert any("cannot be satisfied" in r.getMessage() for r in caplog.records)


def test_indivisible_partitions_raise():
  with pytest.raises(ValueError, match="cannot be automatically partitioned"):
    mesh_lib.get_auto_logical_mesh(3, world_size=8, rank=0, create_groups=False)
  with pytest.raises(ValueError, match="cannot be automatically"):
    partitioning.get_logical_mesh(3, partitioning.get_hardware_mesh(8, 8))


def test_hardware_mesh_shapes():
  hw = partitioning.get_hardware_mesh(16, 8)
  assert hw.shape == (8, 2)
  assert hw[:, 0].tolist() == list(range(8)) and hw[:, 1].tolist() == list(range(8, 16))
  with pytest.raises(ValueError):
    partitioning.get_hardware_mesh(12, 8)


@pytest.mark.parametrize("world, local, partitions", [(8, 8, 8), (16, 8, 4), (16, 8, 16),
                                                      (32, 8, 8), (4, 1, 2)])
def test_logical_mesh_from_hardware_mesh(world, local, partitions):
  lm = partitioning.get_logical_mesh(partitions, partitioning.get_hardware_mesh(world, local))
  assert lm.shape == (partitions, world // partitions)
  assert sorted(lm.reshape(-1).tolist()) == list(range(world))
  assert np.array_equal(lm, np.asarray(mesh_lib.mesh_layout(world, partitions)))
  assert partitioning.processes_have_contiguous_device_slices(lm, local)


def test_non_contiguous_slices_are_detected():
  lm = np.asarray([[0, 8, 1, 9], [2, 10, 3, 11]])
  assert not partitioning.processes_have_contiguous_device_slices(lm, 8)


def test_log_logical_mesh_lists_all_ranks():
  mesh = mesh_lib.get_auto_logical_mesh(2, world_size=4, rank=0, create_groups=False)
  text = mesh_lib.log_logical_mesh(mesh)
  assert "(2, 2)" in text
  for rank in range(4):
    assert str(rank) in text


def test_parse_partition_spec():
  assert partitioning.parse_partition_spec(None) == PartitionSpec()
  assert partitioning.parse_partition_spec("expert") == PartitionSpec("expert")
  assert partitioning.parse_partition_spec(("expert", None)) == PartitionSpec("expert", None)
  assert partitioning.parse_partition_spec([["expert", "replica"]]) == \
      PartitionSpec(("expert", "replica"))
  spec = PartitionSpec(("expert", "replica"), None)
  assert partitioning.parse_partition_spec(spec) is spec
  assert spec.sharded_axes() == ("expert", "replica")
  assert spec.axes_of_dim(1) == () and spec.axes_of_dim(5) == ()


def test_first_matching_regex_wins_and_scalars_stay_replicated():
  tree = {
      "a": torch.zeros(4, 4),
      "b": {"c": torch.zeros(4), "scalar": torch.zeros(()), "one": torch.zeros(1)},
      "d": {"Moe": {"Mlp": {"kernel": torch.zeros(8, 4, 4)}}},
  }
  out = partitioning.tree_axis_resources_from_regexes(
      tree=tree,
      axis_resources_regexes=[("Moe/Mlp/.*", ("expert",)), ("b/.*", ("replica",)),
                              (".*", (None, "expert"))])
  assert out["d"]["Moe"]["Mlp"]["kernel"] == PartitionSpec("expert")
  assert out["b"]["c"] == PartitionSpec("replica")
  assert out["b"]["scalar"] == PartitionSpec() and out["b"]["one"] == PartitionSpec()
  assert out["a"] == PartitionSpec(None, "expert")


def test_unmatched_leaves_are_replicated():
  out = partitioning.tree_axis_resources_from_regexes(
      tree={"x": torch.zeros(3, 3)}, axis_resources_regexes=[("y", ("expert",))])
  assert out == {"x": PartitionSpec()}


@pytest.mark.parametrize("rank, expected", [(0, (0, 2)), (1, (2, 4)), (2, (0, 2)), (3, (2, 4))])
def test_local_shard_slices_expert_axis(rank, expected):
  mesh = mesh_lib.get_auto_logical_mesh(2, world_size=4, rank=rank, create_groups=False)
  sl = partitioning.local_shard_slices((4, 6), PartitionSpec("expert"), mesh)
  assert (sl[0].start, sl[0].stop) == expected and (sl[1].start, sl[1].stop) == (0, 6)


def test_local_shard_slices_over_both_axes_cover_the_array():
  covered = np.zeros(8, dtype=int)
  for rank in range(4):
    mesh = mesh_lib.get_auto_logical_mesh(2, world_size=4, rank=rank, create_groups=False)
    (sl,) = partitioning.local_shard_slices((8,), PartitionSpec(("expert", "replica")), mesh)
    covered[sl] += 1
  assert covered.tolist() == [1] * 8
  mesh = mesh_lib.get_auto_logical_mesh(2, world_size=4, rank=0, create_groups=False)
  with pytest.raises(ValueError):
    partitioning.local_shard_slices((6,), PartitionSpec(("expert", "replica")), mesh)


def test_with_sharding_constraint_is_identity():
  x = torch.arange(4)
  assert partitioning.with_sharding_constraint(x, PartitionSpec("expert")) is x
