"""Regex-driven placement of state-dict leaves on the ('expert', 'replica') mesh.

A ``PartitionSpec`` names, per tensor dimension, the mesh axes that shard it. Keys of the
flattened tree (joined by '/') are *searched* by each regex in order; the first hit wins and
tensors with at most one element are never partitioned (reference:
``vmoe/partitioning.py:309-315`` and ``:359-421``).
"""
from __future__ import annotations

import re
from typing import Any, Mapping, Sequence, Tuple

import numpy as np

from vmoe_b200.utils.misc import flatten_dict, unflatten_dict


class PartitionSpec(tuple):
  """Tuple with one entry per leading tensor dim: None, an axis name or a tuple of names."""

  def __new__(cls, *axes):
    return super().__new__(cls, axes)

  def __repr__(self):
    return "PartitionSpec(" + ", ".join(repr(a) for a in self) + ")"

  def axes_of_dim(self, dim: int) -> Tuple[str, ...]:
    if dim >= len(self) or self[dim] is None:
      return ()
    a = self[dim]
    return (a,) if isinstance(a, str) else tuple(a)

  def sharded_axes(self) -> Tuple[str, ...]:
    out = []
    for d in range(len(self)):
      out.extend(self.axes_of_dim(d))
    return tuple(out)


def parse_partition_spec(spec) -> PartitionSpec:
  if isinstance(spec, PartitionSpec):
    return spec
  if spec is None:
    return PartitionSpec()
  if isinstance(spec, str):
    return PartitionSpec(spec)
  return PartitionSpec(*[tuple(a) if isinstance(a, (list, tuple)) else a for a in spec])


def _num_elements(value: Any) -> int:
  shape = getattr(value, "shape", None)
  if shape is None:
    return 1
  return int(np.prod(tuple(shape))) if len(tuple(shape)) else 1


def tree_axis_resources_from_regexes(*, tree: Mapping[str, Any],
                                     axis_resources_regexes: Sequence[Tuple[str, Any]]):
  """Returns a tree with the structure of ``tree`` whose leaves are ``PartitionSpec``s."""
  compiled = tuple((re.compile(rx), parse_partition_spec(spec))
                   for rx, spec in (axis_resources_regexes or ()))

  def lookup(key: str, value: Any) -> PartitionSpec:
    for rx, spec in compiled:
      if rx.search(key) and _num_elements(value) > 1:
        return spec
    return PartitionSpec()

  flat = flatten_dict(tree, sep="/")
  return unflatten_dict({k: lookup(k, v) for k, v in flat.items()}, sep="/")


def local_shard_slices(shape: Sequence[int], spec: PartitionSpec, mesh) -> Tuple[slice, ...]:
  """Slice of the global array held by ``mesh.rank`` under ``spec``."""
  coords = {"expert": mesh.expert_rank, "replica": mesh.replica_rank}
  sizes = mesh.shape
  out = []
  for d, n in enumerate(shape):
    axes = spec.axes_of_dim(d)
    if not axes:
      out.append(slice(0, n))
      continue
    parts, index = 1, 0
    for a in axes:
      index = index * sizes[a] + coords[a]
      parts *= sizes[a]
    if n % parts:
      raise ValueError(f"dim {d} of size {n} is not divisible by {parts} ({axes})")
    step = n // parts
    out.append(slice(index * step, (index + 1) * step))
  return tuple(out)


# ------------------------------------------------------------------ hardware / logical mesh views
def get_hardware_mesh(world_size: int, local_world_size: int):
  """The 2-D hardware mesh ``(device_on_process -> GPU of the node, process -> node)`` as an
  array of global ranks: ``hw[d][n]`` is GPU ``d`` of node ``n`` (ranks are numbered node by
  node, as torchrun does). Counterpart of ``get_hardware_mesh_other``
  (``vmoe/partitioning.py:213-220``) with one process per GPU instead of one per host."""
  import numpy as np
  if world_size % local_world_size:
    raise ValueError(f"{world_size} ranks do not fill nodes of {local_world_size} GPUs")
  nodes = world_size // local_world_size
  return np.arange(world_size).reshape(nodes, local_world_size).T


def get_logical_mesh(num_partitions: int, hardware_mesh):
  """``(expert, replica)`` array of ranks built from a hardware mesh: expert partitions are
  filled with the GPUs of one node first (NVLink / NVSwitch neighbours) and spill over to
  further nodes only when a node is too small, which is the reference's heuristic
  (``vmoe/partitioning.py:136-151``: ``d = min(P, local)``, ``h = min(P // d, processes)``)."""
  import numpy as np
  hw = np.asarray(hardware_mesh)
  local, nodes = hw.shape
  world = local * nodes
  if num_partitions < 1 or world % num_partitions:
    raise ValueError(f"The hardware mesh with shape {hw.shape} cannot be automatically "
                     f"partitioned into {num_partitions}.")
  # Node-major order of ranks: consecutive ranks share a node.
  order = hw.T.reshape(-1)
  return order.reshape(world // num_partitions, num_partitions).T


def processes_have_contiguous_device_slices(logical_mesh, local_world_size: int) -> bool:
  """True if every node's ranks occupy a contiguous block of the logical mesh's columns or
  rows (``vmoe/partitioning.py:93-114``); always true for the meshes built here."""
  import numpy as np
  lm = np.asarray(logical_mesh)
  node = lm // local_world_size
  for n in np.unique(node):
    es, rs = np.nonzero(node == n)
    if (es.max() - es.min() + 1) * (rs.max() - rs.min() + 1) != es.size:
      return False
  return True


def with_sharding_constraint(x, partition_spec=None):
  """Placement is explicit in this framework (each process owns its shard), so the GSPMD hint
  of the reference (``vmoe/partitioning.py:424-429``) is the identity."""
  del partition_spec
  return x
