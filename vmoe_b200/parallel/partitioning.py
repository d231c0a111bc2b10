"""Regex-driven placement of state-dict leaves on the ('expert', 'replica') mesh.

A ``PartitionSpec`` names, per tensor dimension, the mesh axes that shard it. Keys of the
flattened tree (joined by '/') are *searched* by each regex in order; the first hit wins and
tensors with at most one element are never partitioned (reference:
``vmoe/partitioning.py:309-315`` and ``:359-421``).
"""
from __future__ import annotations

import re
from typing import Any, Mapping, Optional, Sequence, Tuple, Union

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
