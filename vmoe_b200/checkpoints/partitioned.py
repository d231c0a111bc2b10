"""Sharded checkpoints: ``<prefix>.index`` + ``<prefix>.data-nnnnn-of-NNNNN``.

The index is a msgpack dict ``{'shard_count', 'index': tree of IndexInfo, 'version'}``; each
data shard maps the leaf position (order of the flattened tree, dict keys sorted) to the
array chunks it stores. Saving splits every distinct block of every array into chunks of at
most ``max_chunk_bytes``, assigns each chunk greedily to the least-filled shard file among
those written by a process that holds the block (shard ``i`` is written by process
``i % process_count``), and writes all files through the atomic/async machinery of
``base``. Restoring reads only the shard files whose chunks intersect the blocks this process
needs, so a checkpoint can be restored under a different sharding than it was saved with.

One process = one rank of the ('expert', 'replica') mesh. A leaf is described by an
``ArraySharding`` (global shape + which ranks hold which block); plain leaves are replicated.

Reference: ``vmoe/checkpoints/partitioned.py`` (save :127-212, restore :89-124 and :417-539,
chunk splitting :549-580, greedy assignment :292-345).
"""
from __future__ import annotations

import collections
import dataclasses
import enum
import logging
import os
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence, Tuple

import numpy as np

from vmoe_b200.checkpoints import base
from vmoe_b200.checkpoints import serialization
from vmoe_b200.checkpoints.types import (ArrayChunks, IndexInfo, LazyArrayChunks, ShapedArray,
                                         Slice, SliceNd)
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.parallel import multihost_utils
from vmoe_b200.parallel.partitioning import parse_partition_spec

ThreadPool = base.ThreadPool
MAX_CONCURRENT_BYTES = 8 * 1024 * 1024 * 1024
MAX_CHUNK_BYTES = 256 * 1024 * 1024


class Version(enum.Enum):
  UNKNOWN = None
  V1 = "20220622"


# ----------------------------------------------------------------------------- shardings
@dataclasses.dataclass
class ArraySharding:
  """Which ranks hold which block of a global array. ``blocks[rank]`` is the ``SliceNd`` of
  the block stored by that rank (ranks with equal blocks are replicas of each other)."""
  global_shape: Tuple[int, ...]
  blocks: Dict[int, SliceNd]

  def block_of(self, rank: int) -> SliceNd:
    return self.blocks[rank]

  def holders(self) -> Dict[SliceNd, List[int]]:
    out: Dict[SliceNd, List[int]] = collections.defaultdict(list)
    for rank in sorted(self.blocks):
      out[self.blocks[rank]].append(rank)
    return dict(out)

  @classmethod
  def replicated(cls, shape: Sequence[int], world_size: int) -> "ArraySharding":
    full = SliceNd([Slice(0, int(s)) for s in shape])
    return cls(tuple(int(s) for s in shape), {r: full for r in range(world_size)})

  @classmethod
  def from_spec(cls, shape: Sequence[int], spec, mesh) -> "ArraySharding":
    """Blocks implied by a ``PartitionSpec`` on the ('expert', 'replica') mesh."""
    spec = parse_partition_spec(spec)
    sizes = {"expert": mesh.num_partitions, "replica": mesh.world_size // mesh.num_partitions}
    layout = mesh_lib.mesh_layout(mesh.world_size, mesh.num_partitions)
    blocks = {}
    for e in range(sizes["expert"]):
      for r in range(sizes["replica"]):
        coords = {"expert": e, "replica": r}
        slices = []
        for d, n in enumerate(shape):
          axes = spec.axes_of_dim(d)
          parts, index = 1, 0
          for a in axes:
            index = index * sizes[a] + coords[a]
            parts *= sizes[a]
          if n % parts:
            raise ValueError(f"dim {d} of size {n} is not divisible by {parts} ({axes})")
          step = n // parts
          slices.append(Slice(index * step, (index + 1) * step))
        blocks[layout[e][r]] = SliceNd(slices)
    return cls(tuple(int(s) for s in shape), blocks)


def _as_sharding(s, shape, mesh) -> ArraySharding:
  if isinstance(s, ArraySharding):
    return s
  if s is None:
    return ArraySharding.replicated(shape, mesh.world_size)
  return ArraySharding.from_spec(shape, s, mesh)


# ----------------------------------------------------------------------------- tree helpers
def tree_flatten(tree) -> Tuple[List[Any], Any]:
  """Leaves in the reference's order (dict keys sorted) and a structure to rebuild the tree."""
  leaves: List[Any] = []

  def rec(node):
    if isinstance(node, Mapping):
      return {k: rec(node[k]) for k in sorted(node.keys())}
    leaves.append(node)
    return len(leaves) - 1

  return leaves, rec(tree)


def tree_unflatten(struct, leaves: Sequence[Any]):
  if isinstance(struct, Mapping):
    return {k: tree_unflatten(v, leaves) for k, v in struct.items()}
  return leaves[struct]


def _struct_equal(a, b) -> bool:
  if isinstance(a, Mapping) != isinstance(b, Mapping):
    return False
  if isinstance(a, Mapping):
    return set(a) == set(b) and all(_struct_equal(a[k], b[k]) for k in a)
  return True


# ----------------------------------------------------------------------------- slice maths
def _intersect_slicend(a: SliceNd, b: SliceNd) -> Optional[SliceNd]:
  if len(a) != len(b):
    raise ValueError(f"rank mismatch: {a} vs {b}")
  out = []
  for sa, sb in zip(a, b):
    start = max(sa.start or 0, sb.start or 0)
    stop = min(np.inf if sa.stop is None else sa.stop, np.inf if sb.stop is None else sb.stop)
    if stop <= start:
      return None
    out.append(Slice(start, None if stop == np.inf else int(stop)))
  return SliceNd(out)


def _split_slicend(slicend: SliceNd, max_chunk_items: Optional[int] = None) -> List[SliceNd]:
  """Splits a block into chunks of at most ``max_chunk_items`` elements.

  Axes are visited from the smallest extent up; an axis is cut into the smallest number of
  equal parts in 2..9 that divides it and brings the chunk under the limit, or, if there is
  none, into single rows."""
  shape = tuple(s.stop - s.start for s in slicend)
  chunk_items = int(np.prod(shape)) if shape else 1
  chunks = [tuple(slicend)]
  limit = max_chunk_items or -1
  if limit < 1 or chunk_items <= limit:
    return [SliceNd(c) for c in chunks]
  for i, size in sorted(enumerate(shape), key=lambda t: (t[1], t[0])):
    if size == 1:
      continue
    splits = [s for s in range(2, 10) if size % s == 0 and chunk_items // s <= limit]
    splits = (splits or [size])[0]
    start, stop, step = slicend[i].start, slicend[i].stop, size // splits
    chunks = [c[:i] + (Slice(j, j + step),) + c[i + 1:] for c in chunks
              for j in range(start, stop, step)]
    chunk_items /= splits
    if chunk_items <= limit:
      break
  return [SliceNd(c) for c in chunks]


def _find_smallest_ckpt_shard(bytes_per_ckpt_shard: Sequence[int], processes: Sequence[int],
                              process_count: int) -> int:
  order = sorted((b, i) for i, b in enumerate(bytes_per_ckpt_shard))
  return [i for _, i in order if i % process_count in processes][0]


def _create_map_slicend_to_holders(sharding: ArraySharding, itemsize: int,
                                   max_chunk_bytes: Optional[int]) -> Dict[SliceNd, List[int]]:
  if max_chunk_bytes and max_chunk_bytes >= 1:
    max_items = max(max_chunk_bytes // itemsize, 1)
  else:
    max_items = None
  out = {}
  for block, ranks in sharding.holders().items():
    for sub in _split_slicend(block, max_items):
      out[sub] = ranks
  return out


def _create_map_slicend_to_checkpoint_shard(slicend_to_holders: Mapping[SliceNd, Sequence[int]],
                                            itemsize: int, bytes_per_ckpt_shard: List[int],
                                            process_count: int) -> Dict[SliceNd, int]:
  out = {}
  for slicend in sorted(slicend_to_holders):
    processes = tuple(sorted(set(slicend_to_holders[slicend])))
    shard = _find_smallest_ckpt_shard(bytes_per_ckpt_shard, processes, process_count)
    out[slicend] = shard
    bytes_per_ckpt_shard[shard] += int(np.prod(slicend.shape)) * itemsize if len(slicend) else itemsize
  return out


# ----------------------------------------------------------------------------- save
def save_checkpoint(prefix: str, tree, *, shardings=None, mesh=None,
                    num_shards: Optional[int] = None, overwrite: bool = True,
                    makedirs: bool = True, thread_pool: Optional[ThreadPool] = None,
                    max_chunk_bytes: Optional[int] = MAX_CHUNK_BYTES,
                    version: Version = Version.V1):
  """Saves the *local* arrays of ``tree`` into a sharded checkpoint; returns a MapResult.

  ``shardings`` mirrors the (state-dict form of the) tree with ``ArraySharding`` /
  ``PartitionSpec`` / None (= replicated) leaves describing how each global array is spread
  over the ranks of ``mesh``. Every rank must call this function with the same structure.
  """
  assert version == Version.V1, f"version={version} != {Version.V1}"
  mesh = mesh or mesh_lib.get_mesh()
  process_count, process_index = mesh.world_size, mesh.rank
  tree = serialization.to_state_dict(tree)
  leaves, struct = tree_flatten(tree)
  leaves = [serialization.to_numpy(x) if not np.isscalar(x) else np.asarray(x) for x in leaves]
  if shardings is None:
    shard_leaves = [None] * len(leaves)
  else:
    shard_leaves, struct2 = tree_flatten(shardings)  # specs (tuples) are leaves
    if not _struct_equal(struct, struct2):
      raise ValueError("The tree and shardings structures do not match.")
  if num_shards is None or num_shards < process_count:
    if num_shards is not None:
      logging.warning(
          "While saving checkpoint with prefix=%r we found num_shards=%d and process_count=%d. "
          "Resetting num_shards=%d.", prefix, num_shards, process_count, process_count)
    num_shards = process_count

  bytes_per_shard = [0] * num_shards
  index_leaves: List[IndexInfo] = []
  my_shards = {i: LazyArrayChunks() for i in range(num_shards)
               if i % process_count == process_index}
  for i, arr in enumerate(leaves):
    sh = shard_leaves[i]
    if isinstance(sh, ArraySharding):
      sharding = sh
    elif sh is None:
      sharding = ArraySharding.replicated(arr.shape, process_count)
    else:
      # A PartitionSpec: the global shape follows from the local block and the spec.
      spec = parse_partition_spec(sh)
      sizes = mesh.shape
      gshape = list(arr.shape)
      for d in range(len(gshape)):
        for a in spec.axes_of_dim(d):
          gshape[d] *= sizes[a]
      sharding = ArraySharding.from_spec(gshape, spec, mesh)
    my_block = sharding.block_of(process_index)
    if tuple(my_block.shape) != tuple(arr.shape):
      raise ValueError(f"leaf {i}: local array shape {arr.shape} != block {my_block.shape}")
    holders = _create_map_slicend_to_holders(sharding, arr.dtype.itemsize, max_chunk_bytes)
    to_shard = _create_map_slicend_to_checkpoint_shard(holders, arr.dtype.itemsize,
                                                       bytes_per_shard, process_count)
    gslices = sorted(to_shard.keys())
    index_leaves.append(IndexInfo(
        global_shape=ShapedArray(sharding.global_shape, arr.dtype, False),
        global_slices=gslices, shards=[to_shard[s] for s in gslices]))
    for gslice, ckpt_shard in to_shard.items():
      if ckpt_shard % process_count != process_index:
        continue
      if process_index not in holders[gslice]:
        raise ValueError(
            f"No block of leaf index={i} is held by process {process_index} although it must "
            f"write global_slice={gslice} to ckpt_shard={ckpt_shard}. This is a bug.")
      local = SliceNd([Slice(s.start - b.start, s.stop - b.start)
                       for s, b in zip(gslice, my_block)])
      my_shards[ckpt_shard].add(i, arr, local, gslice)

  filepath_to_data: Dict[str, Any] = {
      base.add_shard_suffix(prefix + ".data", shard, num_shards): obj
      for shard, obj in my_shards.items()}
  if process_index == 0:
    index_content = {"shard_count": num_shards, "index": tree_unflatten(struct, index_leaves)}
    if version is not Version.UNKNOWN:
      index_content["version"] = version.value
    filepath_to_data[prefix + ".index"] = index_content
  if makedirs:
    _make_dir_sync(os.path.dirname(prefix), mesh)
  return base.save_multiple_checkpoints_async(filepath_to_data, overwrite=overwrite,
                                              makedirs=False, thread_pool=thread_pool)


def _make_dir_sync(workdir: str, mesh=None):
  mesh = mesh or mesh_lib.get_mesh()
  if mesh.rank == 0 and workdir:
    os.makedirs(workdir, exist_ok=True)
  multihost_utils.sync_devices(f"checkpoints:mkdir:{workdir}")


# ----------------------------------------------------------------------------- restore
def _find_ckpt_shards_to_restore(block: SliceNd, ckpt_slices: Sequence[SliceNd],
                                 ckpt_shards: Sequence[int]) -> Iterator[int]:
  if len(ckpt_slices) != len(ckpt_shards):
    raise ValueError("index lists have different lengths")
  for ckpt_slice, ckpt_shard in zip(ckpt_slices, ckpt_shards):
    if block == ckpt_slice or _intersect_slicend(block, ckpt_slice):
      yield ckpt_shard


def _restore_local_buffers(filepath: str, local_buffers: Sequence[Dict[SliceNd, np.ndarray]]):
  """Copies the intersections of a shard file's chunks with the wanted blocks."""
  ckpt = base.restore_checkpoint(filepath, ArrayChunks())
  for i in ckpt.chunks:
    for chunk, cslice in zip(ckpt.chunks[i], ckpt.global_slices[i]):
      for gslice, buffer in local_buffers[i].items():
        inter = _intersect_slicend(gslice, cslice) if len(gslice) else None
        if gslice == cslice or inter:
          inter = inter if inter is not None else gslice
          dst = tuple(slice(a.start - b.start, a.stop - b.start) for a, b in zip(inter, gslice))
          src = tuple(slice(a.start - b.start, a.stop - b.start) for a, b in zip(inter, cslice))
          buffer[dst] = chunk[src]


def _restore_checkpoint_from_index(prefix: str, shard_count: int, index, shardings, mesh,
                                   thread_pool: Optional[ThreadPool] = None,
                                   max_concurrent_bytes: Optional[int] = MAX_CONCURRENT_BYTES):
  pool = thread_pool or ThreadPool()
  index_leaves, struct = tree_flatten(index)
  if shardings is None:
    shard_leaves = [None] * len(index_leaves)
  else:
    shard_leaves, struct2 = tree_flatten(shardings)
    if not _struct_equal(struct, struct2):
      raise ValueError(f"The tree structs do not match.\nindex: {struct}\nsharding: {struct2}")
  rank = mesh.rank
  blocks: List[SliceNd] = []
  for info, sh in zip(index_leaves, shard_leaves):
    sharding = _as_sharding(sh, info.global_shape.shape, mesh)
    blocks.append(sharding.block_of(rank))
  local_buffers = [{blk: np.zeros(blk.shape, dtype=info.global_shape.dtype)}
                   for blk, info in zip(blocks, index_leaves)]
  needed = set()
  for blk, info in zip(blocks, index_leaves):
    needed.update(_find_ckpt_shards_to_restore(blk, info.global_slices, info.shards))
  files = [base.add_shard_suffix(prefix + ".data", i, shard_count) for i in sorted(needed)]
  chunksize = None
  if max_concurrent_bytes and files:
    total = sum(pool.map(os.path.getsize, files))
    chunksize = max(round(total / max_concurrent_bytes), 1)
  pool.map(lambda fp: _restore_local_buffers(fp, local_buffers), files, chunksize=chunksize)
  arrays = [buf[blk] for buf, blk in zip(local_buffers, blocks)]
  return tree_unflatten(struct, arrays)


def restore_checkpoint(prefix: str, tree=None, *, shardings=None, mesh=None,
                       thread_pool: Optional[ThreadPool] = None,
                       max_concurrent_bytes: Optional[int] = MAX_CONCURRENT_BYTES):
  """Restores the blocks this rank needs. Returns a nested dict of NumPy arrays, or, if
  ``tree`` is given, that structure filled with the restored values.

  Checkpoints without a version (legacy) can only be restored with a ``tree``.
  """
  mesh = mesh or mesh_lib.get_mesh()
  index = base.restore_checkpoint(prefix + ".index")
  version = Version(index.get("version", None))
  shard_count = index["shard_count"]
  index = index["index"]
  if version == Version.UNKNOWN:
    if tree is None:
      raise ValueError(
          f"You must specify the tree arguments when restoring from {Version.UNKNOWN}.")
    index = serialization.from_state_dict(serialization.to_state_dict(tree), index)
  elif version != Version.V1:
    raise NotImplementedError(f"Unsupported checkpoint version: {version!r}")
  state = _restore_checkpoint_from_index(prefix, shard_count, index, shardings, mesh,
                                         thread_pool=thread_pool,
                                         max_concurrent_bytes=max_concurrent_bytes)
  if tree is None:
    return state
  return serialization.from_state_dict(tree, state)


def read_index(prefix: str) -> Dict[str, Any]:
  """The decoded ``.index`` file (``shard_count``, ``index`` tree of IndexInfo, ``version``)."""
  return base.restore_checkpoint(prefix + ".index")
