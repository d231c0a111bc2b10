"""Logical 2-D process mesh with axes ``('expert', 'replica')``.

One process drives one GPU (or is one gloo rank on CPU). ``num_partitions`` ranks form an
expert-parallel group that shards the expert axis of every MoE layer; the ``world /
num_partitions`` groups are replicas of each other. Consecutive ranks make an expert group,
so with the usual node-major rank numbering an expert group stays inside one NVSwitch domain
whenever it fits — the same preference as the reference's heuristic, which fills the devices
of one process before spanning processes (``vmoe/partitioning.py:136-151``). A request for
more partitions than ranks is clipped with an error log (``vmoe/partitioning.py:123-127``).
"""
from __future__ import annotations

import contextlib
import dataclasses
import datetime
import logging
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


@dataclasses.dataclass
class Mesh:
  """Rank layout and process groups of the ('expert', 'replica') mesh."""
  world_size: int = 1
  rank: int = 0
  num_partitions: int = 1          # size of the 'expert' axis
  local_world_size: int = 1
  expert_group: Optional[object] = None    # ranks that shard experts together
  replica_group: Optional[object] = None   # ranks that hold the same expert shard
  world_group: Optional[object] = None
  expert_ranks: Sequence[int] = (0,)
  replica_ranks: Sequence[int] = (0,)

  @property
  def axis_names(self):
    return ("expert", "replica")

  @property
  def shape(self):
    return {"expert": self.num_partitions, "replica": self.world_size // self.num_partitions}

  @property
  def expert_rank(self) -> int:
    return self.rank % self.num_partitions

  @property
  def replica_rank(self) -> int:
    return self.rank // self.num_partitions

  @property
  def num_replicas(self) -> int:
    return self.world_size // self.num_partitions

  @property
  def is_distributed(self) -> bool:
    return self.world_size > 1

  def layout(self) -> List[List[int]]:
    """``layout[e][r]`` = global rank at mesh coordinate (expert e, replica r)."""
    return mesh_layout(self.world_size, self.num_partitions)


def clip_num_partitions(num_partitions: int, world_size: int) -> int:
  if num_partitions > world_size:
    logging.error(
        "num_partitions=%d cannot be satisfied with num_devices=%d. Setting num_partitions=%d.",
        num_partitions, world_size, world_size)
    return world_size
  return max(1, num_partitions)


def mesh_layout(world_size: int, num_partitions: int) -> List[List[int]]:
  if world_size % num_partitions:
    raise ValueError(
        f"The {world_size} ranks cannot be automatically partitioned into {num_partitions}. "
        "The number of partitions must divide the number of ranks.")
  replicas = world_size // num_partitions
  return [[r * num_partitions + e for r in range(replicas)] for e in range(num_partitions)]


def get_auto_logical_mesh(num_partitions: int, world_size: Optional[int] = None,
                          rank: Optional[int] = None, create_groups: bool = True) -> Mesh:
  """Builds the mesh for this process; creates the process groups when distributed."""
  initialized = dist.is_available() and dist.is_initialized()
  if world_size is None:
    world_size = dist.get_world_size() if initialized else 1
  if rank is None:
    rank = dist.get_rank() if initialized else 0
  num_partitions = clip_num_partitions(num_partitions, world_size)
  layout = mesh_layout(world_size, num_partitions)
  replicas = world_size // num_partitions
  my_e, my_r = rank % num_partitions, rank // num_partitions
  expert_ranks = [layout[e][my_r] for e in range(num_partitions)]
  replica_ranks = [layout[my_e][r] for r in range(replicas)]
  mesh = Mesh(world_size=world_size, rank=rank, num_partitions=num_partitions,
              local_world_size=int(os.environ.get("LOCAL_WORLD_SIZE", world_size)),
              expert_ranks=expert_ranks, replica_ranks=replica_ranks)
  if initialized and create_groups and world_size > 1:
    mesh.world_group = dist.group.WORLD
    # new_group must be called by every rank for every group, in the same order.
    for r in range(replicas):
      ranks = [layout[e][r] for e in range(num_partitions)]
      grp = dist.new_group(ranks) if num_partitions > 1 else None
      if r == my_r:
        mesh.expert_group = grp
    for e in range(num_partitions):
      ranks = [layout[e][r] for r in range(replicas)]
      grp = dist.new_group(ranks) if replicas > 1 else None
      if e == my_e:
        mesh.replica_group = grp
  return mesh


def log_logical_mesh(mesh: Mesh, logger=logging) -> str:
  """Pretty-prints which rank sits at each (expert, replica) coordinate."""
  layout = mesh.layout()
  width = max(len(str(mesh.world_size - 1)), 1) + 2
  replicas = mesh.num_replicas
  header = " " * 12 + "".join(f"{'r' + str(r):>{width}}" for r in range(replicas))
  lines = [f"Logical mesh ('expert', 'replica') = ({mesh.num_partitions}, {replicas})", header]
  for e, row in enumerate(layout):
    lines.append(f"expert {e:>4} " + "".join(f"{rk:>{width}}" for rk in row))
  text = "\n".join(lines)
  logger.info("%s", text)
  return text


_CURRENT = Mesh()


def get_mesh() -> Mesh:
  return _CURRENT


def set_mesh(mesh: Mesh) -> None:
  global _CURRENT
  _CURRENT = mesh


@contextlib.contextmanager
def use_mesh(mesh: Mesh):
  global _CURRENT
  prev, _CURRENT = _CURRENT, mesh
  try:
    yield mesh
  finally:
    _CURRENT = prev


def init_distributed(backend: Optional[str] = None, timeout_s: float = 1800.0) -> bool:
  """Initialises ``torch.distributed`` from the torchrun environment, one rank per GPU.

  Returns True if a process group exists afterwards. The backend defaults to NCCL when CUDA
  is available and gloo otherwise.
  """
  if dist.is_initialized():
    return True
  if "RANK" not in os.environ or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
    if torch.cuda.is_available():
      torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    return False
  os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
  os.environ.setdefault("MASTER_PORT", "29500")
  use_cuda = torch.cuda.is_available()
  backend = backend or ("nccl" if use_cuda else "gloo")
  kwargs = {}
  if use_cuda:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if backend == "nccl":
      kwargs["device_id"] = torch.device("cuda", local_rank)
  dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s),
                          **kwargs)
  return True
