"""Named barrier across all ranks with a consistency check.

Rank ``main_process`` contributes CRC32(name), every other rank 0; after a sum all-reduce
every rank must see exactly the CRC, otherwise ranks disagree about which barrier they are in
and a ``ValueError`` is raised (reference: ``vmoe/multihost_utils.py:25-44``).
"""
from __future__ import annotations

import zlib

import torch
import torch.distributed as dist


def sync_devices(name: str, main_process: int = 0, group=None) -> None:
  if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
    return
  h = zlib.crc32(name.encode())
  backend = dist.get_backend(group)
  device = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else "cpu"
  x = torch.tensor([h if dist.get_rank() == main_process else 0], dtype=torch.int64,
                   device=device)
  dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
  got = int(x.item())
  if got != h:
    raise ValueError(f"sync_devices failed for {name!r}. Found value: {got}, expected: {h}")


def all_ranks_ok(ok: bool, group=None) -> bool:
  """True if ``ok`` is true on every rank (a MIN all-reduce); the local value without a
  process group. Lets all ranks take the same branch after a step that can fail on one of
  them, e.g. reading a checkpoint shard."""
  if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
    return bool(ok)
  backend = dist.get_backend(group)
  device = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else "cpu"
  x = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
  dist.all_reduce(x, op=dist.ReduceOp.MIN, group=group)
  return bool(int(x.item()))
