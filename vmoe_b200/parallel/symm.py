"""Symmetric (peer-mapped) device memory for the expert-parallel kernels.

Every rank of a group allocates a buffer of the same size through
``torch.distributed._symmetric_memory`` and exchanges handles, after which each rank knows the
address of every peer's buffer in its own address space. The kernels of
``csrc/moe_p2p.cu`` and the GEMM epilogue store into those addresses directly over NVLink;
arrival is tracked with counters that live in the same buffers.
"""
from __future__ import annotations

from typing import List, Sequence

import torch


def available() -> bool:
  try:
    import torch.distributed._symmetric_memory  # noqa: F401
    return torch.cuda.is_available()
  except ImportError:
    return False


GUARD_BYTES = 256
_GUARD_SEED = 0x5AFEC0DE


def _guard_pattern(offset: int, device) -> torch.Tensor:
  """64 words that depend on the guard's offset, so that a copy of one guard over another (a
  whole region written one region too far) is seen too."""
  words = torch.arange(GUARD_BYTES // 4, dtype=torch.int64, device=device)
  words = (words * 2654435761 + _GUARD_SEED + offset) & 0x7FFFFFFF
  return words.to(torch.int32)


def write_guards(tensor: torch.Tensor, offsets: Sequence[int]) -> None:
  """Writes a canary of ``GUARD_BYTES`` bytes at each byte offset of the uint8 ``tensor``."""
  for off in offsets:
    tensor[off:off + GUARD_BYTES].view(torch.int32).copy_(_guard_pattern(off, tensor.device))


def damaged_guards(tensor: torch.Tensor, offsets: Sequence[int]) -> List[int]:
  """Offsets whose canary no longer holds its pattern (reads the device: synchronises)."""
  if not offsets:
    return []
  got = torch.stack([tensor[off:off + GUARD_BYTES].view(torch.int32) for off in offsets])
  want = torch.stack([_guard_pattern(off, tensor.device) for off in offsets])
  bad = (got != want).any(dim=1).tolist()
  return [off for off, b in zip(offsets, bad) if b]


class BufferOverrun(RuntimeError):
  """A kernel (of this rank or of a peer) wrote outside the region it was given."""


class SymmetricBuffer:
  """One symmetric allocation of ``nbytes`` bytes on every rank of ``group``. Regions that
  peers write can be fenced with canaries (``set_guards`` / ``check_guards``)."""

  def __init__(self, nbytes: int, group, device=None):
    import torch.distributed._symmetric_memory as symm_mem
    device = device or torch.device("cuda", torch.cuda.current_device())
    nbytes = (int(nbytes) + 255) // 256 * 256
    self.tensor = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    self.tensor.zero_()
    self.hdl = symm_mem.rendezvous(self.tensor, group)
    self.ptrs: List[int] = [int(p) for p in self.hdl.buffer_ptrs]
    self.rank = int(self.hdl.rank)
    self.world_size = int(self.hdl.world_size)
    self.nbytes = nbytes
    self.guards: List[int] = []
    torch.cuda.synchronize(device)
    self.hdl.barrier(channel=0)

  def local(self, offset: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
    n = 1
    for s in shape:
      n *= int(s)
    nb = n * torch.empty((), dtype=dtype).element_size()
    return self.tensor[offset:offset + nb].view(dtype).view(*shape)

  def peer(self, rank: int, offset: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
    """Tensor aliasing ``rank``'s buffer (peer memory mapped into this process)."""
    if rank == self.rank:
      return self.local(offset, shape, dtype)
    es = torch.empty((), dtype=dtype).element_size()
    assert offset % es == 0
    return self.hdl.get_buffer(rank, tuple(int(s) for s in shape), dtype, offset // es)

  def set_guards(self, offsets: Sequence[int]) -> None:
    """Canaries at these byte offsets of the LOCAL buffer (nobody may write there)."""
    self.guards = [int(o) for o in offsets]
    write_guards(self.tensor, self.guards)

  def check_guards(self, what: str = "symmetric buffer") -> None:
    bad = damaged_guards(self.tensor, self.guards)
    if bad:
      raise BufferOverrun(f"{what}: canary words at byte offsets {bad} of rank {self.rank}'s "
                          "buffer were overwritten")

  def barrier(self, channel: int = 0) -> None:
    """Stream-ordered barrier over the group (a small kernel on the current stream)."""
    self.hdl.barrier(channel=channel)
