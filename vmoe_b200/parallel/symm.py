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


class SymmetricBuffer:
  """One symmetric allocation of ``nbytes`` bytes on every rank of ``group``."""

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

  def barrier(self, channel: int = 0) -> None:
    """Stream-ordered barrier over the group (a small kernel on the current stream)."""
    self.hdl.barrier(channel=channel)
