"""Column sums (bias gradients) of bf16 matrices on the GPU, PyTorch elsewhere."""
from __future__ import annotations

import ctypes

import torch

from vmoe_b200.ops import _lib


def colsum(x: torch.Tensor) -> torch.Tensor:
  """fp32 sum over the second-to-last dim: ``(.., R, N) -> (.., N)``."""
  if x.is_cuda and x.dtype == torch.bfloat16:
    x3 = x.unsqueeze(0) if x.dim() == 2 else x
    x3 = x3.contiguous()
    b, r, n = x3.shape
    out = torch.zeros(b, n, dtype=torch.float32, device=x.device)
    rc = _lib.lib().vmoe_colsum_bf16(ctypes.c_void_p(x3.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                     ctypes.c_int64(b), ctypes.c_int64(r), ctypes.c_int64(n),
                                     ctypes.c_void_p(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_colsum_bf16")
    _lib.count_launch()
    return out[0] if x.dim() == 2 else out
  return x.float().sum(dim=-2)
