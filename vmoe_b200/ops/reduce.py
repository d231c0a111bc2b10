"""Column sums (bias gradients) of bf16 matrices on the GPU, PyTorch elsewhere."""
from __future__ import annotations

import ctypes

import torch

from vmoe_b200.ops import _lib


def _colsum3(x3: torch.Tensor) -> torch.Tensor:
  b, r, n = x3.shape
  out = torch.zeros(b, n, dtype=torch.float32, device=x3.device)
  rc = _lib.lib().vmoe_colsum_bf16(ctypes.c_void_p(x3.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                   ctypes.c_int64(b), ctypes.c_int64(r), ctypes.c_int64(n),
                                   ctypes.c_void_p(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_colsum_bf16")
  _lib.count_launch()
  return out


def colsum(x: torch.Tensor) -> torch.Tensor:
  """fp32 sum over the second-to-last dim: ``(.., R, N) -> (.., N)``."""
  if x.is_cuda and x.dtype == torch.bfloat16:
    n = x.shape[-1]
    if (x.dim() == 2 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.stride(0) >= n and
        (x.storage_offset() + x.shape[0] * x.stride(0)) * 2 <= x.untyped_storage().nbytes()):
      # A (rows, n) view of a row-padded buffer: sum the padded width, return the first n.
      ld = x.stride(0)
      full = torch.as_strided(x, (x.shape[0], ld), (ld, 1))
      return _colsum3(full.unsqueeze(0))[0, :n]
    x3 = (x.unsqueeze(0) if x.dim() == 2 else x).contiguous()
    if n % 8:
      return x.float().sum(dim=-2)
    out = _colsum3(x3)
    return out[0] if x.dim() == 2 else out
  return x.float().sum(dim=-2)
