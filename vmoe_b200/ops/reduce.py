"""Column sums (bias gradients) of bf16 matrices on the GPU, PyTorch elsewhere."""
from __future__ import annotations

import ctypes

import torch

from vmoe_b200.ops import _lib


def _colsum3(x3: torch.Tensor, out=None) -> torch.Tensor:
  b, r, n = x3.shape
  if out is None:
    out = torch.zeros(b, n, dtype=torch.float32, device=x3.device)
  rc = _lib.lib().vmoe_colsum_bf16(ctypes.c_void_p(x3.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                   ctypes.c_int64(b), ctypes.c_int64(r), ctypes.c_int64(n),
                                   ctypes.c_void_p(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_colsum_bf16")
  _lib.count_launch()
  return out


def colsum(x: torch.Tensor, out=None) -> torch.Tensor:
  """fp32 sum over the second-to-last dim: ``(.., R, N) -> (.., N)``.

  With ``out`` (fp32, contiguous) the sums are *added* to it.
  """
  if out is not None:
    if _direct_ok(x, out):
      x3 = (x.unsqueeze(0) if x.dim() == 2 else x).contiguous()
      _colsum3(x3, out=out.reshape(-1, x.shape[-1]))
    else:
      out.add_(_colsum(x).reshape(out.shape))
    return out
  return _colsum(x)


def _direct_ok(x, out) -> bool:
  return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and
          (x.dim() == 3 or x.is_contiguous()) and out.is_contiguous() and
          out.dtype == torch.float32)


def _colsum(x: torch.Tensor) -> torch.Tensor:
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
