"""Image -> patch matrix conversion on the GPU (``csrc/elementwise.cu``)."""
from __future__ import annotations

import ctypes

import torch

from vmoe_b200.ops import _lib

_vp = ctypes.c_void_p


def patchify(images: torch.Tensor, ph: int, pw: int) -> torch.Tensor:
  """NHWC ``(B, H, W, C)`` fp32/bf16 -> bf16 ``(B, gh*gw, ph*pw*C)`` (no gradient)."""
  assert images.is_cuda and images.dtype in (torch.float32, torch.bfloat16)
  images = images.contiguous()
  b, hh, ww, c = images.shape
  gh, gw = hh // ph, ww // pw
  out = torch.empty(b, gh * gw, ph * pw * c, dtype=torch.bfloat16, device=images.device)
  rc = _lib.lib().vmoe_patchify(
      _vp(images.data_ptr()), ctypes.c_int32(int(images.dtype == torch.bfloat16)),
      _vp(out.data_ptr()), ctypes.c_int64(b), ctypes.c_int64(hh), ctypes.c_int64(ww),
      ctypes.c_int64(c), ctypes.c_int64(ph), ctypes.c_int64(pw), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_patchify")
  _lib.count_launch()
  return out
