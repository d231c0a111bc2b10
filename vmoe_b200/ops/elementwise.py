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


class _EmbedFinalizeFn(torch.autograd.Function):
  """``concat(cls, emb) + pos`` in one kernel; backward sums the incoming gradient over the
  batch once (column sums of the ``(B, T*H)`` view) for the position embedding and the class
  token, and hands the patch rows back as a view."""

  @staticmethod
  def forward(ctx, emb, cls, pos):
    b, t, h = emb.shape
    has_cls = cls is not None
    emb = emb.contiguous()
    out = torch.empty(b, t + int(has_cls), h, dtype=torch.bfloat16, device=emb.device)
    rc = _lib.lib().vmoe_embed_finalize(
        _vp(emb.data_ptr()), _vp(_lib.ptr(None if cls is None else cls.contiguous())),
        _vp(_lib.ptr(None if pos is None else pos.contiguous())), _vp(out.data_ptr()),
        ctypes.c_int64(b), ctypes.c_int64(t), ctypes.c_int64(h), ctypes.c_int(int(has_cls)),
        _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_embed_finalize")
    _lib.count_launch()
    ctx.has_cls = has_cls
    ctx.shapes = (None if cls is None else cls.shape, None if pos is None else pos.shape)
    return out

  @staticmethod
  def backward(ctx, dout):
    from vmoe_b200.ops import reduce
    has_cls = ctx.has_cls
    cls_shape, pos_shape = ctx.shapes
    b, tt, h = dout.shape
    d_emb = dout[:, int(has_cls):] if ctx.needs_input_grad[0] else None
    d_cls = d_pos = None
    if ((cls_shape is not None and ctx.needs_input_grad[1]) or
        (pos_shape is not None and ctx.needs_input_grad[2])):
      total = reduce.colsum(dout.contiguous().reshape(b, tt * h)).reshape(tt, h)  # fp32
      if cls_shape is not None and ctx.needs_input_grad[1]:
        d_cls = total[0].reshape(cls_shape)
      if pos_shape is not None and ctx.needs_input_grad[2]:
        d_pos = total.reshape(pos_shape)
    return d_emb, d_cls, d_pos


def embed_finalize(emb: torch.Tensor, cls, pos) -> torch.Tensor:
  """``emb (B, T, H)`` bf16; ``cls (1, 1, H)`` fp32 or None; ``pos (1, T + has_cls, H)`` fp32 or
  None. Returns ``(B, T + has_cls, H)`` bf16."""
  return _EmbedFinalizeFn.apply(emb, cls, pos)


def mixup_supported(x: torch.Tensor, size: int) -> bool:
  from vmoe_b200.ops import functional
  return (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and 1 <= size <= 8 and
          x.numel() > 0 and functional.cuda_kernels_enabled())


def mixup_rows(x: torch.Tensor, weights: torch.Tensor, roll_axis: int) -> torch.Tensor:
  """``sum_i weights[i] * roll(x, -i, roll_axis)`` in one kernel. ``weights`` has shape
  ``(size,) + x.shape[:roll_axis + 1]`` (already broadcast over the leading dims); no gradient."""
  x = x.contiguous()
  size = weights.shape[0]
  lead = 1
  for d in x.shape[:roll_axis]:
    lead *= d
  batch = x.shape[roll_axis]
  inner = x.numel() // (lead * batch)
  w = weights.to(device=x.device, dtype=torch.float32).reshape(size, lead * batch).contiguous()
  out = torch.empty_like(x)
  rc = _lib.lib().vmoe_mixup(
      _vp(x.data_ptr()), _vp(out.data_ptr()), _vp(w.data_ptr()),
      ctypes.c_int32(int(x.dtype == torch.bfloat16)), ctypes.c_int64(lead), ctypes.c_int64(batch),
      ctypes.c_int64(inner), ctypes.c_int32(size), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_mixup")
  _lib.count_launch()
  return out
