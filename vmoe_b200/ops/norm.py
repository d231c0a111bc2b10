"""LayerNorm on the fused CUDA kernels (``csrc/elementwise.cu``), differentiable."""
from __future__ import annotations

import ctypes

import torch

from vmoe_b200.ops import _lib

_vp = ctypes.c_void_p


class _LayerNormFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, weight, bias, eps):
    h = x.shape[-1]
    x2 = x.reshape(-1, h)
    if not x2.is_contiguous():
      x2 = x2.contiguous()
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    need = any(ctx.needs_input_grad)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device) if need else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if need else None
    rc = _lib.lib().vmoe_layernorm_fwd(
        _vp(x2.data_ptr()), _vp(_lib.ptr(weight)), _vp(_lib.ptr(bias)), _vp(y.data_ptr()),
        _vp(_lib.ptr(mean)), _vp(_lib.ptr(rstd)), ctypes.c_int64(rows), ctypes.c_int64(h),
        ctypes.c_float(eps), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_layernorm_fwd")
    _lib.count_launch()
    ctx.save_for_backward(x2, weight, mean, rstd)
    ctx.has_bias = bias is not None
    ctx.shape = x.shape
    return y.reshape(x.shape)

  @staticmethod
  def backward(ctx, dy):
    x2, weight, mean, rstd = ctx.saved_tensors
    rows, h = x2.shape
    dy2 = dy.reshape(rows, h)
    if not dy2.is_contiguous():
      dy2 = dy2.contiguous()
    dx = torch.empty_like(x2)
    dgamma = torch.zeros(h, dtype=torch.float32, device=dy.device) if weight is not None else None
    dbeta = torch.zeros(h, dtype=torch.float32, device=dy.device) if ctx.has_bias else None
    lib = _lib.lib()
    lib.vmoe_layernorm_bwd_scratch_bytes.restype = ctypes.c_int64
    nbytes = lib.vmoe_layernorm_bwd_scratch_bytes(ctypes.c_int64(rows), ctypes.c_int64(h))
    scratch = torch.empty(max(int(nbytes) // 4, 1), dtype=torch.float32, device=dy.device)
    rc = lib.vmoe_layernorm_bwd(
        _vp(dy2.data_ptr()), _vp(x2.data_ptr()), _vp(_lib.ptr(weight)), _vp(mean.data_ptr()),
        _vp(rstd.data_ptr()), _vp(None), _vp(dx.data_ptr()), _vp(_lib.ptr(dgamma)),
        _vp(_lib.ptr(dbeta)), _vp(scratch.data_ptr()), ctypes.c_int64(rows), ctypes.c_int64(h),
        _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_layernorm_bwd")
    _lib.count_launch(2)
    return dx.reshape(ctx.shape), dgamma, dbeta, None


def layer_norm(x, weight, bias, eps=1e-6):
  assert weight is None or weight.dtype == torch.float32
  return _LayerNormFn.apply(x, weight, bias, eps)
