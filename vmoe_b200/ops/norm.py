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
    ctx.bias_ref = bias
    ctx.shape = x.shape
    return y.reshape(x.shape)

  @staticmethod
  def backward(ctx, dy):
    return _backward(ctx, dy, None) + (None,)


def _grad_or_new(p, h, device):
  """``(buffer the kernel accumulates into, value to hand to autograd)`` for dgamma / dbeta:
  the parameter's bound fp32 gradient when there is one (nothing returned to autograd), else
  a fresh zero tensor."""
  from vmoe_b200.ops.functional import _grad_target
  if p is None:
    return None, None
  tgt = _grad_target(p)
  if tgt is not None:
    return tgt, None
  new = torch.zeros(h, dtype=torch.float32, device=device)
  return new, new


def _backward(ctx, dy, dres):
  x2, weight, mean, rstd = ctx.saved_tensors
  rows, h = x2.shape
  if dy is None:
    dy = torch.zeros_like(x2)
  dy2 = dy.reshape(rows, h)
  if not dy2.is_contiguous():
    dy2 = dy2.contiguous()
  if dres is not None:
    dres = dres.reshape(rows, h)
    if not dres.is_contiguous() or dres.dtype != torch.bfloat16:
      dres = dres.contiguous().to(torch.bfloat16)
  dx = torch.empty_like(x2)
  dgamma_buf, dgamma = _grad_or_new(weight, h, dy.device)
  dbeta_buf, dbeta = _grad_or_new(ctx.bias_ref if ctx.has_bias else None, h, dy.device)
  lib = _lib.lib()
  lib.vmoe_layernorm_bwd_scratch_bytes.restype = ctypes.c_int64
  nbytes = lib.vmoe_layernorm_bwd_scratch_bytes(ctypes.c_int64(rows), ctypes.c_int64(h))
  scratch = torch.empty(max(int(nbytes) // 4, 1), dtype=torch.float32, device=dy.device)
  rc = lib.vmoe_layernorm_bwd(
      _vp(dy2.data_ptr()), _vp(x2.data_ptr()), _vp(_lib.ptr(weight)), _vp(mean.data_ptr()),
      _vp(rstd.data_ptr()), _vp(_lib.ptr(dres)), _vp(dx.data_ptr()), _vp(_lib.ptr(dgamma_buf)),
      _vp(_lib.ptr(dbeta_buf)), _vp(scratch.data_ptr()), ctypes.c_int64(rows), ctypes.c_int64(h),
      _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_layernorm_bwd")
  _lib.count_launch(2)
  return dx.reshape(ctx.shape), dgamma, dbeta


class _LayerNormForkFn(_LayerNormFn):
  """``(LayerNorm(x), x)``: the second output is ``x`` itself, for the residual branch. Because
  both consumers hang off this one node, backward receives both gradients at once and the
  kernel adds the residual gradient while it writes dx, instead of autograd running a separate
  full-size add."""

  @staticmethod
  def forward(ctx, x, weight, bias, eps):
    y = _LayerNormFn.forward(ctx, x, weight, bias, eps)
    return y, x.view_as(x)

  @staticmethod
  def backward(ctx, dy, dres):
    return _backward(ctx, dy, dres) + (None,)


def layer_norm(x, weight, bias, eps=1e-6):
  assert weight is None or weight.dtype == torch.float32
  return _LayerNormFn.apply(x, weight, bias, eps)


def layer_norm_fork(x, weight, bias, eps=1e-6):
  """Returns ``(LayerNorm(x), x)``; use the second value for the residual connection."""
  assert weight is None or weight.dtype == torch.float32
  return _LayerNormForkFn.apply(x, weight, bias, eps)


class _QKNormPackedFn(torch.autograd.Function):
  """LayerNorm over the head dimension of the q and k slices of a packed ``(B, T, 3, H, D)``
  projection, written straight into a new packed tensor (v is copied). The kernels address the
  slices in place, so neither direction materialises contiguous copies of q / k or re-stacks
  the result."""

  @staticmethod
  def forward(ctx, qkv, wq, wk, eps):
    b, t, three, h, d = qkv.shape
    assert three == 3 and qkv.is_contiguous()
    out = torch.empty_like(qkv)
    rows = b * t * h
    outer = 3 * h * d
    stats = torch.empty(4, rows, dtype=torch.float32, device=qkv.device)
    lib = _lib.lib()
    es = qkv.element_size()
    for i, w in enumerate((wq, wk)):
      rc = lib.vmoe_layernorm_fwd_strided(
          _vp(qkv.data_ptr() + i * h * d * es), _vp(_lib.ptr(w)), _vp(None),
          _vp(out.data_ptr() + i * h * d * es), _vp(stats[2 * i].data_ptr()),
          _vp(stats[2 * i + 1].data_ptr()), ctypes.c_int64(rows), ctypes.c_int64(d),
          ctypes.c_float(eps), ctypes.c_int64(h), ctypes.c_int64(outer), ctypes.c_int64(outer),
          _vp(_lib.stream_ptr()))
      _lib.check(rc, "vmoe_layernorm_fwd_strided")
    _lib.count_launch(2)
    out[:, :, 2].copy_(qkv[:, :, 2])
    ctx.save_for_backward(qkv, wq, wk, stats)
    return out

  @staticmethod
  def backward(ctx, dout):
    qkv, wq, wk, stats = ctx.saved_tensors
    b, t, _, h, d = qkv.shape
    dout = dout.contiguous()
    dqkv = torch.empty_like(qkv)
    rows, outer, es = b * t * h, 3 * h * d, qkv.element_size()
    lib = _lib.lib()
    lib.vmoe_layernorm_bwd_scratch_bytes.restype = ctypes.c_int64
    nbytes = lib.vmoe_layernorm_bwd_scratch_bytes(ctypes.c_int64(rows), ctypes.c_int64(d))
    scratch = torch.empty(max(int(nbytes) // 4, 1), dtype=torch.float32, device=qkv.device)
    grads = []
    for i, w in enumerate((wq, wk)):
      buf, ret = _grad_or_new(w, d, qkv.device)
      rc = lib.vmoe_layernorm_bwd_strided(
          _vp(dout.data_ptr() + i * h * d * es), _vp(qkv.data_ptr() + i * h * d * es),
          _vp(_lib.ptr(w)), _vp(stats[2 * i].data_ptr()), _vp(stats[2 * i + 1].data_ptr()),
          _vp(dqkv.data_ptr() + i * h * d * es), _vp(_lib.ptr(buf)), _vp(None),
          _vp(scratch.data_ptr()), ctypes.c_int64(rows), ctypes.c_int64(d), ctypes.c_int64(h),
          ctypes.c_int64(outer), ctypes.c_int64(outer), ctypes.c_int64(outer),
          _vp(_lib.stream_ptr()))
      _lib.check(rc, "vmoe_layernorm_bwd_strided")
      grads.append(ret)
    _lib.count_launch(4)
    dqkv[:, :, 2].copy_(dout[:, :, 2])
    return dqkv, grads[0], grads[1], None


def qk_norm_packed_supported(qkv, wq, wk, bias_q, bias_k) -> bool:
  return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 5 and qkv.shape[2] == 3
          and qkv.shape[-1] in (16, 32, 64, 128) and qkv.is_contiguous() and bias_q is None
          and bias_k is None and wq is not None and wk is not None
          and wq.dtype == torch.float32 and wk.dtype == torch.float32)


def qk_norm_packed(qkv, wq, wk, eps=1e-6):
  """Packed ``(B, T, 3, H, D)`` with LayerNorm (scale only) applied to q and k per head."""
  return _QKNormPackedFn.apply(qkv, wq, wk, eps)
