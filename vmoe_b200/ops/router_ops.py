"""Fused gating of the noisy Top-K router on the GPU.

``gating_logits`` computes ``x @ W^T`` (bf16 operands, fp32 accumulation and output) on the
tcgen05 GEMM, with dgrad / wgrad GEMMs in backward. ``router_stats`` maps logits (+ standard
normal noise) to the softmax gates used for dispatch and the per-group importance, load and
GShard losses in two kernel launches, and back-propagates through all of them in one
(``csrc/router_kernels.cu``). The PyTorch formulation of the same maths lives in
``vmoe_b200/models/routing.py`` and is the oracle of the tests
(reference: ``vmoe/nn/routing.py:71-183``).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from vmoe_b200.ops import _lib
from vmoe_b200.ops import functional as fn
from vmoe_b200.ops.gemm import gemm

_vp = ctypes.c_void_p


class _GatingLogitsFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, weight):
    # x: (..., H) bf16; weight: (E, H) fp32 master with a bf16 shadow.
    w16 = fn.bf16_shadow(weight)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
      x2 = x2.contiguous()
    out = torch.empty(x2.shape[0], weight.shape[0], dtype=torch.float32, device=x.device)
    gemm(x2, w16, out=out)
    ctx.save_for_backward(x2, weight)
    ctx.x_shape = x.shape
    return out.reshape(*x.shape[:-1], weight.shape[0])

  @staticmethod
  def backward(ctx, dlogits):
    x2, weight = ctx.saved_tensors
    e, h = weight.shape
    d16 = dlogits.reshape(-1, e).to(torch.bfloat16)
    dx = dw = None
    if ctx.needs_input_grad[0]:
      dx = gemm(d16, fn.bf16_shadow(weight), b_mn_major=True).reshape(ctx.x_shape)
    if ctx.needs_input_grad[1]:
      dw = fn.wgrad(d16, x2, weight, split_k=fn._wgrad_split(e, h, d16.shape[0]))
    return dx, dw


def gating_logits_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
  return (x.is_cuda and x.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 and
          weight.shape[1] % 8 == 0 and fn.cuda_kernels_enabled())


def gating_logits(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
  return _GatingLogitsFn.apply(x, weight)


class _RouterStatsFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, logits, noise, noise_std, k):
    g, s, e = logits.shape
    logits = logits.contiguous()
    if noise is not None:
      noise = noise.contiguous().float()
    dev = logits.device
    gates = torch.empty_like(logits)
    sums = torch.empty(g, 4, e, dtype=torch.float32, device=dev)
    losses = torch.empty(g, 3, dtype=torch.float32, device=dev)
    coef = torch.empty(g, 3, e, dtype=torch.float32, device=dev)
    rc = _lib.lib().vmoe_router_stats_fwd(
        _vp(logits.data_ptr()), _vp(_lib.ptr(noise)), _vp(gates.data_ptr()),
        _vp(sums.data_ptr()), _vp(losses.data_ptr()), _vp(coef.data_ptr()),
        ctypes.c_int64(g * s), ctypes.c_int64(s), ctypes.c_int(e), ctypes.c_float(noise_std),
        ctypes.c_int(k), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_router_stats_fwd")
    _lib.count_launch(2)
    ctx.save_for_backward(logits, noise, coef)
    ctx.cfg = (noise_std, k)
    imp, load, gshard = losses.unbind(dim=1)
    return gates, imp, load, gshard

  @staticmethod
  def backward(ctx, d_gates, d_imp, d_load, d_gshard):
    logits, noise, coef = ctx.saved_tensors
    noise_std, k = ctx.cfg
    g, s, e = logits.shape
    d_losses = None
    if d_imp is not None or d_load is not None or d_gshard is not None:
      zero = torch.zeros(g, dtype=torch.float32, device=logits.device)
      d_losses = torch.stack([zero if d is None else d.float() for d in (d_imp, d_load, d_gshard)],
                             dim=1).contiguous()
    if d_gates is not None:
      d_gates = d_gates.contiguous().float()
    d_logits = torch.empty_like(logits)
    rc = _lib.lib().vmoe_router_stats_bwd(
        _vp(logits.data_ptr()), _vp(_lib.ptr(noise)), _vp(_lib.ptr(d_gates)),
        _vp(_lib.ptr(d_losses)), _vp(coef.data_ptr()), _vp(d_logits.data_ptr()), _vp(None),
        ctypes.c_int64(e), ctypes.c_int64(g * s), ctypes.c_int64(s), ctypes.c_int(e),
        ctypes.c_float(noise_std), ctypes.c_int(k), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_router_stats_bwd")
    _lib.count_launch()
    return d_logits, None, None, None


def router_stats_supported(logits: torch.Tensor) -> bool:
  return (logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 3 and
          logits.shape[-1] <= 64 and fn.cuda_kernels_enabled())


def router_stats(logits: torch.Tensor, noise: Optional[torch.Tensor], noise_std: float,
                 num_selected_experts: int
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
  """``logits (G, S, E)`` fp32, ``noise`` standard normal of the same shape or None.

  Returns ``(gates, importance_loss (G,), load_loss (G,), gshard_loss (G,))`` where ``gates``
  is ``softmax(logits + noise * noise_std)`` (or the clean softmax without noise), the load
  loss is zero without noise and the GShard loss is computed on ``gates``.
  """
  return _RouterStatsFn.apply(logits, noise, float(noise_std), int(num_selected_experts))


# ----------------------------------------------------------------------------- Soft MoE weights
class _SoftRouterWeightsFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, logits):
    g, m, s = logits.shape
    logits = logits.contiguous()
    dispatch = torch.empty_like(logits)
    combine = torch.empty_like(logits)
    rc = _lib.lib().vmoe_soft_router_fwd(
        _vp(logits.data_ptr()), _vp(dispatch.data_ptr()), _vp(combine.data_ptr()),
        ctypes.c_int64(g), ctypes.c_int32(m), ctypes.c_int32(s), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_soft_router_fwd")
    _lib.count_launch()
    ctx.save_for_backward(dispatch, combine)
    return dispatch, combine

  @staticmethod
  def backward(ctx, d_dispatch, d_combine):
    dispatch, combine = ctx.saved_tensors
    g, m, s = dispatch.shape
    if d_dispatch is None and d_combine is None:
      return None
    if d_dispatch is not None:
      d_dispatch = d_dispatch.contiguous().float()
    if d_combine is not None:
      d_combine = d_combine.contiguous().float()
    d_logits = torch.empty_like(dispatch)
    rc = _lib.lib().vmoe_soft_router_bwd(
        _vp(dispatch.data_ptr()), _vp(combine.data_ptr()), _vp(_lib.ptr(d_dispatch)),
        _vp(_lib.ptr(d_combine)), _vp(d_logits.data_ptr()), ctypes.c_int64(g),
        ctypes.c_int32(m), ctypes.c_int32(s), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_soft_router_bwd")
    _lib.count_launch()
    return d_logits


def soft_router_weights_supported(logits: torch.Tensor) -> bool:
  if not (logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 3 and
          fn.cuda_kernels_enabled()):
    return False
  _, m, s = logits.shape
  limit = _lib.lib().vmoe_soft_router_max_group_elements
  limit.restype = ctypes.c_int64
  return 0 < m <= 4096 and 0 < s <= 4096 and m * s <= int(limit())


def soft_router_weights(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
  """``logits (G, tokens, slots)`` fp32 -> ``(dispatch, combine)``: softmax over the tokens
  (axis 1) and softmax over the slots (axis 2), computed by one kernel per direction of the
  autograd graph (reference formulation: ``vmoe/projects/soft_moe/router.py:94-96``)."""
  return _SoftRouterWeightsFn.apply(logits)
