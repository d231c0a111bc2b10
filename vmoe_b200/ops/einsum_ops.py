"""Dense (einsum) dispatch and combine of the MoE layer on the tcgen05 GEMM.

``dispatch``: ``out[g, n, h] = sum_s w[g, s, n] * x[g, s, h]`` and ``combine``:
``out[g, s, h] = sum_n w[g, s, n] * y[g, n, h]`` with ``n`` = flattened (expert, slot). With
real-valued weights (Soft MoE) these are true weighted sums, i.e. batched GEMMs with one small
problem per group; the kernel reads both operands in the layout they already have (MN-major
where needed), so no transposes are materialised, and backward is four more GEMMs of the same
kind. Weights are rounded to bf16 for the tensor cores; accumulation is fp32
(reference: the einsums of ``vmoe/moe.py:148-161``).
"""
from __future__ import annotations

import torch

from vmoe_b200.ops import functional as fn
from vmoe_b200.ops.gemm import gemm


def supported(w: torch.Tensor, data: torch.Tensor) -> bool:
  """``w (G, S, N)``, ``data (G, S or N, H)`` bf16 on CUDA with N and H multiples of 8."""
  return (fn.cuda_kernels_enabled() and data.is_cuda and data.dtype == torch.bfloat16 and
          w.is_cuda and w.dim() == 3 and data.dim() == 3 and w.shape[-1] % 8 == 0 and
          data.shape[-1] % 8 == 0 and w.shape[0] == data.shape[0])


def _w16(w: torch.Tensor) -> torch.Tensor:
  return w.to(torch.bfloat16).contiguous()


class _DispatchFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, w, x):
    w16, x = _w16(w), x.contiguous()
    ctx.save_for_backward(w16, x)
    ctx.w_dtype = w.dtype
    # a: (G, K=S, M=N) MN-major, b: (G, K=S, N=H) MN-major -> (G, N, H)
    return gemm(w16, x, a_mn_major=True, b_mn_major=True)

  @staticmethod
  def backward(ctx, dout):
    w16, x = ctx.saved_tensors
    dout = dout.contiguous()
    dw = dx = None
    if ctx.needs_input_grad[0]:
      # dw[g, s, n] = sum_h x[g, s, h] dout[g, n, h]
      dw = gemm(x, dout, out_dtype=torch.float32).to(ctx.w_dtype)
    if ctx.needs_input_grad[1]:
      # dx[g, s, h] = sum_n w[g, s, n] dout[g, n, h]
      dx = gemm(w16, dout, b_mn_major=True)
    return dw, dx


class _CombineFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, w, y):
    w16, y = _w16(w), y.contiguous()
    ctx.save_for_backward(w16, y)
    ctx.w_dtype = w.dtype
    # a: (G, M=S, K=N) K-major, b: (G, K=N, N=H) MN-major -> (G, S, H)
    return gemm(w16, y, b_mn_major=True)

  @staticmethod
  def backward(ctx, dout):
    w16, y = ctx.saved_tensors
    dout = dout.contiguous()
    dw = dy = None
    if ctx.needs_input_grad[0]:
      # dw[g, s, n] = sum_h dout[g, s, h] y[g, n, h]
      dw = gemm(dout, y, out_dtype=torch.float32).to(ctx.w_dtype)
    if ctx.needs_input_grad[1]:
      # dy[g, n, h] = sum_s w[g, s, n] dout[g, s, h]
      dy = gemm(w16, dout, a_mn_major=True, b_mn_major=True)
    return dw, dy


def dispatch(w: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
  """``w (G, S, N)``, ``x (G, S, H)`` -> ``(G, N, H)``."""
  return _DispatchFn.apply(w, x)


def combine(w: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
  """``w (G, S, N)``, ``y (G, N, H)`` -> ``(G, S, H)``."""
  return _CombineFn.apply(w, y)
