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


def _rows(t: torch.Tensor) -> torch.Tensor:
  """``t`` itself when the GEMM can read it in place (rows contiguous, every other stride and
  the base address a multiple of 16 bytes), else a contiguous copy. Expert-major buffers viewed
  group-major (``(E, G, H)`` seen as ``(G, E, H)``) pass, which saves the transposing copies
  around the experts when every expert has one slot."""
  if (t.stride(-1) == 1 and all(st % 8 == 0 for st in t.stride()[:-1]) and
      t.data_ptr() % 16 == 0):
    return t
  return t.contiguous()


def _slot_major_out(g: int, n: int, h: int, like: torch.Tensor, slots: int) -> torch.Tensor:
  """Output buffer of shape ``(G, N, H)``. With one slot per expert it is laid out ``(N, G, H)``
  in memory, i.e. already expert-major: the transpose that follows is then a view."""
  if slots == 1:
    return torch.empty(n, g, h, dtype=like.dtype, device=like.device).transpose(0, 1)
  return torch.empty(g, n, h, dtype=like.dtype, device=like.device)


class _DispatchFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, w, x, slots):
    w16, x = _w16(w), _rows(x)
    ctx.save_for_backward(w16, x)
    ctx.w_dtype = w.dtype
    # a: (G, K=S, M=N) MN-major, b: (G, K=S, N=H) MN-major -> (G, N, H)
    out = _slot_major_out(w.shape[0], w.shape[2], x.shape[2], x, slots)
    return gemm(w16, x, a_mn_major=True, b_mn_major=True, out=out)

  @staticmethod
  def backward(ctx, dout):
    w16, x = ctx.saved_tensors
    dout = _rows(dout)
    dw = dx = None
    if ctx.needs_input_grad[0]:
      # dw[g, s, n] = sum_h x[g, s, h] dout[g, n, h]
      dw = gemm(x, dout, out_dtype=torch.float32).to(ctx.w_dtype)
    if ctx.needs_input_grad[1]:
      # dx[g, s, h] = sum_n w[g, s, n] dout[g, n, h]
      dx = gemm(w16, dout, b_mn_major=True)
    return dw, dx, None


class _CombineFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, w, y, slots):
    w16, y = _w16(w), _rows(y)
    ctx.save_for_backward(w16, y)
    ctx.w_dtype = w.dtype
    ctx.slots = slots
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
      out = _slot_major_out(w16.shape[0], w16.shape[2], dout.shape[2], dout, ctx.slots)
      dy = gemm(w16, dout, a_mn_major=True, b_mn_major=True, out=out)
    return dw, dy, None


def dispatch(w: torch.Tensor, x: torch.Tensor, slots_per_expert: int = 0) -> torch.Tensor:
  """``w (G, S, N)``, ``x (G, S, H)`` -> ``(G, N, H)``. ``slots_per_expert`` = 1 lays the result
  out expert-major in memory (a hint: values and shape are the same)."""
  return _DispatchFn.apply(w, x, slots_per_expert)


def combine(w: torch.Tensor, y: torch.Tensor, slots_per_expert: int = 0) -> torch.Tensor:
  """``w (G, S, N)``, ``y (G, N, H)`` -> ``(G, S, H)``; the hint lays out the gradient of ``y``."""
  return _CombineFn.apply(w, y, slots_per_expert)
