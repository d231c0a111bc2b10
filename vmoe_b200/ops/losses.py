"""Classification losses with a fused forward+backward GPU kernel (``csrc/train_kernels.cu``).

``sigmoid_xent`` sums the binary cross-entropy over classes, ``softmax_xent`` is the softmax
cross-entropy with soft labels; both return one value per example (reference:
``vmoe/train/trainer.py:441-477``).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from vmoe_b200.ops import _lib
from vmoe_b200.ops import functional

_vp = ctypes.c_void_p
_LABEL_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.uint8: 2, torch.bool: 2}


class _XentFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, logits, labels, kind):
    n = logits.shape[-1]
    lg = logits.reshape(-1, n)
    lb = labels.reshape(-1, n)
    assert lg.stride(-1) == 1 and lb.stride(-1) == 1
    rows, ld = lg.shape[0], lg.stride(0)
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    need = ctx.needs_input_grad[0]
    # The gradient keeps the (possibly padded) row stride of the logits; padding gets zeros.
    dfull = torch.empty(rows, ld, dtype=torch.bfloat16, device=logits.device) if need else None
    rc = _lib.lib().vmoe_xent(
        ctypes.c_int32(kind), _vp(lg.data_ptr()), _vp(lb.data_ptr()),
        ctypes.c_int32(_LABEL_CODES[lb.dtype]), _vp(loss.data_ptr()), _vp(_lib.ptr(dfull)),
        ctypes.c_int64(rows), ctypes.c_int64(n), ctypes.c_int64(ld),
        ctypes.c_int64(lb.stride(0)), ctypes.c_float(1.0), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_xent")
    _lib.count_launch()
    ctx.save_for_backward(dfull)
    ctx.shape = logits.shape
    return loss.reshape(logits.shape[:-1])

  @staticmethod
  def backward(ctx, dloss):
    (dfull,) = ctx.saved_tensors
    n = ctx.shape[-1]
    g = dfull * dloss.reshape(-1, 1).to(dfull.dtype)
    return g[:, :n], None, None


def _fast(logits, labels) -> bool:
  return (functional.cuda_kernels_enabled() and logits.is_cuda and
          logits.dtype == torch.bfloat16 and labels.dtype in _LABEL_CODES and
          logits.dim() == 2 and logits.stride(-1) == 1 and labels.shape == logits.shape)


def sigmoid_xent(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
  if _fast(logits, labels):
    return _XentFn.apply(logits, labels.contiguous(), 0)
  x = logits.float()
  return F.binary_cross_entropy_with_logits(x, labels.float(), reduction="none").sum(-1)


def softmax_xent(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
  if _fast(logits, labels):
    return _XentFn.apply(logits, labels.contiguous(), 1)
  return -(labels.float() * F.log_softmax(logits.float(), dim=-1)).sum(-1)
