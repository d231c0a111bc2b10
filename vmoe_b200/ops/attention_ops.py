"""Fused softmax attention on the tcgen05 kernels (``csrc/attention_tcgen05.cu``).

The kernels cover what the shipped ViT configs need on the hot path: self-attention with head
dim 64 and up to 256 tokens (50, 197, 257 -> only the 64-dim ones), reading Q, K and V out of
the packed ``(B, T, 3, H, 64)`` output of the fused QKV projection and writing the packed QKV
gradient, so no slicing or concatenation copies surround the kernel. Other shapes use the
PyTorch formulation in ``vmoe_b200.ops.functional.attention``.
"""
from __future__ import annotations

import ctypes
import math

import torch

from vmoe_b200.ops import _lib

_vp = ctypes.c_void_p


class AttnArgs(ctypes.Structure):
  _fields_ = [
      ("q", _vp), ("k", _vp), ("v", _vp), ("out", _vp), ("lse", _vp), ("d_out", _vp),
      ("dq", _vp), ("dk", _vp), ("dv", _vp), ("status", _vp),
      ("B", ctypes.c_int64), ("H", ctypes.c_int64), ("T", ctypes.c_int64), ("D", ctypes.c_int64),
      ("q_tok", ctypes.c_int64), ("q_head", ctypes.c_int64), ("q_batch", ctypes.c_int64),
      ("o_tok", ctypes.c_int64), ("o_head", ctypes.c_int64), ("o_batch", ctypes.c_int64),
      ("g_tok", ctypes.c_int64), ("g_head", ctypes.c_int64), ("g_batch", ctypes.c_int64),
      ("scale", ctypes.c_float),
  ]


def packed_supported(qkv: torch.Tensor) -> bool:
  """``qkv``: (B, T, 3, H, D) bf16 CUDA, contiguous, D == 64, T <= 256."""
  return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 5 and qkv.shape[2] == 3 and
          qkv.shape[4] == 64 and 1 <= qkv.shape[1] <= 256 and qkv.is_contiguous())


def _fill_common(args, qkv, out, lse):
  b, t, _, h, d = qkv.shape
  es = qkv.element_size()
  base = qkv.data_ptr()
  args.q, args.k, args.v = base, base + h * d * es, base + 2 * h * d * es
  args.out, args.lse = out.data_ptr(), lse.data_ptr()
  args.B, args.H, args.T, args.D = b, h, t, d
  args.q_tok, args.q_head, args.q_batch = 3 * h * d, d, t * 3 * h * d
  args.o_tok, args.o_head, args.o_batch = h * d, d, t * h * d
  args.scale = 1.0 / math.sqrt(d)


class _PackedAttentionFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, qkv):
    b, t, _, h, d = qkv.shape
    out = torch.empty(b, t, h, d, dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty(b, h, t, dtype=torch.float32, device=qkv.device)
    args = AttnArgs()
    _fill_common(args, qkv, out, lse)
    rc = _lib.lib().vmoe_attention_fwd(ctypes.byref(args), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_attention_fwd")
    _lib.count_launch()
    ctx.save_for_backward(qkv, out, lse)
    return out

  @staticmethod
  def backward(ctx, d_out):
    qkv, out, lse = ctx.saved_tensors
    b, t, _, h, d = qkv.shape
    d_out = d_out.contiguous()
    dqkv = torch.empty_like(qkv)
    args = AttnArgs()
    _fill_common(args, qkv, out, lse)
    es = qkv.element_size()
    args.d_out = d_out.data_ptr()
    gb = dqkv.data_ptr()
    args.dq, args.dk, args.dv = gb, gb + h * d * es, gb + 2 * h * d * es
    args.g_tok, args.g_head, args.g_batch = 3 * h * d, d, t * 3 * h * d
    rc = _lib.lib().vmoe_attention_bwd(ctypes.byref(args), _vp(_lib.stream_ptr()))
    _lib.check(rc, "vmoe_attention_bwd")
    _lib.count_launch()
    return dqkv


def packed_attention(qkv: torch.Tensor) -> torch.Tensor:
  """Self-attention on packed projections: (B, T, 3, H, 64) -> (B, T, H, 64)."""
  return _PackedAttentionFn.apply(qkv)
