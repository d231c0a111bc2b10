"""Fused softmax attention on the tcgen05 kernels (``csrc/attention_tcgen05.cu``).

The kernels cover the attention shapes of the shipped Vision Transformers: any number of
queries, up to about 700 keys, head dims 16..80 in steps of 16 (ViT-S/B/L use 64, ViT-H 80),
optional dropout of the attention weights, self-attention on the packed ``(B, T, 3, H, D)``
output of the fused QKV projection (the backward pass writes the packed gradient, so no slicing
or concatenation copies surround the kernel) and attention with separate query and key / value
tensors (the pooling head's probe attending over the tokens). Anything else uses the PyTorch
formulation in ``vmoe_b200.ops.functional.attention``.

The dropout mask is not stored: it is a hash of (seed, batch, head, query, key) that the
backward kernel evaluates again; ``dropout_keep_mask`` restates it in PyTorch for tests.
"""
from __future__ import annotations

import ctypes
import math

import torch

from vmoe_b200.ops import _lib

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64


class AttnArgs(ctypes.Structure):
  _fields_ = [
      ("q", _vp), ("k", _vp), ("v", _vp), ("out", _vp), ("lse", _vp), ("d_out", _vp),
      ("dq", _vp), ("dk", _vp), ("dv", _vp), ("status", _vp),
      ("B", _i64), ("H", _i64), ("T", _i64), ("D", _i64),
      ("q_tok", _i64), ("q_head", _i64), ("q_batch", _i64),
      ("o_tok", _i64), ("o_head", _i64), ("o_batch", _i64),
      ("g_tok", _i64), ("g_head", _i64), ("g_batch", _i64),
      ("scale", ctypes.c_float), ("dropout_p", ctypes.c_float),
      ("Tk", _i64),
      ("kv_tok", _i64), ("kv_head", _i64), ("kv_batch", _i64),
      ("gkv_tok", _i64), ("gkv_head", _i64), ("gkv_batch", _i64),
      ("seed", ctypes.c_uint64),
      ("dq_acc", _vp),
  ]


def shape_supported(tq: int, tk: int, d: int) -> bool:
  return bool(_lib.lib().vmoe_attention_supported(_i64(tq), _i64(tk), _i64(d)))


def packed_supported(qkv: torch.Tensor) -> bool:
  """``qkv``: (B, T, 3, H, D) bf16 CUDA, contiguous, of a shape the kernels cover."""
  return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 5 and qkv.shape[2] == 3 and
          qkv.is_contiguous() and shape_supported(qkv.shape[1], qkv.shape[1], qkv.shape[4]))


def separate_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
  """``q``: (B, Tq, H, D), ``k``, ``v``: (B, Tk, H, D), bf16 CUDA."""
  return (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16 and q.dim() == 4 and
          k.shape == v.shape and shape_supported(q.shape[1], k.shape[1], q.shape[3]))


def new_seed() -> int:
  """A dropout seed drawn from PyTorch's CPU generator (reproducible under manual_seed)."""
  return int(torch.randint(0, 2 ** 62, (1,)).item())


def _mix32(x: torch.Tensor) -> torch.Tensor:
  m = 0xFFFFFFFF
  x = x ^ (x >> 16)
  x = (x * 0x7FEB352D) & m
  x = x ^ (x >> 15)
  x = (x * 0x846CA68B) & m
  return x ^ (x >> 16)


def dropout_keep_quantum(dropout_p: float) -> int:
  """Keep probability in 1/256ths as the kernels apply it."""
  if dropout_p <= 0:
    return 256
  return max(1, min(256, int((1.0 - dropout_p) * 256.0 + 0.5)))


def dropout_keep_mask(seed: int, b: int, h: int, tq: int, tk: int, dropout_p: float,
                      device="cpu") -> torch.Tensor:
  """The kernels' keep mask as a bool tensor (B, H, Tq, Tk)."""
  keep_q = dropout_keep_quantum(dropout_p)
  bh = torch.arange(b * h, dtype=torch.int64, device=device).reshape(b * h, 1, 1)
  q = torch.arange(tq, dtype=torch.int64, device=device).reshape(1, tq, 1)
  k = torch.arange(tk, dtype=torch.int64, device=device).reshape(1, 1, tk)
  idx = ((bh * tq + q) * ((tk + 3) // 4) + k // 4) & 0xFFFFFFFF
  word = _mix32(_mix32(idx ^ (seed & 0xFFFFFFFF)) ^ ((seed >> 32) & 0xFFFFFFFF))
  byte = (word >> (8 * (k % 4))) & 0xFF
  return (byte < keep_q).reshape(b, h, tq, tk)


_STATUS: dict = {}


def status_word(device) -> torch.Tensor:
  """Device status word that the attention kernels OR their wait-timeout bits into (one per
  device; zero while every bounded wait completed)."""
  key = torch.device(device).index or 0
  t = _STATUS.get(key)
  if t is None:
    t = torch.zeros(1, dtype=torch.int32, device=device)
    _STATUS[key] = t
  return t


def _strides(t: torch.Tensor):
  """(tok, head, batch) element strides of a (B, T, H, D) tensor view."""
  assert t.stride(3) == 1
  return t.stride(1), t.stride(2), t.stride(0)


def _launch(fn_name, args):
  rc = getattr(_lib.lib(), fn_name)(ctypes.byref(args), _vp(_lib.stream_ptr()))
  _lib.check(rc, fn_name)
  _lib.count_launch()


def _dq_acc(b, tq, h, d, device):
  if _lib.lib().vmoe_attention_bwd_needs_dq_acc(_i64(tq), _i64(d)):
    return torch.zeros(b, tq, h, d, dtype=torch.float32, device=device)
  return None


class _AttentionFn(torch.autograd.Function):
  """q: (B, Tq, H, D) view, k / v: (B, Tk, H, D) views with equal strides (e.g. slices of one
  packed projection). Returns (B, Tq, H, D)."""

  @staticmethod
  def forward(ctx, q, k, v, dropout_p, seed, packed_grad):
    b, tq, h, d = q.shape
    tk = k.shape[1]
    assert k.stride() == v.stride()
    out = torch.empty(b, tq, h, d, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(b, h, tq, dtype=torch.float32, device=q.device)
    args = AttnArgs()
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    args.out, args.lse = out.data_ptr(), lse.data_ptr()
    args.B, args.H, args.T, args.D, args.Tk = b, h, tq, d, tk
    args.q_tok, args.q_head, args.q_batch = _strides(q)
    args.kv_tok, args.kv_head, args.kv_batch = _strides(k)
    args.o_tok, args.o_head, args.o_batch = _strides(out)
    args.scale = 1.0 / math.sqrt(d)
    args.dropout_p, args.seed = float(dropout_p), int(seed)
    args.status = status_word(q.device).data_ptr()
    _launch("vmoe_attention_fwd", args)
    ctx.save_for_backward(q, k, v, out, lse)
    ctx.conf = (float(dropout_p), int(seed), packed_grad)
    return out

  @staticmethod
  def backward(ctx, d_out):
    q, k, v, out, lse = ctx.saved_tensors
    dropout_p, seed, packed_grad = ctx.conf
    b, tq, h, d = q.shape
    tk = k.shape[1]
    d_out = d_out.contiguous()
    if packed_grad:
      # q, k, v are the three slices of one (B, T, 3, H, D) tensor: one packed gradient.
      dqkv = torch.empty(b, tq, 3, h, d, dtype=torch.bfloat16, device=q.device)
      dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
    else:
      dq = torch.empty(b, tq, h, d, dtype=torch.bfloat16, device=q.device)
      dkv = torch.empty(b, tk, 2, h, d, dtype=torch.bfloat16, device=q.device)
      dk, dv = dkv[:, :, 0], dkv[:, :, 1]
    acc = _dq_acc(b, tq, h, d, q.device)
    args = AttnArgs()
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    args.out, args.lse, args.d_out = out.data_ptr(), lse.data_ptr(), d_out.data_ptr()
    args.dq, args.dk, args.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    args.dq_acc = _lib.ptr(acc)
    args.B, args.H, args.T, args.D, args.Tk = b, h, tq, d, tk
    args.q_tok, args.q_head, args.q_batch = _strides(q)
    args.kv_tok, args.kv_head, args.kv_batch = _strides(k)
    args.o_tok, args.o_head, args.o_batch = _strides(out)
    args.g_tok, args.g_head, args.g_batch = _strides(dq)
    args.gkv_tok, args.gkv_head, args.gkv_batch = _strides(dk)
    args.scale = 1.0 / math.sqrt(d)
    args.dropout_p, args.seed = dropout_p, seed
    args.status = status_word(q.device).data_ptr()
    _launch("vmoe_attention_bwd", args)
    if packed_grad:
      return dqkv, None, None, None, None, None
    return dq, dk, dv, None, None, None


class _PackedFn(torch.autograd.Function):
  """Self-attention on the packed projection; autograd sees one input and one packed gradient."""

  @staticmethod
  def forward(ctx, qkv, dropout_p, seed):
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    return _AttentionFn.forward(ctx, q, k, v, dropout_p, seed, True)

  @staticmethod
  def backward(ctx, d_out):
    return _AttentionFn.backward(ctx, d_out)[0], None, None


def packed_attention(qkv: torch.Tensor, dropout_p: float = 0.0, seed: int = 0) -> torch.Tensor:
  """Self-attention on packed projections: (B, T, 3, H, D) -> (B, T, H, D)."""
  return _PackedFn.apply(qkv, float(dropout_p), int(seed))


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dropout_p: float = 0.0,
              seed: int = 0) -> torch.Tensor:
  """(B, Tq, H, D), (B, Tk, H, D) x 2 -> (B, Tq, H, D). ``k`` and ``v`` with different strides
  are copied into one packed tensor first."""
  if q.stride(3) != 1:
    q = q.contiguous()
  if k.stride() != v.stride() or k.stride(3) != 1:
    kv = torch.stack([k, v], dim=2)
    k, v = kv[:, :, 0], kv[:, :, 1]
  return _AttentionFn.apply(q, k, v, float(dropout_p), int(seed), False)
