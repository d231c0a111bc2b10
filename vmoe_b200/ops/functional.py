"""Differentiable front-ends of the hot ops.

Dispatch rule: a CUDA bf16 input with kernels enabled runs the sm_100a kernels (and raises if
the library is missing — there is no silent fallback on a GPU); anything else runs PyTorch.
"""
from __future__ import annotations

import contextlib
import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from vmoe_b200.ops import reduce
from vmoe_b200.ops.gemm import ACT_GELU, ACT_NONE, gemm

_ENABLED = os.environ.get("VMOE_B200_KERNELS", "1") != "0"


def cuda_kernels_enabled() -> bool:
  return _ENABLED


@contextlib.contextmanager
def use_cuda_kernels(enabled: bool):
  """Temporarily switches the CUDA kernels on/off (off = PyTorch library ops, the baseline)."""
  global _ENABLED
  prev, _ENABLED = _ENABLED, enabled
  try:
    yield
  finally:
    _ENABLED = prev


def _fast(x: torch.Tensor) -> bool:
  return _ENABLED and x.is_cuda and x.dtype == torch.bfloat16


def bf16_shadow(p: torch.Tensor) -> torch.Tensor:
  """bf16 copy of an fp32 master parameter, refreshed when the parameter changes.

  The fused optimizer refreshes shadows in the same kernel that updates the master weights
  (it bumps ``_shadow_version``), so the cast below only runs after out-of-band changes.
  """
  if p.dtype == torch.bfloat16:
    return p.detach()
  sh = getattr(p, "_bf16_shadow", None)
  ver = p._version
  if sh is None or getattr(p, "_shadow_version", -1) != ver or sh.shape != p.shape:
    if sh is None or sh.shape != p.shape or sh.device != p.device:
      sh = torch.empty_like(p, dtype=torch.bfloat16)
      p._bf16_shadow = sh
    sh.copy_(p.detach())
    p._shadow_version = ver
  return sh


def _grad_target(p: torch.Tensor):
  """The fp32 gradient buffer of a parameter if one is bound (flat optimizer buffers), so the
  weight-gradient GEMM can accumulate into it in place instead of going through autograd's
  allocate + add."""
  if not p.is_leaf:
    return None  # an intermediate result used as a weight: autograd owns its gradient
  g = getattr(p, "grad", None)
  if (g is not None and g.dtype == torch.float32 and g.shape == p.shape and g.is_contiguous()
      and not g.requires_grad):
    return g
  return None


def wgrad(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, split_k: int = 1):
  """dW = dy^T x for ``weight`` (.., N, K); returns None if accumulated into ``weight.grad``."""
  tgt = _grad_target(weight)
  if tgt is not None:
    gemm(dy, x, a_mn_major=True, b_mn_major=True, out=tgt, accumulate=True, split_k=split_k)
    return None
  dw = torch.zeros(weight.shape, dtype=torch.float32, device=dy.device)
  gemm(dy, x, a_mn_major=True, b_mn_major=True, out=dw, accumulate=True, split_k=split_k)
  return dw


def bias_grad(dy: torch.Tensor, bias: torch.Tensor):
  """Column sums of ``dy`` for ``bias``; None if accumulated into ``bias.grad``."""
  tgt = _grad_target(bias)
  if tgt is not None:
    reduce.colsum(dy, out=tgt)
    return None
  return reduce.colsum(dy)


# ----------------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
  """y = act(x W^T + b) (+ residual) on the tcgen05 GEMM; backward = dgrad + wgrad GEMMs."""

  @staticmethod
  def forward(ctx, x, weight, bias, residual, act):
    w16 = bf16_shadow(weight)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
      x2 = x2.contiguous()
    k_pad = (-x2.shape[1]) % 8
    if k_pad:
      # TMA needs 16-byte aligned rows: zero-pad the contraction dim (e.g. 14x14x3 patches).
      x2 = F.pad(x2, (0, k_pad))
      w16 = F.pad(w16, (0, k_pad))
    ctx.k_pad = k_pad
    need_grad = any(ctx.needs_input_grad)
    n = weight.shape[0]
    pre = None
    if act == ACT_GELU and need_grad:
      pre = torch.empty(x2.shape[0], n, dtype=torch.bfloat16, device=x.device)
    res2 = residual.reshape(-1, n) if residual is not None else None
    out = None
    if n % 8:
      # Rows are padded to a 16-byte multiple so the backward GEMMs can read dy through TMA;
      # the caller sees the (rows, n) view.
      n_pad = (n + 7) // 8 * 8
      out = torch.empty(x2.shape[0], n_pad, dtype=torch.bfloat16, device=x.device)[:, :n]
    y = gemm(x2, w16, bias=bias, act=act, residual=res2, out_pre=pre, out=out)
    ctx.save_for_backward(x2, weight, pre)
    ctx.has_bias = bias is not None
    ctx.bias = bias
    ctx.has_res = residual is not None
    ctx.x_shape = x.shape
    return y.reshape(*x.shape[:-1], n)

  @staticmethod
  def backward(ctx, dy):
    x2, weight, pre = ctx.saved_tensors
    w16 = bf16_shadow(weight)
    n, k = weight.shape
    k_pad = ctx.k_pad
    if k_pad:
      w16 = F.pad(w16, (0, k_pad))
    dy2 = dy.reshape(-1, n)
    if dy2.stride(1) != 1 or dy2.stride(0) % 8:
      n_pad = (n + 7) // 8 * 8
      padded = torch.zeros(dy2.shape[0], n_pad, dtype=dy2.dtype, device=dy2.device)
      padded[:, :n].copy_(dy2)
      dy2 = padded[:, :n]
    d_res = dy if ctx.has_res else None
    if pre is not None:
      # Stand-alone GELU linear layers are off the hot path (the MLP blocks use expert_mlp,
      # whose dgrad GEMM applies gelu' in its epilogue).
      from vmoe_b200.ops.gemm import gelu_tanh_grad
      dy2 = (dy2.float() * gelu_tanh_grad(pre.float())).to(torch.bfloat16)
    dbias = bias_grad(dy2, ctx.bias) if ctx.has_bias else None  # handles padded rows
    dx = None
    if ctx.needs_input_grad[0]:
      dx = gemm(dy2, w16, b_mn_major=True)
      if k_pad:
        dx = dx[:, :k]
      dx = dx.reshape(ctx.x_shape)
    dw = None
    if ctx.needs_input_grad[1]:
      if k_pad:
        full = torch.zeros(n, k + k_pad, dtype=torch.float32, device=dy2.device)
        gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=full, accumulate=True,
             split_k=_wgrad_split(n, k, dy2.shape[0]))
        dw = full[:, :k]
      else:
        dw = wgrad(dy2, x2, weight, split_k=_wgrad_split(n, k, dy2.shape[0]))
    return dx, dw, dbias, d_res, None


def _wgrad_split(n: int, k: int, m: int) -> int:
  """Split-K factor of a weight-gradient GEMM with an (n, k) output and contraction length m.

  The output has few 256 x 256 tiles (27 for the qkv weights of ViT-B) against 74 CTA pairs, so
  the contraction is cut into pieces that fill whole rounds of the machine. The cost of a
  factor is rounds / factor plus 1.5 % per piece (each piece adds its tile to the output with
  atomics); the cheapest factor wins."""
  tiles = ((n + 255) // 256) * ((k + 255) // 256)
  pairs = 74
  if tiles >= 2 * pairs or m < 4096:
    return 1
  best, best_cost = 1, -(-tiles // pairs) + 0.015
  for split in range(2, max(1, min(16, m // 2048)) + 1):
    cost = -(-tiles * split // pairs) / split + 0.015 * split
    if cost < best_cost:
      best, best_cost = split, cost
  return best


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
           act: Optional[str] = None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
  """``act(x @ weight^T + bias) + residual`` with ``weight: [out, in]``; ``act`` in {None, 'gelu'}."""
  if _fast(x):
    code = ACT_GELU if act == "gelu" else ACT_NONE
    return _LinearFn.apply(x, weight, bias, residual, code)
  y = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
  if act == "gelu":
    y = F.gelu(y, approximate="tanh")
  if residual is not None:
    y = y + residual
  return y


# ----------------------------------------------------------------------------------- expert MLP
class _ExpertMlpFn(torch.autograd.Function):
  """Batched (per local expert) GEMM1 + bias + GELU, GEMM2 + bias; rows fixed by capacity."""

  @staticmethod
  def forward(ctx, x, w1, b1, w2, b2, residual):
    # x: (E, R, H) bf16; w1: (E, M, H); w2: (E, H, M)
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    e, r, h = x.shape
    m = w1.shape[1]
    x = x.contiguous()
    need_grad = any(ctx.needs_input_grad)
    pre = torch.empty(e, r, m, dtype=torch.bfloat16, device=x.device) if need_grad else None
    hid = gemm(x, w1h, bias=b1, act=ACT_GELU, out_pre=pre, out_pre_is_grad=True)
    y = gemm(hid, w2h, bias=b2, residual=residual)
    ctx.save_for_backward(x, w1, w2, pre, hid)
    ctx.biases = (b1, b2)
    ctx.has_res = residual is not None
    return y

  @staticmethod
  def backward(ctx, dy):
    x, w1, w2, pre, hid = ctx.saved_tensors
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    e, r, h = x.shape
    m = w1.shape[1]
    dy = dy.contiguous()
    b1, b2 = ctx.biases
    db2 = bias_grad(dy, b2)
    dw2 = wgrad(dy, hid, w2, split_k=_wgrad_split(h, m, r) if e == 1 else 1)
    tgt = _grad_target(b1)
    db1 = tgt if tgt is not None else torch.zeros(e, m, dtype=torch.float32, device=dy.device)
    dpre = gemm(dy, w2h, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True, colsum=db1)
    if tgt is not None:
      db1 = None
    dw1 = wgrad(dpre, x, w1, split_k=_wgrad_split(m, h, r) if e == 1 else 1)
    dx = gemm(dpre, w1h, b_mn_major=True) if ctx.needs_input_grad[0] else None
    return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None)


def expert_mlp(x: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor, w2: torch.Tensor,
               b2: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
  """Per-expert MLP on ``x: (E_local, rows, H)`` with ``w1: (E, M, H)``, ``w2: (E, H, M)``.

  ``residual`` (same shape as the output) is added in the second GEMM's epilogue.
  """
  if _fast(x):
    return _ExpertMlpFn.apply(x, w1, b1, w2, b2, residual)
  dt = x.dtype
  hid = torch.baddbmm(b1.to(dt).unsqueeze(1), x, w1.to(dt).transpose(1, 2))
  hid = F.gelu(hid, approximate="tanh")
  y = torch.baddbmm(b2.to(dt).unsqueeze(1), hid, w2.to(dt).transpose(1, 2))
  return y if residual is None else y + residual


# ----------------------------------------------------------------------------------- layer norm
def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
               eps: float = 1e-6) -> torch.Tensor:
  if _fast(x) and x.shape[-1] % 8 == 0:
    from vmoe_b200.ops import norm
    return norm.layer_norm(x, weight, bias, eps)
  w = None if weight is None else weight.to(x.dtype)
  b = None if bias is None else bias.to(x.dtype)
  return F.layer_norm(x, (x.shape[-1],), w, b, eps)


def layer_norm_fork(x: torch.Tensor, weight: Optional[torch.Tensor],
                    bias: Optional[torch.Tensor], eps: float = 1e-6):
  """``(layer_norm(x), x)``. On the CUDA path the second value is routed through the same
  autograd node, so the gradient of the residual branch is added inside the LayerNorm
  backward kernel."""
  if _fast(x) and x.shape[-1] % 8 == 0 and x.requires_grad and torch.is_grad_enabled():
    from vmoe_b200.ops import norm
    return norm.layer_norm_fork(x, weight, bias, eps)
  return layer_norm(x, weight, bias, eps), x


# ----------------------------------------------------------------------------------- attention
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              dropout_p: float = 0.0, training: bool = False) -> torch.Tensor:
  """Non-causal softmax attention; ``q: (B, Tq, heads, d)``, ``k, v: (B, Tk, heads, d)``.

  bf16 CUDA tensors of a shape the fused kernels cover run on them (dropout of the attention
  weights included); everything else is evaluated with PyTorch ops."""
  p_drop = dropout_p if training else 0.0
  if _fast(q) and k.dtype == q.dtype and v.dtype == q.dtype:
    from vmoe_b200.ops import attention_ops
    if attention_ops.separate_supported(q, k, v):
      seed = attention_ops.new_seed() if p_drop > 0 else 0
      return attention_ops.attention(q, k, v, p_drop, seed)
  d = q.shape[-1]
  scale = 1.0 / math.sqrt(d)
  logits = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
  probs = torch.softmax(logits.float(), dim=-1).to(q.dtype)
  if p_drop > 0:
    probs = F.dropout(probs, p_drop, True)
  return torch.einsum("bhqk,bkhd->bqhd", probs, v)


def attention_packed(qkv: torch.Tensor, dropout_p: float = 0.0, training: bool = False):
  """Self-attention on the packed QKV projection ``(B, T, 3, H, D)`` -> ``(B, T, H, D)``."""
  if _fast(qkv):
    from vmoe_b200.ops import attention_ops
    if attention_ops.packed_supported(qkv):
      p_drop = dropout_p if training else 0.0
      seed = attention_ops.new_seed() if p_drop > 0 else 0
      return attention_ops.packed_attention(qkv, p_drop, seed)
  return attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], dropout_p, training)
