"""GPU Top-K MoE layer in indices form: routing-plan kernel, row gather/combine kernels and the
expert GEMMs, tied together by one autograd Function.

Forward:  plan -> gather rows into the expert buffers (local memory, or pushed into the peer
GPUs' buffers when experts are sharded) -> batched GEMM1 + bias + GELU -> batched GEMM2 + bias
-> gate-weighted combine (+ residual). Backward mirrors it: the backward of combine is a
gather (fused with the gate-gradient dot products) and the backward of dispatch is a combine
with unit weights.

Semantics are those of the reference's dispatchers (``vmoe/moe.py:148-209``) with the Top-K
plan of ``vmoe/moe.py:547-652``; tests compare against ``vmoe_b200.moe`` on CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from vmoe_b200 import moe as moe_core
from vmoe_b200.ops import _lib, reduce
from vmoe_b200.ops.functional import _grad_target, bf16_shadow, bias_grad, wgrad
from vmoe_b200.ops.gemm import ACT_GELU, gemm
from vmoe_b200.parallel.exchange import ExpertExchange, LOCAL_EXCHANGE

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64


def routing_plan(gates: torch.Tensor, num_selected_experts: int, capacity: int,
                 batch_priority: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
  """Runs the routing-plan kernel on ``gates (G, S, E)`` fp32 (CUDA).

  Returns int32 tensors ``expert (G, S, K)``, ``slot (G, S, K)`` and ``slot_pair (G, E, C)``.
  """
  assert gates.is_cuda and gates.dtype == torch.float32 and gates.dim() == 3
  gates = gates.contiguous()
  g, s, e = gates.shape
  k = num_selected_experts
  expert = torch.empty(g, s, k, dtype=torch.int32, device=gates.device)
  slot = torch.empty(g, s, k, dtype=torch.int32, device=gates.device)
  slot_pair = torch.empty(g, e, capacity, dtype=torch.int32, device=gates.device)
  rc = _lib.lib().vmoe_routing_plan(
      _vp(gates.data_ptr()), _vp(expert.data_ptr()), _vp(slot.data_ptr()),
      _vp(slot_pair.data_ptr()), _i64(g), _i64(s), _i64(e), _i64(k), _i64(capacity),
      ctypes.c_int32(int(batch_priority)), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_routing_plan")
  _lib.count_launch()
  return expert, slot, slot_pair


def _base_table(buf: torch.Tensor) -> torch.Tensor:
  """Device table of per-expert base addresses for a local ``(E, rows, H)`` buffer."""
  e = buf.shape[0]
  addrs = [buf.data_ptr() + i * buf.stride(0) * buf.element_size() for i in range(e)]
  return torch.tensor(addrs, dtype=torch.int64, device=buf.device)


_TABLE_CACHE: dict = {}


def base_table(buf: torch.Tensor) -> torch.Tensor:
  key = (buf.data_ptr(), buf.shape[0], buf.stride(0), buf.device)
  t = _TABLE_CACHE.get(key)
  if t is None:
    if len(_TABLE_CACHE) > 4096:
      _TABLE_CACHE.clear()
    t = _base_table(buf)
    _TABLE_CACHE[key] = t
  return t


def gather_rows(x, slot_pair, weight, table, g, s, e, c, k, h):
  rc = _lib.lib().vmoe_moe_gather_rows(
      _vp(x.data_ptr()), _vp(slot_pair.data_ptr()), _vp(_lib.ptr(weight)), _vp(table.data_ptr()),
      _i64(g), _i64(s), _i64(e), _i64(c), _i64(k), _i64(h), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_gather_rows")
  _lib.count_launch()


def combine_rows(table, expert, slot, weight, residual, out, g, s, e, c, k, h, status=None):
  rc = _lib.lib().vmoe_moe_combine_rows(
      _vp(table.data_ptr()), _vp(expert.data_ptr()), _vp(slot.data_ptr()), _vp(_lib.ptr(weight)),
      _vp(_lib.ptr(residual)), _vp(out.data_ptr()), _i64(g), _i64(s), _i64(e), _i64(c), _i64(k),
      _i64(h), _vp(_lib.ptr(status)), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_combine_rows")
  _lib.count_launch()


def combine_bwd(dy, slot_pair, gate, ytable, dtable, dgate, g, s, e, c, k, h):
  rc = _lib.lib().vmoe_moe_combine_bwd(
      _vp(dy.data_ptr()), _vp(slot_pair.data_ptr()), _vp(gate.data_ptr()), _vp(ytable.data_ptr()),
      _vp(dtable.data_ptr()), _vp(dgate.data_ptr()), _i64(g), _i64(s), _i64(e), _i64(c), _i64(k),
      _i64(h), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_combine_bwd")
  _lib.count_launch()


def _a2a_to_experts(buf: torch.Tensor, ex: ExpertExchange) -> torch.Tensor:
  """NCCL baseline exchange ``(E, R, H) -> (E_local, ep*R, H)`` (no autograd)."""
  if ex.size == 1:
    return buf
  e, r, h = buf.shape
  el = e // ex.size
  recv = torch.empty_like(buf)
  dist.all_to_all_single(recv, buf, group=ex.group)
  if el == 1:
    return recv.reshape(1, ex.size * r, h)
  return recv.reshape(ex.size, el, r, h).transpose(0, 1).reshape(el, ex.size * r, h)


def _a2a_from_experts(buf: torch.Tensor, ex: ExpertExchange) -> torch.Tensor:
  """Inverse of ``_a2a_to_experts``: ``(E_local, ep*R, H) -> (E, R, H)``."""
  if ex.size == 1:
    return buf
  el, rows, h = buf.shape
  r = rows // ex.size
  send = buf if el == 1 else buf.reshape(el, ex.size, r, h).transpose(0, 1).contiguous()
  recv = torch.empty(ex.size * el, r, h, dtype=buf.dtype, device=buf.device)
  dist.all_to_all_single(recv, send.reshape(ex.size * el, r, h), group=ex.group)
  return recv


class _FusedMoeFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, gate, w1, b1, w2, b2, residual, expert, slot, slot_pair, capacity,
              exchange):
    g, s, h = x.shape
    k = expert.shape[-1]
    e = slot_pair.shape[1]
    c = capacity
    x = x.contiguous()
    gate = gate.contiguous().float()
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    m = w1.shape[1]
    # Dispatch: expert buffers (E, G*C, H), rows ordered (group, slot).
    xbuf = torch.empty(e, g * c, h, dtype=torch.bfloat16, device=x.device)
    gather_rows(x, slot_pair, None, base_table(xbuf), g, s, e, c, k, h)
    xe = _a2a_to_experts(xbuf, exchange)
    need = any(ctx.needs_input_grad)
    pre = torch.empty(xe.shape[0], xe.shape[1], m, dtype=torch.bfloat16,
                      device=x.device) if need else None
    hid = gemm(xe, w1h, bias=b1, act=ACT_GELU, out_pre=pre, out_pre_is_grad=True)
    ye = gemm(hid, w2h, bias=b2)
    ybuf = _a2a_from_experts(ye, exchange)
    out = torch.empty_like(x)
    combine_rows(base_table(ybuf), expert, slot, gate, residual, out, g, s, e, c, k, h)
    ctx.save_for_backward(gate, w1, w2, expert, slot, slot_pair, xe, pre, hid, ybuf)
    ctx.dims = (g, s, e, c, k, h, m)
    ctx.biases = (b1, b2)
    ctx.exchange = exchange
    ctx.has_res = residual is not None
    return out

  @staticmethod
  def backward(ctx, dy):
    gate, w1, w2, expert, slot, slot_pair, xe, pre, hid, ybuf = ctx.saved_tensors
    g, s, e, c, k, h, m = ctx.dims
    ex = ctx.exchange
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    dy = dy.contiguous()
    dev = dy.device
    # Backward of combine: d(ybuf) rows and gate gradients in one pass.
    dybuf = torch.empty(e, g * c, h, dtype=torch.bfloat16, device=dev)
    dgate = torch.zeros(g, s, k, dtype=torch.float32, device=dev)
    combine_bwd(dy, slot_pair, gate, base_table(ybuf), base_table(dybuf), dgate, g, s, e, c, k, h)
    dye = _a2a_to_experts(dybuf, ex)
    el = dye.shape[0]
    b1, b2 = ctx.biases
    db2 = bias_grad(dye, b2)
    dw2 = wgrad(dye, hid, w2)
    tgt = _grad_target(b1)
    db1 = tgt if tgt is not None else torch.zeros(el, m, dtype=torch.float32, device=dev)
    dpre = gemm(dye, w2h, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True, colsum=db1)
    if tgt is not None:
      db1 = None
    dw1 = wgrad(dpre, xe, w1)
    dxe = gemm(dpre, w1h, b_mn_major=True)
    dxbuf = _a2a_from_experts(dxe, ex)
    # Backward of dispatch: unit-weight combine.
    dx = torch.empty(g, s, h, dtype=torch.bfloat16, device=dev)
    combine_rows(base_table(dxbuf), expert, slot, None, None, dx, g, s, e, c, k, h)
    d_res = dy if ctx.has_res else None
    return dx, dgate, dw1, db1, dw2, db2, d_res, None, None, None, None, None


class FusedTopKDispatcher(moe_core.BaseDispatcher):
  """Top-K dispatcher for CUDA bf16 activations backed by the kernels of this module.

  It also implements the generic ``dispatch`` / ``combine`` protocol (through the PyTorch
  indices dispatcher) so code written against ``BaseDispatcher`` keeps working, but the MoE
  block calls ``apply_experts`` which runs the whole layer in one autograd node.
  """

  def __init__(self, gates: torch.Tensor, num_selected_experts: int, capacity: int,
               batch_priority: bool, exchange: ExpertExchange = LOCAL_EXCHANGE):
    self.gates = gates
    self.capacity = capacity
    self.num_experts = gates.shape[-1]
    self.exchange = exchange
    self.expert, self.slot, self.slot_pair = routing_plan(
        gates.detach().float(), num_selected_experts, capacity, batch_priority)
    # Differentiable gate values of the selected experts (raw softmax, not renormalised).
    self.combine_weights = torch.gather(gates, -1, self.expert.long())

  @property
  def indices(self) -> torch.Tensor:
    return torch.stack([self.expert, self.slot], dim=-1)

  def _generic(self) -> moe_core.ExpertIndicesDispatcher:
    return moe_core.ExpertIndicesDispatcher(
        indices=self.indices, combine_weights=self.combine_weights,
        num_experts=self.num_experts, capacity=self.capacity, exchange=self.exchange)

  def dispatch(self, data):
    return self._generic().dispatch(data)

  def combine(self, data):
    return self._generic().combine(data)

  def apply_experts(self, mlp, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
    if mlp.training and getattr(mlp, "dropout_rate", 0.0) > 0:
      out = moe_core.sparse_moe_apply(mlp, self._generic(), x)
      return out if residual is None else out + residual
    return _FusedMoeFn.apply(x, self.combine_weights, mlp.w1, mlp.b1, mlp.w2, mlp.b2, residual,
                             self.expert, self.slot, self.slot_pair, self.capacity,
                             self.exchange)
