"""Expert-parallel token exchange (the all-to-all between the two sharding constraints of the
reference's ``_dispatch`` / ``_receive``, ``vmoe/moe.py:488-519``).

``to_experts`` takes ``(E, R, ...)`` — R rows for each of the E global experts produced by
this rank — and returns ``(E_local, ep*R, ...)``: for every expert held by this rank, the rows
from all ranks of the expert group, ordered by source rank. ``from_experts`` is the inverse.
Both are differentiable (the backward of one is the other). This NCCL/gloo implementation is
the portable baseline; the fused GPU path pushes rows straight into peer memory instead.
"""
from __future__ import annotations


import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    x = x.contiguous()
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out

  @staticmethod
  def backward(ctx, grad):
    grad = grad.contiguous()  # the incoming gradient is usually a transposed view
    out = torch.empty_like(grad)
    dist.all_to_all_single(out, grad, group=ctx.group)
    return out, None


class ExpertExchange:
  """All-to-all over one expert group (identity when the group has a single rank)."""

  def __init__(self, group=None, size: int = 1):
    self.group = group
    self.size = size

  def to_experts(self, x: torch.Tensor) -> torch.Tensor:
    if self.size == 1:
      return x
    e, r = x.shape[:2]
    if e % self.size:
      raise ValueError(f"{e} experts cannot be split over {self.size} ranks")
    el = e // self.size
    tail = x.shape[2:]
    # (ep_dst, E_local, R, ...) -> a2a -> (ep_src, E_local, R, ...) -> (E_local, ep_src*R, ...)
    y = _AllToAll.apply(x.reshape(self.size, el, r, *tail).contiguous(), self.group)
    return y.transpose(0, 1).reshape(el, self.size * r, *tail)

  def from_experts(self, y: torch.Tensor) -> torch.Tensor:
    if self.size == 1:
      return y
    el, rows = y.shape[:2]
    r = rows // self.size
    tail = y.shape[2:]
    x = y.reshape(el, self.size, r, *tail).transpose(0, 1).contiguous()
    x = _AllToAll.apply(x, self.group)  # (ep_dst==owner of expert block, E_local, R, ...)
    return x.reshape(self.size * el, r, *tail)

  @classmethod
  def from_mesh(cls, mesh) -> "ExpertExchange":
    if mesh is None or mesh.num_partitions == 1:
      return LOCAL_EXCHANGE
    return cls(group=mesh.expert_group, size=mesh.num_partitions)


LOCAL_EXCHANGE = ExpertExchange()
