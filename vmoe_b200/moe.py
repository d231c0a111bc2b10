"""Sparse-MoE core: capacity, routing algorithms, dispatchers and the expert-parallel lift.

Everything here is plain PyTorch and runs on any device; it is both the CPU path and the
oracle the CUDA kernels in ``vmoe_b200.ops`` are tested against. The fused GPU path builds
the same ``RoutingPlan`` with one kernel and never materialises ``(S, E, C)`` tensors.

Conventions (as in the reference, ``vmoe/moe.py:58-67``): data enters a dispatcher as
``(G, S, ...)`` (G groups of S items), experts see ``(E, G*C, ...)`` (capacity C per group and
expert) and ``combine`` returns ``(G, S, ...)``. With expert parallelism over ``ep`` ranks each
rank holds ``E/ep`` experts and sees ``(E/ep, ep*G*C, ...)``; rows of an expert buffer are
ordered ``(source rank, group, slot)``.

Reference: ``vmoe/moe.py`` — ``compute_capacity`` :230-257, Top-K/BPR :547-652, experts-choose
:655-694, dispatchers :94-227, ``sparse_moe_spmd`` :388-448.
"""
from __future__ import annotations

import dataclasses
import logging
import math
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from vmoe_b200.parallel.exchange import ExpertExchange, LOCAL_EXCHANGE

Tensor = torch.Tensor


# --------------------------------------------------------------------------------- capacity
_CAPACITY_WARNED: set = set()


def compute_capacity(num_tokens: int, num_experts: int, capacity_factor: float,
                     ceil_or_round: str = "ceil", multiple_of: Optional[int] = 4) -> int:
  """Slots per expert needed to spread ``num_tokens`` over ``num_experts``."""
  if ceil_or_round == "ceil":
    capacity = int(math.ceil(num_tokens * capacity_factor / num_experts))
  elif ceil_or_round == "round":
    capacity = int(round(num_tokens * capacity_factor / num_experts))
  else:
    raise ValueError(f"Unsupported ceil_or_round={ceil_or_round!r}")
  if capacity < 1:
    raise ValueError(
        f"The values num_tokens = {num_tokens}, num_experts = {num_experts} and "
        f"capacity_factor = {capacity_factor} lead to capacity = {capacity}, but it must be "
        "greater than or equal to 1.")
  if multiple_of and multiple_of > 0:
    capacity += (-capacity) % multiple_of
  actual = capacity * num_experts / num_tokens
  key = (capacity_factor, num_tokens, num_experts, multiple_of)
  if abs(actual - capacity_factor) > 1e-6 and key not in _CAPACITY_WARNED:
    # Once per geometry: the reference logs this while tracing, i.e. once per compiled step.
    _CAPACITY_WARNED.add(key)
    logging.warning(
        "The target capacity_factor is %f, but with num_tokens=%d and num_experts=%d the "
        "actual capacity_factor is %f.", capacity_factor, num_tokens, num_experts, actual)
  return capacity


def _resolve_capacity(capacity, capacity_factor, num_tokens, num_experts, ceil_or_round,
                      multiple_of) -> int:
  if (capacity is None) == (capacity_factor is None):
    raise ValueError(
        "You must specify either 'capacity' or 'capacity_factor', and not both. Current "
        f"values are capacity = {capacity!r}, capacity_factor = {capacity_factor!r}")
  if not capacity:
    capacity = compute_capacity(num_tokens, num_experts, capacity_factor, ceil_or_round,
                                multiple_of)
  return capacity


def _grouped(gates: Tensor) -> Tuple[Tensor, bool]:
  """Views ``(S, E)`` gates as one group."""
  if gates.dim() == 2:
    return gates.unsqueeze(0), True
  if gates.dim() != 3:
    raise ValueError(f"gates must be (S, E) or (G, S, E), got {tuple(gates.shape)}")
  return gates, False


def _einsum_ops():
  from vmoe_b200.ops import einsum_ops
  return einsum_ops


# --------------------------------------------------------------------------------- dispatchers
class BaseDispatcher:
  """Moves items to experts (``dispatch``) and expert outputs back (``combine``)."""

  exchange: ExpertExchange = LOCAL_EXCHANGE

  def dispatch(self, data: Tensor) -> Tensor:
    raise NotImplementedError

  def combine(self, data: Tensor) -> Tensor:
    raise NotImplementedError


def _to_experts(data_gec: Tensor, exchange: ExpertExchange) -> Tensor:
  """``(G, E, C, ...) -> (E_local, ep*G*C, ...)`` (the all-to-all of ``vmoe/moe.py:488-500``)."""
  g, e, c = data_gec.shape[:3]
  x = data_gec.transpose(0, 1).reshape(e, g * c, *data_gec.shape[3:])
  return exchange.to_experts(x)


def _from_experts(data: Tensor, num_groups: int, exchange: ExpertExchange) -> Tensor:
  """Inverse of ``_to_experts``: ``(E_local, ep*G*C, ...) -> (G, E, C, ...)``."""
  x = exchange.from_experts(data)  # (E, G*C, ...)
  e = x.shape[0]
  c = x.shape[1] // num_groups
  return x.reshape(e, num_groups, c, *x.shape[2:]).transpose(0, 1)


@dataclasses.dataclass
class DenseEinsumDispatcher(BaseDispatcher):
  """Every item goes to every expert (C = S); ``combine_weights`` is ``(G, S, E)``."""
  combine_weights: Tensor
  exchange: ExpertExchange = LOCAL_EXCHANGE
  partition_spec: Any = None      # accepted for config compatibility; placement is explicit
  einsum_precision: Any = None

  def dispatch(self, data: Tensor) -> Tensor:
    g, s, e = self.combine_weights.shape
    x = data.unsqueeze(1).expand(g, e, *data.shape[1:])  # (G, E, S, ...)
    return _to_experts(x, self.exchange)

  def combine(self, data: Tensor) -> Tensor:
    g = self.combine_weights.shape[0]
    x = _from_experts(data, g, self.exchange)  # (G, E, S, ...)
    w = self.combine_weights.to(x.dtype).transpose(1, 2)  # (G, E, S)
    w = w.reshape(*w.shape, *([1] * (x.dim() - 3)))
    return (x * w).sum(dim=1)


@dataclasses.dataclass
class EinsumDispatcher(BaseDispatcher):
  """Dense ``(G, S, E, C)`` weights; dispatch weights default to ``combine_weights > 0``.

  With boolean dispatch weights this is a gather written as a matmul; with real-valued ones
  (Soft MoE) it is a true weighted sum.
  """
  combine_weights: Tensor
  dispatch_weights: Optional[Tensor] = None
  exchange: ExpertExchange = LOCAL_EXCHANGE
  partition_spec: Any = None
  einsum_precision: Any = None

  def _dispatch_w(self) -> Tensor:
    return self.combine_weights > 0 if self.dispatch_weights is None else self.dispatch_weights

  def dispatch(self, data: Tensor) -> Tensor:
    w = self._dispatch_w()
    g, s, e, c = w.shape
    flat = data.reshape(g, s, -1)
    w2 = w.reshape(g, s, e * c)
    if _einsum_ops().supported(w2, flat):
      out = _einsum_ops().dispatch(w2 if w2.is_floating_point() else w2.to(flat.dtype), flat,
                                   slots_per_expert=c)
    else:
      out = torch.einsum("gsn,gsh->gnh", w2.to(flat.dtype), flat)
    return _to_experts(out.reshape(g, e, c, *data.shape[2:]), self.exchange)

  def combine(self, data: Tensor) -> Tensor:
    g, s, e, c = self.combine_weights.shape
    x = _from_experts(data, g, self.exchange)  # (G, E, C, ...)
    flat = x.reshape(g, e * c, -1)
    w2 = self.combine_weights.reshape(g, s, e * c)
    if _einsum_ops().supported(w2, flat):
      out = _einsum_ops().combine(w2, flat, slots_per_expert=c)
    else:
      out = torch.einsum("gsn,gnh->gsh", w2.to(flat.dtype), flat)
    return out.reshape(g, s, *x.shape[3:])

  def apply_experts(self, mlp, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
    """Dispatch, experts, combine in one call. When the experts are spread over several GPUs
    with peer memory, the slot rows travel inside the expert GEMMs (``ops/moe_dense_p2p.py``)
    instead of through two all-to-alls; otherwise this is ``sparse_moe_apply``."""
    g, s, e, c = self.combine_weights.shape
    out = None
    if x.is_cuda and x.dim() == 3:
      from vmoe_b200.ops import moe_dense_p2p
      w_d = self._dispatch_w().reshape(g, s, e * c)
      w_c = self.combine_weights.reshape(g, s, e * c)
      if (moe_dense_p2p.applicable(self.exchange, mlp, g, e, c, x) and
          _einsum_ops().supported(w_c, x)):
        ops_ = _einsum_ops()
        xs = ops_.dispatch(w_d if w_d.is_floating_point() else w_d.to(x.dtype), x)
        ys = moe_dense_p2p.expert_exchange_and_mlp(mlp, self.exchange, xs, e, c)
        out = ops_.combine(w_c, ys)
    if out is None:
      out = sparse_moe_apply(mlp, self, x)
    return out if residual is None else out + residual


@dataclasses.dataclass
class ExpertIndicesDispatcher(BaseDispatcher):
  """Indices form: ``indices (G, S, K, 2)`` = (expert, slot), ``combine_weights (G, S, K)``.

  Pairs whose expert or slot is out of range are dropped: they write nothing on dispatch and
  read zero on combine.
  """
  indices: Tensor
  combine_weights: Tensor
  num_experts: int
  capacity: int
  exchange: ExpertExchange = LOCAL_EXCHANGE
  partition_spec: Any = None
  einsum_precision: Any = None

  def _flat_index(self) -> Tuple[Tensor, Tensor]:
    e, p = self.indices[..., 0].long(), self.indices[..., 1].long()
    valid = (e >= 0) & (e < self.num_experts) & (p >= 0) & (p < self.capacity)
    flat = torch.where(valid, e * self.capacity + p, torch.zeros_like(e))
    return flat, valid  # (G, S, K)

  def dispatch(self, data: Tensor) -> Tensor:
    g, s, k = self.combine_weights.shape
    flat, valid = self._flat_index()
    x = data.reshape(g, s, 1, -1).expand(g, s, k, -1)
    x = torch.where(valid.unsqueeze(-1), x, torch.zeros_like(x)).reshape(g, s * k, -1)
    out = torch.zeros(g, self.num_experts * self.capacity, x.shape[-1], dtype=data.dtype,
                      device=data.device)
    out = out.scatter_add(1, flat.reshape(g, s * k, 1).expand_as(x), x)
    out = out.reshape(g, self.num_experts, self.capacity, *data.shape[2:])
    return _to_experts(out, self.exchange)

  def combine(self, data: Tensor) -> Tensor:
    g, s, k = self.combine_weights.shape
    x = _from_experts(data, g, self.exchange)  # (G, E, C, ...)
    tail = x.shape[3:]
    x = x.reshape(g, self.num_experts * self.capacity, -1)
    flat, valid = self._flat_index()
    got = torch.gather(x, 1, flat.reshape(g, s * k, 1).expand(g, s * k, x.shape[-1]))
    got = got.reshape(g, s, k, -1)
    w = (self.combine_weights * valid).to(got.dtype).unsqueeze(-1)
    return (got * w).sum(dim=2).reshape(g, s, *tail)


@dataclasses.dataclass
class Bfloat16Dispatcher(BaseDispatcher):
  """Casts floating payloads to bf16 for dispatch and combine, returning the caller's dtype."""
  dispatcher: BaseDispatcher

  @property
  def exchange(self):  # type: ignore[override]
    return self.dispatcher.exchange

  def dispatch(self, data: Tensor) -> Tensor:
    dtype = data.dtype
    if data.is_floating_point():
      data = data.to(torch.bfloat16)
    return self.dispatcher.dispatch(data).to(dtype)

  def combine(self, data: Tensor) -> Tensor:
    dtype = data.dtype
    if data.is_floating_point():
      data = data.to(torch.bfloat16)
    return self.dispatcher.combine(data).to(dtype)

  def apply_experts(self, mlp, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
    inner = getattr(self.dispatcher, "apply_experts", None)
    if inner is not None and x.dtype == torch.bfloat16:
      return inner(mlp, x, residual=residual)  # the payload already is bf16
    out = sparse_moe_apply(mlp, self, x)
    return out if residual is None else out + residual


# --------------------------------------------------------------------------------- routing
@dataclasses.dataclass
class RoutingPlan:
  """Top-K routing in indices form, for all groups at once.

  ``expert (G, S, K)`` int32, ``slot (G, S, K)`` int32 (position inside the expert's buffer of
  this group; ``>= capacity`` means dropped) and ``gate (G, S, K)`` (the raw softmax value of
  the chosen expert — not renormalised over the K choices).
  """
  expert: Tensor
  slot: Tensor
  gate: Tensor
  num_experts: int
  capacity: int

  def kept(self) -> Tensor:
    return self.slot < self.capacity


def top_experts_per_item_plan(gates: Tensor, num_selected_experts: int, capacity: int,
                              batch_priority: bool) -> RoutingPlan:
  """Top-K "tokens choose" routing with buffer positions (vanilla or Batch Priority Routing).

  Per group: take the K best experts of every item; all first choices precede all second
  choices (K-major order); inside one choice level items are served in index order (vanilla)
  or by decreasing top-1 gate, ties by index (BPR); the position of an (item, choice) pair in
  its expert's buffer is the number of pairs for the same expert served before it.
  """
  gates, _ = _grouped(gates)
  g, s, e = gates.shape
  k = num_selected_experts
  top_w, top_i = torch.topk(gates, k, dim=-1)  # (G, S, K); ties -> lowest index first
  if batch_priority:
    order = torch.sort(-top_w[..., 0], dim=-1, stable=True).indices  # (G, S)
    top_i_sorted = torch.gather(top_i, 1, order.unsqueeze(-1).expand(g, s, k))
  else:
    order = None
    top_i_sorted = top_i
  kmajor = top_i_sorted.transpose(1, 2).reshape(g, k * s)  # (G, K*S)
  onehot = torch.nn.functional.one_hot(kmajor, e).to(torch.int32)  # (G, K*S, E)
  pos = (torch.cumsum(onehot, dim=1) * onehot).sum(dim=-1) - 1  # (G, K*S)
  pos = pos.reshape(g, k, s).transpose(1, 2)  # (G, S, K) in served order
  if order is not None:
    inv = torch.empty_like(order)
    inv.scatter_(1, order, torch.arange(s, device=gates.device).expand(g, s))
    pos = torch.gather(pos, 1, inv.unsqueeze(-1).expand(g, s, k))
  return RoutingPlan(expert=top_i.to(torch.int32), slot=pos.to(torch.int32), gate=top_w,
                     num_experts=e, capacity=capacity)


def _plan_to_einsum(plan: RoutingPlan, gates: Tensor, **kw) -> EinsumDispatcher:
  g, s, e = gates.shape
  c = plan.capacity
  kept = plan.kept()
  # (G, S, E) buffer index of each (item, expert) pair, -1 if not selected or dropped.
  buf = torch.full((g, s, e), -1, dtype=torch.long, device=gates.device)
  buf.scatter_(2, plan.expert.long(), torch.where(kept, plan.slot.long(), -1))
  dispatch = torch.zeros(g, s, e, c + 1, dtype=torch.bool, device=gates.device)
  dispatch.scatter_(3, torch.where(buf >= 0, buf, c).unsqueeze(-1), True)
  dispatch = dispatch[..., :c]
  combine = gates.unsqueeze(-1) * dispatch
  return EinsumDispatcher(combine_weights=combine, dispatch_weights=dispatch, **kw)


def get_top_experts_per_item_dispatcher(
    gates: Tensor, name: str, num_selected_experts: int, batch_priority: bool,
    capacity: Optional[int] = None, capacity_factor: Optional[float] = None,
    capacity_ceil_or_round: str = "ceil", capacity_multiple_of: Optional[int] = 4,
    **dispatcher_kwargs) -> BaseDispatcher:
  """Dispatcher for Top-K routing; ``name`` is ``"einsum"`` or ``"indices"``.

  ``gates`` is ``(S, E)`` or ``(G, S, E)``; the capacity defaults to
  ``compute_capacity(S*K, E, capacity_factor)``.
  """
  gates3, single = _grouped(gates)
  _, s, e = gates3.shape
  capacity = _resolve_capacity(capacity, capacity_factor, s * num_selected_experts, e,
                               capacity_ceil_or_round, capacity_multiple_of)
  if name not in ("einsum", "indices"):
    raise ValueError(f"Unknown dispatcher type: {name!r}")
  plan = top_experts_per_item_plan(gates3, num_selected_experts, capacity, batch_priority)
  if name == "einsum":
    d = _plan_to_einsum(plan, gates3, **dispatcher_kwargs)
    if single:
      d.single_group = True  # type: ignore[attr-defined]
    return d
  indices = torch.stack([plan.expert, plan.slot], dim=-1)
  return ExpertIndicesDispatcher(indices=indices, combine_weights=plan.gate, num_experts=e,
                                 capacity=capacity, **dispatcher_kwargs)


def get_top_items_per_expert_dispatcher(
    gates: Tensor, name: str, capacity: Optional[int] = None,
    capacity_factor: Optional[float] = None, capacity_ceil_or_round: str = "ceil",
    capacity_multiple_of: Optional[int] = 4,
    **dispatcher_kwargs) -> Tuple[BaseDispatcher, Dict[str, Tensor]]:
  """"Experts choose" routing: every expert takes its ``capacity`` best items of the group.

  Returns the dispatcher and per-group monitoring metrics.
  """
  gates3, _ = _grouped(gates)
  g, s, e = gates3.shape
  capacity = _resolve_capacity(capacity, capacity_factor, s, e, capacity_ceil_or_round,
                               capacity_multiple_of)
  if name != "einsum":
    raise ValueError(f"Unknown dispatcher type: {name!r}")
  top_g, top_idx = torch.topk(gates3.transpose(1, 2), capacity, dim=-1)  # (G, E, C)
  dispatch = torch.zeros(g, s, e, capacity, dtype=torch.bool, device=gates3.device)
  dispatch.scatter_(1, top_idx.unsqueeze(1), True)
  combine = gates3.unsqueeze(-1) * dispatch
  dispatcher = EinsumDispatcher(combine_weights=combine, dispatch_weights=dispatch,
                                **dispatcher_kwargs)
  per_item = dispatch.sum(dim=(2, 3)).to(torch.int32)  # (G, S)
  metrics = {
      "num_experts_per_item_min": per_item.min(dim=1).values,
      "num_experts_per_item_max": per_item.max(dim=1).values,
      "min_selected_gate": top_g.amin(dim=(1, 2)),
      "max_selected_gate": top_g.amax(dim=(1, 2)),
  }
  log2e = int(math.log2(e))
  for t in [2 ** i for i in range(log2e + 1)] + [e]:
    metrics[f"ratio_processed_items_by_at_least_{t}_experts"] = (
        (per_item >= t).sum(dim=1).to(gates3.dtype) / s)
  return dispatcher, metrics


def get_dense_einsum_dispatcher(gates: Tensor, **dispatcher_kwargs) -> DenseEinsumDispatcher:
  gates3, _ = _grouped(gates)
  return DenseEinsumDispatcher(combine_weights=gates3, **dispatcher_kwargs)


# --------------------------------------------------------------------------------- expert lift
def sparse_moe_apply(expert_fn: Callable[..., Any], dispatcher: BaseDispatcher, *inputs: Tensor,
                     has_aux: bool = False):
  """Dispatch every input, run ``expert_fn`` on ``(E_local, rows, ...)`` buffers, combine.

  ``expert_fn`` must map leading axis ``E_local`` to the experts held by this rank (a batched
  module, e.g. ``ExpertMlp``). With ``has_aux`` it returns ``(outputs, aux)`` and ``aux`` is
  passed through un-combined. Counterpart of ``sparse_moe_spmd`` (``vmoe/moe.py:388-448``):
  the lift over the expert axis is an explicit batch dimension instead of a vmap.
  """
  dispatched = [dispatcher.dispatch(x) for x in inputs]
  out = expert_fn(*dispatched)
  aux = None
  if has_aux:
    out, aux = out
  if isinstance(out, (tuple, list)):
    combined = type(out)(dispatcher.combine(o) for o in out)
  elif isinstance(out, dict):
    combined = {k: dispatcher.combine(v) for k, v in out.items()}
  else:
    combined = dispatcher.combine(out)
  return (combined, aux) if has_aux else combined


def sparse_moe_spmd(target: Callable[..., Any], variable_axes=None, split_rngs=None,
                    has_aux: bool = False, methods=None):
  """Reference-named lift (``vmoe/moe.py:388-448``): wraps a batched expert module / function
  so that calling the result with ``(dispatcher, *inputs)`` dispatches every input, applies the
  experts and combines the outputs.

  ``variable_axes`` / ``split_rngs`` / ``methods`` configure Flax's vmap in the reference; here
  the expert axis is the leading dimension of the module's parameters (each rank holds the
  experts of its 'expert' mesh coordinate), so they are accepted and ignored.
  """
  del variable_axes, split_rngs, methods

  def apply(dispatcher: BaseDispatcher, *inputs: Tensor):
    return sparse_moe_apply(target, dispatcher, *inputs, has_aux=has_aux)

  return apply


def sparse_moe_spmd_with_axes(target: Callable[..., Any], variable_axes=None, partitioning_axis_names=None,
                              split_rngs=None, has_aux: bool = False, methods=None):
  """As ``sparse_moe_spmd``; the axis-name annotations of the reference
  (``vmoe/moe.py:451-474``) have no counterpart because placement is explicit."""
  del partitioning_axis_names
  return sparse_moe_spmd(target, variable_axes, split_rngs, has_aux, methods)
