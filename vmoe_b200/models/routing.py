"""Routers: noisy Top-K "tokens choose" (with Batch Priority Routing) and "experts choose".

Each router owns the gating layer (``dense``: hidden -> experts, no bias), turns gating logits
into softmax gates (with Gaussian noise of std ``noise_std / E`` on the logits when stochastic),
computes the auxiliary losses per group and returns ``(dispatcher, metrics)``.

Reference: ``vmoe/nn/routing.py`` — Top-K router :31-183 (importance loss :151-157, load loss
:159-183, GShard loss :133-148), experts-choose router :186-244, weighted sum :247-252.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Mapping, Optional, Tuple

import torch
from torch import nn

from vmoe_b200 import moe
from vmoe_b200 import ops
from vmoe_b200.parallel.exchange import ExpertExchange, LOCAL_EXCHANGE

Tensor = torch.Tensor


def _weighted_sum(*pairs):
  """Sum of ``w * x`` over pairs with ``w > 0`` (ill-defined losses are switched off by w=0)."""
  total = 0.0
  for w, x in pairs:
    if w > 0:
      total = total + x * w
  return total


def lecun_normal_(w: Tensor, fan_in: int, generator=None) -> Tensor:
  """Truncated-normal (±2 sigma) init with variance 1/fan_in, as Flax's default kernel init."""
  std = math.sqrt(1.0 / fan_in) / 0.87962566103423978
  with torch.no_grad():
    nn.init.trunc_normal_(w, mean=0.0, std=std, a=-2 * std, b=2 * std, generator=generator)
  return w


def _std_pop(x: Tensor, dim=None) -> Tensor:
  return x.std(dim=dim, unbiased=False) if dim is not None else x.std(unbiased=False)


class _RouterBase(nn.Module):

  def __init__(self, num_experts: int, hidden_size: int, noise_std: float = 1.0,
               dispatcher: Optional[Mapping[str, Any]] = None,
               deterministic: Optional[bool] = None, dtype: Optional[torch.dtype] = None,
               exchange: ExpertExchange = LOCAL_EXCHANGE):
    super().__init__()
    self.num_experts = num_experts
    self.noise_std = noise_std
    self.dispatcher_kwargs = dict(dispatcher or {})
    self.deterministic = deterministic
    self.dtype = dtype
    self.exchange = exchange
    self.dense = nn.Linear(hidden_size, num_experts, bias=False)
    lecun_normal_(self.dense.weight, hidden_size)
    # Test hook: noise to add to the logits instead of sampling (same shape as the logits).
    self.injected_noise: Optional[Tensor] = None

  def is_deterministic(self) -> bool:
    return (not self.training) if self.deterministic is None else self.deterministic

  def gating_logits(self, inputs: Tensor) -> Tensor:
    if inputs.dim() != 3:
      raise ValueError(f"inputs.ndim must be 3, but it is {inputs.dim()}")
    dtype = self.dtype or inputs.dtype
    # Gating runs in fp32 on bf16 activations too: logits feed a softmax and a top-k whose
    # ties/ordering should not depend on bf16 rounding.
    if dtype == torch.bfloat16:
      from vmoe_b200.ops import router_ops
      if router_ops.gating_logits_supported(inputs, self.dense.weight):
        return router_ops.gating_logits(inputs, self.dense.weight)
      dtype = torch.float32
    return torch.matmul(inputs.to(dtype), self.dense.weight.to(dtype).t())

  def sample_noise(self, logits: Tensor) -> Tensor:
    std = self.noise_std / self.num_experts
    if self.injected_noise is not None:
      return self.injected_noise.to(logits) * std
    return torch.randn_like(logits) * std


class NoisyTopExpertsPerItemRouter(_RouterBase):
  """Noisy Top-K router of V-MoE (https://arxiv.org/abs/2106.05974)."""

  def __init__(self, num_experts: int, hidden_size: int, num_selected_experts: int = 1,
               noise_std: float = 1.0, gshard_loss_weight: float = 0.0,
               importance_loss_weight: float = 1.0, load_loss_weight: float = 1.0,
               dispatcher: Optional[Mapping[str, Any]] = None,
               deterministic: Optional[bool] = None, dtype: Optional[torch.dtype] = None,
               exchange: ExpertExchange = LOCAL_EXCHANGE):
    super().__init__(num_experts, hidden_size, noise_std, dispatcher, deterministic, dtype,
                     exchange)
    self.num_selected_experts = num_selected_experts
    self.gshard_loss_weight = gshard_loss_weight
    self.importance_loss_weight = importance_loss_weight
    self.load_loss_weight = load_loss_weight

  def forward(self, inputs: Tensor) -> Tuple[moe.BaseDispatcher, Dict[str, Tensor]]:
    gates, metrics = self._compute_gates_softmax_and_metrics(inputs, self.num_experts)
    return self._create_dispatcher(gates, inputs), metrics

  def _compute_gates_softmax_and_metrics(self, inputs: Tensor, num_experts: int):
    if not num_experts >= self.num_selected_experts >= 1:
      raise ValueError(
          "num_experts >= num_selected_experts >= 1, but got "
          f"num_experts = {num_experts} and num_selected_experts = {self.num_selected_experts}.")
    return self._gates_and_metrics_from_logits(self.gating_logits(inputs), num_experts)

  def _gates_and_metrics_from_logits(self, logits: Tensor, num_experts: int, noise=None):
    """``logits (G, S, E)`` -> (softmax gates used for dispatch, per-group metrics)."""
    from vmoe_b200.ops import router_ops
    if router_ops.router_stats_supported(logits):
      return self._fused_gates_and_metrics(logits, num_experts, noise)
    gates = torch.softmax(logits, dim=-1)
    importance_loss = self._importance_auxiliary_loss(gates)
    if self.is_deterministic() or self.noise_std == 0.0:
      gshard_loss = self._gshard_auxiliary_loss(gates)
      metrics = {
          "auxiliary_loss": _weighted_sum((self.gshard_loss_weight, gshard_loss),
                                          (self.importance_loss_weight, importance_loss)),
          "gshard_loss": gshard_loss,
          "importance_loss": importance_loss,
      }
      return gates, metrics
    noise_std = self.noise_std / num_experts
    if noise is None:
      noise = (self.injected_noise.to(logits) if self.injected_noise is not None
               else torch.randn_like(logits))
    logits_noisy = logits + noise * noise_std
    gates_noisy = torch.softmax(logits_noisy, dim=-1)
    load_loss = self._load_auxiliary_loss(logits, logits_noisy, noise_std,
                                          self.num_selected_experts)
    gshard_loss = self._gshard_auxiliary_loss(gates_noisy)
    metrics = {
        "auxiliary_loss": _weighted_sum((self.gshard_loss_weight, gshard_loss),
                                        (self.importance_loss_weight, importance_loss),
                                        (self.load_loss_weight, load_loss)),
        "gshard_loss": gshard_loss,
        "importance_loss": importance_loss,
        "load_loss": load_loss,
    }
    return gates_noisy, metrics

  def _fused_gates_and_metrics(self, logits: Tensor, num_experts: int, noise=None):
    """Same contract as the PyTorch branch of ``_gates_and_metrics_from_logits``, evaluated by
    the router-statistics kernels."""
    from vmoe_b200.ops import router_ops
    noisy = not (self.is_deterministic() or self.noise_std == 0.0)
    noise_std = self.noise_std / num_experts
    if noisy and noise is None:
      noise = (self.injected_noise.to(logits) if self.injected_noise is not None
               else torch.randn_like(logits))
    gates, importance_loss, load_loss, gshard_loss = router_ops.router_stats(
        logits, noise if noisy else None, noise_std if noisy else 1.0,
        self.num_selected_experts)
    pairs = [(self.gshard_loss_weight, gshard_loss),
             (self.importance_loss_weight, importance_loss)]
    metrics = {"gshard_loss": gshard_loss, "importance_loss": importance_loss}
    if noisy:
      pairs.append((self.load_loss_weight, load_loss))
      metrics["load_loss"] = load_loss
    metrics["auxiliary_loss"] = _weighted_sum(*pairs)
    return gates, metrics

  def _create_dispatcher(self, gates: Tensor, inputs: Optional[Tensor] = None):
    kwargs = dict(self.dispatcher_kwargs)
    use_bf16 = kwargs.pop("bfloat16", False)
    if (inputs is not None and inputs.is_cuda and inputs.dtype == torch.bfloat16 and
        ops.cuda_kernels_enabled() and kwargs.get("name") in ("einsum", "indices")):
      # GPU path: one routing-plan kernel, indices form (identical semantics for both names).
      from vmoe_b200.ops import moe_ops
      g, s, e = gates.shape
      capacity = moe._resolve_capacity(
          kwargs.get("capacity"), kwargs.get("capacity_factor"),
          s * self.num_selected_experts, e, kwargs.get("capacity_ceil_or_round", "ceil"),
          kwargs.get("capacity_multiple_of", 4))
      return moe_ops.FusedTopKDispatcher(gates, self.num_selected_experts, capacity,
                                         bool(kwargs.get("batch_priority", False)),
                                         exchange=self.exchange)
    d = moe.get_top_experts_per_item_dispatcher(
        gates, num_selected_experts=self.num_selected_experts, exchange=self.exchange, **kwargs)
    return moe.Bfloat16Dispatcher(d) if use_bf16 else d

  # Losses below take (G, S, E) and return one value per group, (G,).
  @classmethod
  def _gshard_auxiliary_loss(cls, gates: Tensor) -> Tensor:
    e = gates.shape[-1]
    mean_gates = gates.mean(dim=-2)
    top1 = torch.nn.functional.one_hot(gates.argmax(dim=-1), e).to(gates.dtype).mean(dim=-2)
    return (top1 * mean_gates).mean(dim=-1) * (e ** 2)

  @classmethod
  def _importance_auxiliary_loss(cls, gates: Tensor) -> Tensor:
    importance = gates.sum(dim=-2)  # (G, E)
    return (_std_pop(importance, -1) / importance.mean(dim=-1)) ** 2

  @classmethod
  def _load_auxiliary_loss(cls, logits: Tensor, logits_noisy: Tensor, noise_std: float,
                           num_selected_experts: int) -> Tensor:
    # Threshold = K-th largest noisy logit of each item (differentiable through the gather).
    idx = torch.topk(logits_noisy, num_selected_experts, dim=-1).indices[..., -1:]
    threshold = torch.gather(logits_noisy, -1, idx)
    noise_required_to_win = (threshold - logits) / noise_std
    p = 1.0 - 0.5 * (1.0 + torch.erf(noise_required_to_win / math.sqrt(2.0)))
    p_mean = p.mean(dim=-2)  # (G, E)
    return (_std_pop(p_mean, -1) / p_mean.mean(dim=-1)) ** 2


class NoisyTopItemsPerExpertRouter(_RouterBase):
  """"Experts choose" router (https://arxiv.org/abs/2202.09368): no auxiliary loss needed."""

  def forward(self, inputs: Tensor) -> Tuple[moe.BaseDispatcher, Dict[str, Tensor]]:
    logits = self.gating_logits(inputs)
    if not (self.is_deterministic() or self.noise_std == 0.0):
      logits = logits + self.sample_noise(logits)
    gates = torch.softmax(logits, dim=-1)
    kwargs = dict(self.dispatcher_kwargs)
    use_bf16 = kwargs.pop("bfloat16", False)
    if (inputs.is_cuda and inputs.dtype == torch.bfloat16 and ops.cuda_kernels_enabled() and
        kwargs.get("name", "einsum") in ("einsum", "indices")):
      # GPU path: plan kernel + the indices-form layer shared with Top-K routing.
      from vmoe_b200.ops import moe_ops
      g, s, e = gates.shape
      if s <= moe_ops.EXPERTS_CHOOSE_MAX_ITEMS:
        capacity = moe._resolve_capacity(
            kwargs.get("capacity"), kwargs.get("capacity_factor"), s, e,
            kwargs.get("capacity_ceil_or_round", "ceil"), kwargs.get("capacity_multiple_of", 4))
        d = moe_ops.FusedTopItemsDispatcher(gates, capacity, exchange=self.exchange)
        metrics = d.metrics()
        metrics["auxiliary_loss"] = torch.zeros(g, dtype=gates.dtype, device=gates.device)
        return d, metrics
    d, metrics = moe.get_top_items_per_expert_dispatcher(gates, exchange=self.exchange, **kwargs)
    if use_bf16:
      d = moe.Bfloat16Dispatcher(d)
    metrics["auxiliary_loss"] = torch.zeros(gates.shape[0], dtype=gates.dtype, device=gates.device)
    return d, metrics
