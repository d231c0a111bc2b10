"""Routing for efficient ensembles of experts (E^3, https://arxiv.org/abs/2110.03360).

The batch is repeated M times (members adjacent), the E experts are split into M disjoint
sets of E/M, and member m is only routed inside set m: the gating matrix is block diagonal.
The gating layer has one ``(hidden, E/M)`` kernel per member — ``(hidden, M, E/M)`` in the
reference's layout (reference: ``vmoe/nn/ensemble_routing.py:43-134``).
"""
from __future__ import annotations


import torch
from torch import nn

from vmoe_b200.models import routing

Tensor = torch.Tensor


def reshape_to_group_size_representation(x: Tensor, group_size: int, ensemble_size: int) -> Tensor:
  """``(B*M, T, H)`` with members adjacent -> ``(G, group_size, H)`` where, inside a group,
  the M members of a token are adjacent."""
  bm, t, h = x.shape
  b = bm // ensemble_size
  x = x.reshape(b, ensemble_size, t, h).transpose(1, 2)
  return x.reshape(-1, group_size, h)


def reshape_from_group_size_representation(x: Tensor, num_tokens_per_image: int,
                                           ensemble_size: int) -> Tensor:
  h = x.shape[2]
  x = x.reshape(-1, num_tokens_per_image, ensemble_size, h).transpose(1, 2)
  return x.reshape(-1, num_tokens_per_image, h)


class NoisyTopExpertsPerItemEnsembleRouter(routing.NoisyTopExpertsPerItemRouter):

  def __init__(self, num_experts: int, hidden_size: int, ensemble_size: int = 1, **kwargs):
    super().__init__(num_experts, hidden_size, **kwargs)
    self.ensemble_size = ensemble_size
    if ensemble_size >= 1 and num_experts % ensemble_size == 0:
      del self.dense
      self.dense = _MemberGating(hidden_size, ensemble_size, num_experts // ensemble_size)

  def forward(self, inputs: Tensor):
    gates, metrics = self._compute_gates_softmax_and_metrics(inputs)
    return self._create_dispatcher(gates, inputs), metrics

  def _compute_gates_softmax_and_metrics(self, inputs: Tensor, num_experts=None):
    if inputs.dim() != 3:
      raise ValueError(f"inputs.ndim must be 3, but it is {inputs.dim()}")
    m, e = self.ensemble_size, self.num_experts
    if m <= 0:
      raise ValueError(f"Ensemble size must be >= 1; got {m}.")
    if e % m != 0:
      raise ValueError(f"num_experts must be multiple of ensemble_size, but got {e} and {m}.")
    g, s, h = inputs.shape
    if s % m != 0:
      raise ValueError(f"group_size must be multiple of ensemble_size, but got {s} and {m}.")
    em = e // m
    if not em >= self.num_selected_experts >= 1:
      raise ValueError(
          "num_experts >= num_selected_experts >= 1, but got "
          f"num_experts = {em} and num_selected_experts = {self.num_selected_experts}.")
    x = inputs.reshape(g, s // m, m, h)
    dtype = torch.float32 if (self.dtype or inputs.dtype) == torch.bfloat16 else (self.dtype or inputs.dtype)
    logits = torch.einsum("gsmh,meh->gsme", x.to(dtype), self.dense.weight.to(dtype))
    gates = inputs.new_zeros((g, s // m, m, e), dtype=dtype)
    per_member = []
    for i in range(m):
      noise = None
      if self.injected_noise is not None:
        noise = self.injected_noise.reshape(g, s // m, m, em)[:, :, i].to(logits)
      gi, mi = self._gates_and_metrics_from_logits(logits[:, :, i], em, noise=noise)
      gates[:, :, i, i * em:(i + 1) * em] = gi
      per_member.append(mi)
    metrics = {k: torch.stack([pm[k] for pm in per_member], dim=1) for k in per_member[0]}
    return gates.reshape(g, s, e), metrics


class _MemberGating(nn.Module):
  """Gating kernels of all members: ``weight (M, E/M, hidden)``."""

  def __init__(self, hidden_size: int, members: int, experts_per_member: int):
    super().__init__()
    self.weight = nn.Parameter(torch.empty(members, experts_per_member, hidden_size))
    for i in range(members):
      routing.lecun_normal_(self.weight[i], hidden_size)
