"""Ensemble router and Soft MoE router: stochasticity, expert partitioning, layouts and
metric values. The cases follow the reference's tests
(``vmoe/nn/ensemble_routing_test.py:45-233``, ``vmoe/projects/soft_moe/router_test.py:33-98``).
"""
import math

import numpy as np
import pytest
import scipy.spatial.distance
import torch

from vmoe_b200 import moe
from vmoe_b200.models import ensemble_routing
from vmoe_b200.projects.soft_moe import router as soft_router


def _ensemble_router(num_groups, ens_size, deterministic):
  num_experts, batch = 4, 6 * ens_size
  x = torch.arange(num_experts * batch * num_groups, dtype=torch.float32)
  x = x.reshape(num_groups, batch, num_experts)
  layer = ensemble_routing.NoisyTopExpertsPerItemEnsembleRouter(
      num_experts=num_experts, hidden_size=num_experts, ensemble_size=ens_size,
      num_selected_experts=2 if ens_size == 1 else 1, noise_std=1.0,
      deterministic=deterministic,
      dispatcher=dict(name="einsum", capacity_factor=1.0, batch_priority=False))
  kernel = torch.eye(num_experts).reshape(num_experts, ens_size, num_experts // ens_size)
  with torch.no_grad():  # reference layout (hidden, M, E/M) -> (M, E/M, hidden)
    layer.dense.weight.copy_(kernel.permute(1, 2, 0))
  return layer, x


@pytest.mark.parametrize("num_groups, ens_size", [(1, 1), (1, 2), (2, 1), (2, 2)])
def test_ensemble_router_deterministic_ignores_the_seed(num_groups, ens_size):
  layer, x = _ensemble_router(num_groups, ens_size, deterministic=True)
  torch.manual_seed(0)
  g1, m1 = layer._compute_gates_softmax_and_metrics(x)
  torch.manual_seed(1)
  g2, m2 = layer._compute_gates_softmax_and_metrics(x)
  torch.testing.assert_close(g1, g2)
  for key in m1:
    torch.testing.assert_close(m1[key], m2[key])
    assert m1[key].shape == (num_groups, ens_size)


@pytest.mark.parametrize("num_groups, ens_size", [(1, 1), (1, 2), (2, 1), (2, 2)])
def test_ensemble_router_noise_depends_on_the_seed(num_groups, ens_size):
  layer, x = _ensemble_router(num_groups, ens_size, deterministic=False)
  torch.manual_seed(0)
  g1, m1 = layer._compute_gates_softmax_and_metrics(x)
  torch.manual_seed(1)
  g2, m2 = layer._compute_gates_softmax_and_metrics(x)
  assert (g1 - g2).abs().sum() > 1e-3
  # The importance loss is computed before the noise is added.
  torch.testing.assert_close(m1["importance_loss"], m2["importance_loss"])
  assert (m1["load_loss"] - m2["load_loss"]).abs().sum() > 1e-6
  for key in m1:
    assert m1[key].shape == (num_groups, ens_size)


def test_ensemble_router_selects_inside_the_members_expert_set():
  # x @ kernel alone would pick expert 3 for the first row and expert 1 for the second;
  # the partition restricts them to {0, 1} and {2, 3}.
  x = torch.arange(6, dtype=torch.float32).reshape(1, 2, 3)
  kernel = torch.tensor([[[1.0, 1.0], [-1.0, -1.0]],
                         [[-1.0, 1.0], [-1.0, -1.0]],
                         [[-1.0, -1.0], [-1.0, 1.0]]])  # (hidden, M, E/M)
  layer = ensemble_routing.NoisyTopExpertsPerItemEnsembleRouter(
      num_experts=4, hidden_size=3, ensemble_size=2, num_selected_experts=1, noise_std=1.0,
      deterministic=False, dispatcher=dict(name="einsum", capacity_factor=1.0))
  with torch.no_grad():
    layer.dense.weight.copy_(kernel.permute(1, 2, 0))
  torch.manual_seed(0)
  gates, _ = layer._compute_gates_softmax_and_metrics(x)
  selected = gates.argmax(dim=-1)
  assert int(selected[0, 0]) in (0, 1) and int(selected[0, 1]) in (2, 3)
  free = (x @ kernel.reshape(3, 4)).argmax(dim=-1)
  assert int(free[0, 0]) != int(selected[0, 0]) and int(free[0, 1]) != int(selected[0, 1])
  # Block-diagonal gates: nothing outside the member's own experts.
  gates = gates.detach()
  assert float(gates[0, 0, 2:].abs().sum()) == 0.0 and float(gates[0, 1, :2].abs().sum()) == 0.0


def test_ensemble_router_returns_a_dispatcher_and_validates():
  layer, x = _ensemble_router(2, 2, deterministic=True)
  dispatcher, metrics = layer(x)
  assert isinstance(dispatcher, moe.BaseDispatcher)
  assert "auxiliary_loss" in metrics
  bad = ensemble_routing.NoisyTopExpertsPerItemEnsembleRouter(
      num_experts=4, hidden_size=4, ensemble_size=3, num_selected_experts=1,
      dispatcher=dict(name="einsum", capacity_factor=1.0))
  with pytest.raises(ValueError, match="multiple of ensemble_size"):
    bad._compute_gates_softmax_and_metrics(torch.zeros(1, 6, 4))
  with pytest.raises(ValueError, match="group_size must be multiple"):
    layer._compute_gates_softmax_and_metrics(torch.zeros(1, 5, 4))


def test_group_representation_keeps_members_adjacent_and_round_trips():
  images, members, tokens, groups = 4, 2, 3, 2
  # Encode (image, member, token) in the value.
  x = torch.tensor([[[i * 100 + e * 10 + t] for t in range(tokens)]
                    for i in range(images) for e in range(members)], dtype=torch.float32)
  assert x.shape == (images * members, tokens, 1)
  group_size = images * members * tokens // groups
  y = ensemble_routing.reshape_to_group_size_representation(x, group_size, members)
  assert y.shape == (groups, group_size, 1)
  for g in range(groups):
    y_g = y[g].reshape(group_size // members, members, 1)
    for e in range(members):
      assert all(int(v) // 10 % 10 == e for v in y_g[:, e, 0])
  z = ensemble_routing.reshape_from_group_size_representation(y, tokens, members)
  assert torch.equal(z, x)


def test_cosine_psim_matches_scipy():
  x = torch.randn(6, 5, 4, 3, 2, generator=torch.Generator().manual_seed(0))
  y = soft_router.cosine_psim(x, (0,), (3, 4))
  assert y.shape == (6, 5, 4, 5, 4)
  pdist, squareform = scipy.spatial.distance.pdist, scipy.spatial.distance.squareform
  expected = np.stack([
      (1 - squareform(pdist(xi.reshape(20, -1).numpy(), metric="cosine"))).reshape(5, 4, 5, 4)
      for xi in x])
  np.testing.assert_allclose(y.numpy(), expected, rtol=1e-3, atol=1e-5)


def test_soft_router_parameter_shapes_and_dispatcher_type():
  layer = soft_router.SoftRouter(num_experts=5, hidden_size=16)
  dispatcher, _ = layer(torch.ones(1, 8, 16))
  assert layer.mu.shape == (16, 5, 2) and layer.scale.shape == ()
  assert isinstance(dispatcher, moe.Bfloat16Dispatcher)


def test_soft_router_metric_values():
  x = torch.tensor([[
      [[1, 0], [0, 1], [0, 0]],
      [[0, 0], [1, 0], [0, 0]],
      [[0, 1], [0, 0], [1, 0]],
      [[0, 0], [0, 0], [0, 1]],
  ]], dtype=torch.float32)
  mu = torch.tensor([
      [[1, 0], [2, 1], [-1, 0]],
      [[0, 1], [0, 1], [0, -1]],
  ], dtype=torch.float32)
  metrics = soft_router.SoftRouter(num_experts=3, hidden_size=2).get_metrics(x, x, mu)
  expected = {
      "auxiliary_loss": 0.0,
      "combine_weights_min_mean": 0.0, "combine_weights_max_mean": 1.0,
      "dispatch_weights_min_mean": 0.0, "dispatch_weights_max_mean": 1.0,
      "combine_weights_similarity_min": 0.0, "combine_weights_similarity_max": 0.0,
      "combine_weights_similarity_mean": 0.0,
      "dispatch_weights_similarity_min": 0.0, "dispatch_weights_similarity_max": 1.0,
      "dispatch_weights_similarity_mean": 4 / 30,
      "mu_similarity_min": -1.0, "mu_similarity_max": 1.0,
      "mu_similarity_mean": (1 / math.sqrt(2) - 2) / 15,
  }
  assert set(metrics) == set(expected)
  for key, value in expected.items():
    assert float(metrics[key]) == pytest.approx(value, abs=1e-5), key
