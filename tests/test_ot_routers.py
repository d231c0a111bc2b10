"""Optimal-transport routers: plans for a constant cost matrix are uniform, plans respect the
row / column marginals and the sparsity bound, noise follows the seed. Cases follow
``vmoe/projects/sparsity_constrained_ot/kl_projection_routing_test.py:35-150`` and
``ksparse_projection_routing_test.py:30-120``."""
import pytest
import torch

from vmoe_b200 import moe
from vmoe_b200.projects.sparsity_constrained_ot import ot_routing

_DISPATCHER = {"name": "einsum", "capacity_factor": 1.0, "batch_priority": False,
               "bfloat16": False}


def _set_identity_kernel(layer, n):
  with torch.no_grad():
    layer.dense.weight.copy_(torch.eye(n))


@pytest.mark.parametrize("use_lbfgs", [False, True])
def test_kl_plan_of_constant_costs_is_uniform(use_lbfgs):
  layer = ot_routing.KLProjectionNoisyTopExpertsPerItemRouter(
      num_experts=4, hidden_size=4, num_selected_experts=4, use_lbfgs=use_lbfgs, noise_std=0.0,
      deterministic=True, dispatcher=dict(_DISPATCHER))
  _set_identity_kernel(layer, 4)
  logits = layer.gating_logits(torch.ones(1, 5, 4))
  plan = layer.plan(logits)
  torch.testing.assert_close(plan.detach(), torch.full((1, 5, 4), 0.25), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("cls", [ot_routing.KLProjectionNoisyTopExpertsPerItemRouter,
                                 ot_routing.KSparseProjectionTransportTopExpertsPerItemRouter])
def test_tokens_choose_routers_follow_the_seed_only_with_noise(cls):
  x = torch.arange(2 * 8 * 4, dtype=torch.float32).reshape(2, 8, 4) / 16

  def run(deterministic, seed):
    layer = cls(num_experts=4, hidden_size=4, num_selected_experts=2, noise_std=2.0,
                load_loss_weight=1.0, deterministic=deterministic,
                dispatcher=dict(_DISPATCHER))
    _set_identity_kernel(layer, 4)
    torch.manual_seed(seed)
    dispatcher, metrics = layer(x)
    return dispatcher.combine_weights.detach(), metrics

  c1, m1 = run(True, 0)
  c2, m2 = run(True, 1)
  torch.testing.assert_close(c1, c2)
  torch.testing.assert_close(m1["auxiliary_loss"], m2["auxiliary_loss"])
  c1, m1 = run(False, 0)
  c2, m2 = run(False, 1)
  assert (c1 - c2).abs().sum() > 0.01
  torch.testing.assert_close(m1["importance_loss"], m2["importance_loss"])
  assert (m1["load_loss"] - m2["load_loss"]).abs().sum() > 1e-4


def test_row_sparse_plan_marginals_and_support():
  group_size, num_experts = 4, 2
  sim = torch.rand(1, group_size, num_experts, generator=torch.Generator().manual_seed(1))
  plan = ot_routing.regularized_semi_dual_plan(sim, nnz_k=1, row_sparse=True, maxiter=500,
                                               lr=0.05)
  torch.testing.assert_close(plan[0].sum(dim=1), torch.ones(group_size), atol=1e-3, rtol=0)
  torch.testing.assert_close(plan[0].sum(dim=0), torch.full((num_experts,), 2.0), atol=1e-1,
                             rtol=0)
  assert int((plan[0] > 0).sum(dim=1).max()) <= num_experts
  assert bool((plan >= 0).all())


def test_column_sparse_plan_has_at_most_capacity_nonzeros_per_expert():
  sim = torch.rand(2, 8, 4, generator=torch.Generator().manual_seed(0))
  plan = ot_routing.regularized_semi_dual_plan(sim, nnz_k=2, row_sparse=False, maxiter=300,
                                               lr=0.05)
  assert int((plan > 0).sum(dim=1).max()) <= 2
  torch.testing.assert_close(plan.sum(dim=1), torch.full((2, 4), 2.0), atol=1e-4, rtol=0)
  assert bool((plan >= 0).all())


def test_quadratic_plan_columns_carry_their_mass():
  sim = torch.rand(1, 8, 4, generator=torch.Generator().manual_seed(0))
  plan = ot_routing.regularized_semi_dual_plan(sim, nnz_k=None, row_sparse=False, maxiter=300,
                                               lr=0.05)
  torch.testing.assert_close(plan.sum(dim=1), torch.full((1, 4), 2.0), atol=1e-4, rtol=0)
  torch.testing.assert_close(plan.sum(dim=2), torch.ones(1, 8), atol=0.1, rtol=0)


@pytest.mark.parametrize("cls", [ot_routing.KLProjectionNoisyTopItemsPerExpertRouter,
                                 ot_routing.KSparseProjectionTransportTopItemsPerExpertRouter,
                                 ot_routing.SparseProjectionTransportTopItemsPerExpertRouter])
def test_experts_choose_routers_build_dispatchers(cls):
  layer = cls(num_experts=4, hidden_size=4, noise_std=1.0, deterministic=True,
              dispatcher={"name": "einsum", "capacity_factor": 1.0, "bfloat16": False})
  _set_identity_kernel(layer, 4)
  x = torch.randn(2, 8, 4, generator=torch.Generator().manual_seed(0))
  dispatcher, metrics = layer(x)
  assert isinstance(dispatcher, moe.BaseDispatcher)
  assert metrics["auxiliary_loss"].shape == (2,)
  y = dispatcher.combine(dispatcher.dispatch(x))
  assert y.shape == x.shape and bool(torch.isfinite(y).all())


def test_plans_are_differentiable_with_respect_to_the_logits():
  sim = torch.randn(1, 6, 3, generator=torch.Generator().manual_seed(0)).requires_grad_()
  ot_routing.sinkhorn_plan(sim, maxiter=10).square().sum().backward()
  assert sim.grad is not None and bool(torch.isfinite(sim.grad).all())
  assert float(sim.grad.abs().sum()) > 0
