"""Router losses (golden values from ``vmoe/nn/routing_test.py:39-80``) and stochasticity."""
import pytest
import torch

from vmoe_b200.models import routing

R = routing.NoisyTopExpertsPerItemRouter
GATES = torch.tensor([[.5, .4, .1], [.3, .3, .4], [.1, .2, .7], [.8, .2, .0]])


def test_gshard_auxiliary_loss():
  assert abs(float(R._gshard_auxiliary_loss(GATES)) - 1.0875) < 1e-6


def test_importance_auxiliary_loss():
  assert abs(float(R._importance_auxiliary_loss(GATES)) - 0.03874999) < 1e-6


def test_load_auxiliary_loss():
  logits = torch.tensor([[.9, .06, .04], [.7, .18, .12], [.85, .05, .1]])
  noise = torch.tensor([[-.037, .026, -.018], [-.074, .045, -.015], [-.067, -.059, .073]])
  out = R._load_auxiliary_loss(logits, logits + noise, noise_std=.1, num_selected_experts=2)
  assert abs(float(out) - 0.48573864536489236) < 1e-5


def _router(**kw):
  r = R(num_experts=4, hidden_size=4, num_selected_experts=2,
        dispatcher=dict(name="einsum", capacity=5, batch_priority=False), **kw)
  with torch.no_grad():
    r.dense.weight.copy_(torch.eye(4))
  return r


def test_forward_deterministic():
  x = torch.arange(20.).reshape(1, 5, 4)
  r = _router(noise_std=1.0, deterministic=True)
  torch.manual_seed(0); d1, m1 = r(x)
  torch.manual_seed(1); d2, m2 = r(x)
  torch.testing.assert_close(d1.combine_weights, d2.combine_weights)
  assert set(m1) == {"auxiliary_loss", "gshard_loss", "importance_loss"}
  torch.testing.assert_close(m1["auxiliary_loss"], m2["auxiliary_loss"])


def test_forward_not_deterministic():
  x = torch.arange(20.).reshape(1, 5, 4) / 10
  r = _router(noise_std=2.0, deterministic=False)
  torch.manual_seed(0); d1, m1 = r(x)
  torch.manual_seed(1); d2, m2 = r(x)
  assert (d1.combine_weights - d2.combine_weights).abs().sum() > 0.01
  torch.testing.assert_close(m1["importance_loss"], m2["importance_loss"])
  assert (m1["load_loss"] - m2["load_loss"]).abs().sum() > 1e-6


def test_injected_noise_and_gradients():
  x = torch.randn(2, 6, 4)
  r = _router(noise_std=1.0, deterministic=False)
  r.injected_noise = torch.zeros(2, 6, 4)
  d, m = r(x)
  m["auxiliary_loss"].sum().backward()
  assert r.dense.weight.grad is not None and r.dense.weight.grad.abs().sum() > 0


def test_router_validation():
  with pytest.raises(ValueError, match="num_experts >= num_selected_experts >= 1"):
    R(num_experts=2, hidden_size=4, num_selected_experts=3,
      dispatcher=dict(name="einsum", capacity=2, batch_priority=False))(torch.zeros(1, 2, 4))
  with pytest.raises(ValueError, match="inputs.ndim must be 3"):
    _router()(torch.zeros(5, 4))


def test_experts_choose_router():
  r = routing.NoisyTopItemsPerExpertRouter(num_experts=4, hidden_size=4, noise_std=0.0,
                                           dispatcher=dict(name="einsum", capacity=2))
  d, m = r(torch.randn(3, 8, 4))
  assert d.combine_weights.shape == (3, 8, 4, 2)
  assert float(m["auxiliary_loss"].abs().sum()) == 0.0
  assert "ratio_processed_items_by_at_least_4_experts" in m
