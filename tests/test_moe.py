"""MoE core: capacity, Top-K / BPR / experts-choose golden vectors, dispatcher equivalence.

Golden vectors are the reference's (``vmoe/moe_test.py:187-308``)."""
import numpy as np
import pytest
import torch

from vmoe_b200 import moe

GATES = torch.tensor([[.4, .0, .2], [.5, .1, .4], [.3, .2, .6]])


@pytest.mark.parametrize("n,e,cf,ror,mult,expected", [
    (32 * 2, 32, 1.0, "ceil", 4, 4), (1576 * 2, 8, 1.05, "ceil", 4, 416),
    (128, 32, 2.0, "ceil", 4, 8), (196, 128, 1.0, "round", 1, 2), (10, 4, 1.0, "ceil", None, 3)])
def test_compute_capacity(n, e, cf, ror, mult, expected):
  assert moe.compute_capacity(n, e, cf, ror, mult) == expected


def test_compute_capacity_raises():
  with pytest.raises(ValueError, match="must be greater than or equal to 1"):
    moe.compute_capacity(10, 100, 0.01, "round")
  with pytest.raises(ValueError, match="Unsupported"):
    moe.compute_capacity(10, 2, 1.0, "floor")


@pytest.mark.parametrize("bpr,expected", [
    (False, [[[.4, .0], [.0, .0], [.0, .2]], [[.0, .5], [.0, .0], [.0, .0]],
             [[.0, .0], [.0, .0], [.6, .0]]]),
    (True, [[[.0, .4], [.0, .0], [.0, .0]], [[.5, .0], [.0, .0], [.0, .4]],
            [[.0, .0], [.0, .0], [.6, .0]]])])
def test_top_experts_per_item_einsum(bpr, expected):
  d = moe.get_top_experts_per_item_dispatcher(GATES, "einsum", 2, bpr, capacity=2)
  np.testing.assert_allclose(d.combine_weights[0].numpy(), np.asarray(expected), atol=1e-6)


@pytest.mark.parametrize("bpr,expected", [
    (False, [[(0, 0), (2, 1)], [(0, 1), (2, 2)], [(2, 0), (0, 2)]]),
    (True, [[(0, 1), (2, 2)], [(0, 0), (2, 1)], [(2, 0), (0, 2)]])])
def test_top_experts_per_item_indices(bpr, expected):
  d = moe.get_top_experts_per_item_dispatcher(GATES, "indices", 2, bpr, capacity=2)
  assert d.num_experts == 3 and d.capacity == 2
  np.testing.assert_array_equal(d.indices[0].numpy(), np.asarray(expected))
  np.testing.assert_allclose(d.combine_weights[0].numpy(), [[.4, .2], [.5, .4], [.6, .3]], atol=1e-6)


def test_top_items_per_expert():
  d, metrics = moe.get_top_items_per_expert_dispatcher(GATES, "einsum", capacity=2)
  np.testing.assert_array_equal(
      d.dispatch_weights[0].numpy(),
      np.asarray([[[0, 1], [0, 0], [0, 0]], [[1, 0], [0, 1], [0, 1]], [[0, 0], [1, 0], [1, 0]]], bool))
  np.testing.assert_allclose(
      d.combine_weights[0].numpy(),
      [[[.0, .4], [.0, .0], [.0, .0]], [[.5, .0], [.0, .1], [.0, .4]], [[.0, .0], [.2, .0], [.6, .0]]],
      atol=1e-6)
  exp = {"num_experts_per_item_min": 1, "num_experts_per_item_max": 3, "min_selected_gate": .1,
         "max_selected_gate": .6, "ratio_processed_items_by_at_least_1_experts": 1.0,
         "ratio_processed_items_by_at_least_2_experts": 2 / 3,
         "ratio_processed_items_by_at_least_3_experts": 1 / 3}
  for k, v in exp.items():
    assert abs(float(metrics[k][0]) - v) < 1e-6, k


def test_dispatcher_errors():
  g = torch.zeros(4, 32)
  with pytest.raises(ValueError, match="Unknown dispatcher type"):
    moe.get_top_experts_per_item_dispatcher(g, "foo", 2, False, capacity=2)
  with pytest.raises(ValueError, match="You must specify either 'capacity' or 'capacity_factor'"):
    moe.get_top_experts_per_item_dispatcher(g, "einsum", 2, False)
  with pytest.raises(ValueError, match="Unknown dispatcher type"):
    moe.get_top_items_per_expert_dispatcher(g, "foo", capacity=2)


def test_capacity_factor_resolution():
  d = moe.get_top_experts_per_item_dispatcher(torch.rand(32, 32).softmax(-1), "indices", 2, False,
                                              capacity_factor=1.0)
  assert d.capacity == 4  # roundup4(ceil(32 * 2 / 32))
  d, _ = moe.get_top_items_per_expert_dispatcher(torch.rand(128, 32).softmax(-1), "einsum",
                                                 capacity_factor=2.0)
  assert d.combine_weights.shape[-1] == 128 * 2 // 32


@pytest.mark.parametrize("bpr", [False, True])
def test_einsum_and_indices_dispatchers_agree(bpr):
  torch.manual_seed(0)
  g, s, e, h, k, c = 3, 20, 4, 5, 2, 6
  gates = torch.rand(g, s, e).softmax(-1)
  x = torch.randn(g, s, h)
  d1 = moe.get_top_experts_per_item_dispatcher(gates, "einsum", k, bpr, capacity=c)
  d2 = moe.get_top_experts_per_item_dispatcher(gates, "indices", k, bpr, capacity=c)
  a, b = d1.dispatch(x), d2.dispatch(x)
  assert a.shape == (e, g * c, h)
  torch.testing.assert_close(a, b)
  y = torch.randn(e, g * c, h)
  torch.testing.assert_close(d1.combine(y), d2.combine(y))


def test_dispatch_combine_identity_expert():
  """With ample capacity, combine(dispatch(x)) = x * sum of the selected gates."""
  torch.manual_seed(1)
  g, s, e, h = 2, 8, 4, 3
  gates = torch.rand(g, s, e).softmax(-1)
  x = torch.randn(g, s, h)
  d = moe.get_top_experts_per_item_dispatcher(gates, "indices", 2, False, capacity=s)
  out = moe.sparse_moe_apply(lambda t: t, d, x)
  w = gates.topk(2, -1).values.sum(-1, keepdim=True)
  torch.testing.assert_close(out, x * w)


def test_dense_and_bfloat16_dispatchers():
  torch.manual_seed(2)
  gates = torch.rand(2, 5, 3).softmax(-1)
  x = torch.randn(2, 5, 4)
  d = moe.get_dense_einsum_dispatcher(gates)
  xe = d.dispatch(x)
  assert xe.shape == (3, 2 * 5, 4)
  torch.testing.assert_close(d.combine(xe), x)  # gates sum to one
  bd = moe.Bfloat16Dispatcher(moe.get_top_experts_per_item_dispatcher(gates, "einsum", 1, False, capacity=5))
  out = bd.dispatch(x)
  assert out.dtype == x.dtype
  torch.testing.assert_close(out, bd.dispatcher.dispatch(x.bfloat16()).float())


def test_sparse_moe_apply_has_aux_and_structures():
  gates = torch.rand(2, 6, 2).softmax(-1)
  x = torch.randn(2, 6, 3)
  d = moe.get_top_experts_per_item_dispatcher(gates, "indices", 1, False, capacity=6)
  (a, b), aux = moe.sparse_moe_apply(lambda t: ((t, 2 * t), t.sum()), d, x, has_aux=True)
  torch.testing.assert_close(b, 2 * a)
  assert aux.dim() == 0
