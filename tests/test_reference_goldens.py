"""Golden values taken from the reference's unit tests: ensemble losses and predictions
(``vmoe/evaluate/ensemble_test.py:26-98``), mixup (``vmoe/train/trainer_test.py:281-310``),
few-shot ridge regression (``vmoe/evaluate/fewshot_test.py:28-85``), best-L2 selection."""
from unittest import mock

import numpy as np
import pytest
import torch

from vmoe_b200.evaluate import ensemble
from vmoe_b200.evaluate import fewshot
from vmoe_b200.train import trainer

_P2 = torch.tensor([[.1, .9], [.2, .8], [.3, .7], [.4, .6]])
_P1 = torch.tensor([[.1], [.2], [.3], [.4]])


@pytest.mark.parametrize("size, expected", [(1, [1, 0, 1, 0]), (2, [1, 1]), (4, [1])])
def test_label_pred_ensemble_softmax(size, expected):
  logits = torch.log(torch.tensor([[.1, .9], [.8, .2], [.3, .7], [.6, .3]]))
  assert ensemble.label_pred_ensemble_softmax(logits, size).tolist() == expected


@pytest.mark.parametrize("size, labels, expected", [
    (1, [0, 1, 0, 1], [.1, .8, .3, .6]),
    (2, [0, 1], [.1, .2, .7, .6]),
    (4, [1], [.9, .8, .7, .6]),
])
def test_ensemble_softmax_xent_train(size, labels, expected):
  onehot = torch.nn.functional.one_hot(torch.tensor(labels), 2).float()
  loss = ensemble.ensemble_softmax_xent_train(torch.log(_P2), onehot, size)
  np.testing.assert_allclose(loss.numpy(), -np.log(expected), rtol=1e-5)


@pytest.mark.parametrize("size, labels, expected", [
    (1, [0, 1, 0, 1], [.1, .8, .3, .6]),
    (2, [0, 1], [.15, .65]),
    (4, [1], [(.9 + .8 + .7 + .6) / 4]),
])
def test_ensemble_softmax_xent_eval(size, labels, expected):
  onehot = torch.nn.functional.one_hot(torch.tensor(labels), 2).float()
  loss = ensemble.ensemble_softmax_xent_eval(torch.log(_P2), onehot, size)
  np.testing.assert_allclose(loss.numpy(), -np.log(expected), rtol=1e-5)


@pytest.mark.parametrize("size, labels, expected", [
    (1, [[0.], [1.], [0.], [1.]], [.9, .2, .7, .4]),
    (2, [[0.], [1.]], [.9, .8, .3, .4]),
    (4, [[1.]], [.1, .2, .3, .4]),
])
def test_ensemble_sigmoid_xent_train(size, labels, expected):
  logits = torch.log(_P1) - torch.log1p(-_P1)
  loss = ensemble.ensemble_sigmoid_xent_train(logits, torch.tensor(labels), size)
  np.testing.assert_allclose(loss.numpy(), -np.log(expected), rtol=1e-5)


@pytest.mark.parametrize("size, labels, expected", [
    (1, [[0.], [1.], [0.], [1.]], [.9, .2, .7, .4]),
    (2, [[0.], [1.]], [.85, .35]),
    (4, [[1.]], [.25]),
])
def test_ensemble_sigmoid_xent_eval(size, labels, expected):
  logits = torch.log(_P1) - torch.log1p(-_P1)
  loss = ensemble.ensemble_sigmoid_xent_eval(logits, torch.tensor(labels), size)
  np.testing.assert_allclose(loss.numpy(), -np.log(expected), rtol=1e-5)


@pytest.mark.parametrize("alphas, shape, expected", [
    ([[.6, .4]], (1, 2), [1.4, 2.4, 3.4, 4.4, 5.4, 4.]),
    ([[.6, .4], [.7, .3], [.5, .5], [1., 0.], [.9, .1], [.8, .2]], (6, 2),
     [1.4, 2.3, 3.5, 4., 5.1, 5.0]),
])
def test_mixup_with_given_weights(alphas, shape, expected):
  x = torch.tensor([1., 2., 3., 4., 5., 6.])
  # Dirichlet weights are normalised gamma draws: rows that already sum to one stay as given.
  with mock.patch.object(torch, "_standard_gamma", return_value=torch.tensor(alphas)):
    out = trainer.mixup(None, x, concentration=10.0, shape=shape)
  np.testing.assert_allclose(out.numpy(), expected, rtol=1e-6)


def test_mixup_argument_checks():
  x = torch.zeros(6, 2)
  with pytest.raises(ValueError, match="inconsistent shapes"):
    trainer.mixup(None, (x, torch.zeros(5, 2)), concentration=1.0, shape=(6, 2))
  with pytest.raises(ValueError, match="length >= 2"):
    trainer.mixup(None, x, concentration=1.0, shape=(2,))
  with pytest.raises(ValueError, match="roll_axis"):
    trainer.mixup(None, x, concentration=1.0, shape=(1, 2), roll_axis=1)
  with pytest.raises(ValueError, match="concentration"):
    trainer.mixup(None, x, concentration=0.0, shape=(1, 2))


@pytest.mark.parametrize("ndim, l2_reg", [(1, 0.0), (10, 10.0)])
def test_fewshot_ridge_regression_golden(ndim, l2_reg):
  # One informative dimension, two classes: the first test point is classified correctly,
  # the second is not.
  tr = np.pad(np.asarray([[-1.], [-2.], [2.], [1.]]), [(0, 0), (0, ndim - 1)])
  te = np.pad(np.asarray([[-1.], [-2.]]), [(0, 0), (0, ndim - 1)])
  cache = fewshot._precompute_cache(tr.astype(np.float32), np.asarray([0, 0, 1, 1]), 2)
  acc = fewshot._eig_fewshot_acc_fn(cache, te.astype(np.float32), np.asarray([0, 1]), l2_reg)
  assert acc == pytest.approx(0.5)


def test_fewshot_metrics_skip_invalid_examples():
  class Identity(torch.nn.Module):
    def forward(self, images):
      return images, {}
  tr = [{"image": torch.tensor([[-1.], [-2.], [2.], [1.], [1e9], [1e9]]),
         "label": torch.tensor([0, 0, 1, 1, 0, 1]),
         fewshot.VALID_KEY: torch.tensor([1, 1, 1, 1, 0, 0], dtype=torch.bool)}]
  te = [{"image": torch.tensor([[-1.], [-2.]]), "label": torch.tensor([0, 1]),
         fewshot.VALID_KEY: torch.tensor([1, 1], dtype=torch.bool)}]
  results = fewshot._compute_fewshot_metrics(Identity(), [2], [0.0], 2, tr, te,
                                             torch.device("cpu"))
  assert float(results[2, 0.0]) == pytest.approx(0.5)


def test_best_l2_is_chosen_by_mean_rank_over_datasets():
  l2_regs = [0.1, 1.0, 10.0]
  results = {
      "a": {(1, 0.1): 0.1, (1, 1.0): 0.5, (1, 10.0): 0.4, (5, 0.1): 0.9, (5, 1.0): 0.2, (5, 10.0): 0.1},
      "b": {(1, 0.1): 0.2, (1, 1.0): 0.3, (1, 10.0): 0.9, (5, 0.1): 0.8, (5, 1.0): 0.7, (5, 10.0): 0.1},
      "c": {(1, 0.1): 0.0, (1, 1.0): 0.6, (1, 10.0): 0.5, (5, 0.1): 0.7, (5, 1.0): 0.1, (5, 10.0): 0.6},
  }
  best = fewshot._find_best_l2_reg(results, [1, 5], l2_regs)
  assert best == {1: 1.0, 5: 0.1}
