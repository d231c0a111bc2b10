"""Data pipeline, evaluator, ensemble losses and few-shot solver (CPU)."""
import math

import numpy as np
import pytest
import torch

from vmoe_b200.data import builder, input_pipeline, pjit_utils, pp_ops
from vmoe_b200.evaluate import ensemble, evaluator, fewshot


def test_parse_split_and_even_split():
  assert builder.parse_split("train[:99%]", 1000)[1:] == (0, 990)
  assert builder.parse_split("train[99%:]", 1000)[1:] == (990, 1000)
  assert builder.parse_split("validation[10:20]", 50)[1:] == (10, 20)
  parts = [builder.even_split(0, 10, i, 3) for i in range(3)]
  assert parts[0][0] == 0 and parts[-1][1] == 10
  assert sum(b - a for a, b in parts) == 10


def test_process_string_value_range_onehot_keep():
  fn = input_pipeline.get_data_process_fn(
      'value_range(-1,1)|onehot(5, inkey="label", outkey="labels")|keep("image", "labels")')
  out = fn({"image": np.full((4, 4, 3), 255, np.uint8), "label": np.int64(3), "extra": 1})
  assert set(out) == {"image", "labels"}
  np.testing.assert_allclose(np.asarray(out["image"]), 1.0)
  np.testing.assert_array_equal(np.asarray(out["labels"]), [0, 0, 0, 1, 0])


def test_resize_crop_flip_shapes():
  img = np.arange(8 * 6 * 3, dtype=np.uint8).reshape(8, 6, 3)
  out = pp_ops.resize(4)({"image": img})["image"]
  assert tuple(np.asarray(out).shape) == (4, 4, 3)
  out = pp_ops.central_crop(4)({"image": img})["image"]
  assert tuple(np.asarray(out).shape) == (4, 4, 3)
  pp_ops.set_rng(np.random.default_rng(0))
  flipped = [np.asarray(pp_ops.flip_lr()({"image": img})["image"]) for _ in range(8)]
  assert any(np.array_equal(f, img[:, ::-1]) for f in flipped)
  assert any(np.array_equal(f, img) for f in flipped)


def test_eval_dataset_pads_last_batch_with_invalid_examples():
  ds = input_pipeline.get_dataset(
      variant="test", name="synthetic", split="validation", batch_size=4, image_size=8,
      num_classes=3, num_eval_examples=6,
      process='value_range(-1,1)|onehot(3, inkey="label", outkey="labels")|keep("image", "labels")')
  batches = list(ds)
  assert len(batches) == 2
  valid = np.concatenate([np.asarray(b[input_pipeline.VALID_KEY]) for b in batches])
  assert valid.sum() == 6 and valid.shape == (8,)
  assert batches[0]["image"].shape == (4, 8, 8, 3)


def test_prefetch_to_device_passthrough_on_cpu():
  data = [{"x": np.ones((2, 3), np.float32) * i} for i in range(3)]
  out = list(pjit_utils.prefetch_to_device(iter(data), size=2, device=torch.device("cpu")))
  assert [float(o["x"].mean()) for o in out] == [0.0, 1.0, 2.0]


def test_prefetch_transforms_match_the_host_value_range_op():
  """uint8 images mapped to [-1, 1] by the prefetcher equal the host-side ``value_range`` op;
  uint8 labels are cast. (On a GPU the same functions run on the copy stream.)"""
  from vmoe_b200.data import pp_ops
  rng = np.random.default_rng(0)
  images = rng.integers(0, 256, size=(3, 2, 8, 8, 3), dtype=np.uint8)
  labels = rng.integers(0, 2, size=(3, 2, 5), dtype=np.uint8)
  data = [{"image": images[i], "labels": labels[i]} for i in range(3)]
  out = list(pjit_utils.prefetch_to_device(
      iter(data), size=2, device=torch.device("cpu"),
      dtypes={"labels": torch.float32},
      transforms={"image": pjit_utils.value_range_on_device(-1.0, 1.0)}))
  host_op = pp_ops.value_range(-1, 1)
  for i, o in enumerate(out):
    want = np.stack([host_op({"image": img})["image"] for img in images[i]])
    assert o["image"].dtype == torch.float32 and o["labels"].dtype == torch.float32
    np.testing.assert_allclose(o["image"].numpy(), want, atol=1e-6)
    np.testing.assert_array_equal(o["labels"].numpy(), labels[i].astype(np.float32))


def test_ensemble_losses_reduce_to_plain_losses_for_identical_members():
  torch.manual_seed(0)
  logits = torch.randn(4, 7)
  labels = torch.nn.functional.one_hot(torch.tensor([1, 3, 0, 6]), 7).float()
  rep = logits.repeat_interleave(3, dim=0)
  plain = -(labels * torch.log_softmax(logits, -1)).sum(-1)
  assert torch.allclose(ensemble.ensemble_softmax_xent_eval(rep, labels, 3), plain, atol=1e-5)
  train = ensemble.ensemble_softmax_xent_train(rep, labels, 3)
  assert train.shape == (12,) and torch.allclose(train[::3], plain, atol=1e-5)
  assert torch.equal(ensemble.label_pred_ensemble_softmax(rep, 3), logits.argmax(-1))
  bce = torch.nn.functional.binary_cross_entropy_with_logits(logits, labels, reduction="none").sum(-1)
  assert torch.allclose(ensemble.ensemble_sigmoid_xent_eval(rep, labels, 3), bce, atol=1e-5)


def test_ensemble_eval_averages_probabilities_not_logits():
  logits = torch.tensor([[4.0, 0.0], [0.0, 2.0]])  # two members, one example
  labels = torch.tensor([[1.0, 0.0]])
  p = torch.softmax(logits, -1).mean(0)
  want = -math.log(float(p[0]))
  got = float(ensemble.ensemble_softmax_xent_eval(logits, labels, 2))
  assert got == pytest.approx(want, rel=1e-5)


class _Const(torch.nn.Module):
  def __init__(self, logits):
    super().__init__()
    self.logits = torch.nn.Parameter(logits)

  def forward(self, images):
    return self.logits[: images.shape[0]], {}


def test_evaluate_dataset_masks_invalid_examples():
  logits = torch.tensor([[5.0, 0.0], [0.0, 5.0], [5.0, 0.0], [5.0, 0.0]])
  labels = torch.tensor([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0], [0.0, 1.0]])
  batch = {"image": torch.zeros(4, 2, 2, 3), "labels": labels,
           input_pipeline.VALID_KEY: torch.tensor([1.0, 1.0, 1.0, 0.0])}
  loss_fn = lambda lg, lb: -(lb * torch.log_softmax(lg, -1)).sum(-1)
  state = evaluator.evaluate_dataset(model=_Const(logits), dataset=[batch], loss_fn=loss_fn,
                                     label_pred_fn=lambda lg: lg.argmax(-1))
  assert float(state.num) == 3 and float(state.sum_correct) == 1


def test_fewshot_ridge_solver_separates_clusters():
  rng = np.random.default_rng(0)
  centers = rng.normal(size=(3, 8)) * 5
  y = np.repeat(np.arange(3), 5)
  x = centers[y] + rng.normal(size=(15, 8)) * 0.1
  cache = fewshot._precompute_cache(x.astype(np.float32), y, 3)
  acc = fewshot._eig_fewshot_acc_fn(cache, x.astype(np.float32), y, 2.0 ** -6)
  assert acc == pytest.approx(1.0)
