"""Trainer units: gradient accumulation over micro-steps gives the gradients of the whole
batch, loss registry, training-cost function, config override
(reference tests: ``vmoe/train/trainer_test.py:245-296,606-650``)."""
import pytest
import torch

from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.train import optimizer as optim
from vmoe_b200.train import train_state
from vmoe_b200.train import trainer
from vmoe_b200.utils.config_dict import ConfigDict


class _Toy(torch.nn.Module):

  def __init__(self):
    super().__init__()
    g = torch.Generator().manual_seed(0)
    self.fc1 = torch.nn.Linear(6, 8)
    self.fc2 = torch.nn.Linear(8, 3)
    with torch.no_grad():
      for p in self.parameters():
        p.copy_(torch.randn(p.shape, generator=g) * 0.3)

  def forward(self, x):
    h = torch.tanh(self.fc1(x))
    return self.fc2(h), {"auxiliary_loss": h.square().mean(dim=-1)}


def _state():
  model = _Toy()
  named = [("params/" + n.replace(".", "/"), p) for n, p in model.named_parameters()]
  opt = optim.create_optimizer(named, name="sgd", total_steps=4, learning_rate=0.1, momentum=None)
  return train_state.TrainState(model=model, optimizer=opt,
                                mesh=mesh_lib.get_auto_logical_mesh(1))


@pytest.mark.parametrize("microsteps", [2, 4])
def test_microsteps_give_the_gradients_of_the_whole_batch(microsteps):
  g = torch.Generator().manual_seed(1)
  images = torch.randn(8, 6, generator=g)
  labels = torch.nn.functional.one_hot(torch.randint(0, 3, (8,), generator=g), 3).float()
  loss_fn, _, _ = trainer.get_loss_fn("softmax_xent")

  whole = _state()
  m1 = trainer.accumulate_gradients_and_metrics(whole, images, labels, loss_fn, None)
  split = _state()
  m2 = trainer.accumulate_gradients_and_metrics(split, images, labels, loss_fn, microsteps)
  for (n1, p1), (_, p2) in zip(whole.model.named_parameters(), split.model.named_parameters()):
    # Summed over the slices; the optimizer divides by the number of slices.
    torch.testing.assert_close(p2.grad / microsteps, p1.grad, rtol=1e-5, atol=1e-6, msg=n1)
  for key in ("main_loss", "auxiliary_loss", "total_loss"):
    torch.testing.assert_close(m2[key], m1[key], rtol=1e-5, atol=1e-6)

  # One optimizer update from either state lands on the same parameters.
  whole.apply_gradients_and_compute_global_norms(1)
  split.apply_gradients_and_compute_global_norms(microsteps)
  for p1, p2 in zip(whole.model.parameters(), split.model.parameters()):
    torch.testing.assert_close(p2, p1, rtol=1e-5, atol=1e-6)


def test_microsteps_must_divide_the_batch():
  state = _state()
  loss_fn, _, _ = trainer.get_loss_fn("softmax_xent")
  with pytest.raises(ValueError, match="not divisible"):
    trainer.accumulate_gradients_and_metrics(state, torch.zeros(6, 6), torch.zeros(6, 3),
                                             loss_fn, 4)


def test_loss_registry():
  logits = torch.tensor([[2.0, 0.0, -1.0]])
  labels = torch.tensor([[1.0, 0.0, 0.0]])
  train_fn, eval_fn, pred_fn = trainer.get_loss_fn("softmax_xent")
  want = -torch.log_softmax(logits, -1)[0, 0]
  torch.testing.assert_close(train_fn(logits, labels)[0], want)
  torch.testing.assert_close(eval_fn(logits, labels)[0], want)
  assert pred_fn(logits).tolist() == [0]
  train_fn, _, _ = trainer.get_loss_fn("sigmoid_xent")
  want = torch.nn.functional.binary_cross_entropy_with_logits(logits, labels,
                                                             reduction="none").sum(-1)
  torch.testing.assert_close(train_fn(logits, labels), want)
  _, eval_fn, pred_fn = trainer.get_loss_fn("ensemble_softmax_xent", ensemble_size=1)
  torch.testing.assert_close(eval_fn(logits, labels)[0], -torch.log_softmax(logits, -1)[0, 0])
  with pytest.raises(ValueError, match="Unknown loss"):
    trainer.get_loss_fn("hinge")


@pytest.mark.parametrize("flops, seconds, expected", [
    (None, None, {}),
    (2.0, None, {"flops": 2.0 * 42 * 2}),
    (None, 3.0, {"device_seconds": 3.0 * 42 * 2}),
    (2.0, 3.0, {"flops": 2.0 * 42 * 2, "device_seconds": 3.0 * 42 * 2}),
])
def test_train_cost_fn(flops, seconds, expected):
  fn = trainer.make_train_cost_fn(flops, seconds, num_devices=2)
  assert fn(42) == expected


def test_override_base_config():
  base = ConfigDict({"a": 1, "model": {"name": "x", "depth": 2}})
  out = trainer.override_base_config(base, ConfigDict({"model": {"depth": 3}, "b": 4}))
  assert out.a == 1 and out.b == 4 and out.model.depth == 3 and out.model.name == "x"
  assert base.model.depth == 2
