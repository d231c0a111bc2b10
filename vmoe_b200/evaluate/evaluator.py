"""Periodic evaluation on several datasets.

For every dataset the model runs in deterministic mode over all batches, accumulating the
number of valid examples, the number of correct predictions and the summed loss (each masked
by ``__valid__``), reduced over all ranks; the written metrics are ``<name>/prec@1``,
``<name>/loss`` and ``<name>/duration_secs``. A prediction counts as correct when the
predicted class is among the positive labels, so multi-label data works too (reference:
``vmoe/evaluate/evaluator.py:46-281``).
"""
from __future__ import annotations

import dataclasses
import time
from typing import Any, Callable, Dict, Iterable, Mapping, Optional

import torch
import torch.distributed as dist

from vmoe_b200.data import pjit_utils
from vmoe_b200.data.pp_ops import VALID_KEY
from vmoe_b200.train import periodic_actions


@dataclasses.dataclass
class EvalState:
  """Running sums of an evaluation pass."""
  num: torch.Tensor
  sum_correct: torch.Tensor
  sum_loss: torch.Tensor
  rngs: Optional[Dict[str, torch.Generator]] = None

  @classmethod
  def zeros(cls, device, rngs=None) -> "EvalState":
    z = lambda: torch.zeros((), dtype=torch.float64, device=device)
    return cls(num=z(), sum_correct=z(), sum_loss=z(), rngs=rngs)

  def update(self, num, correct, loss, rngs=None) -> "EvalState":
    return EvalState(num=self.num + num.sum().double(),
                     sum_correct=self.sum_correct + correct.sum().double(),
                     sum_loss=self.sum_loss + loss.sum().double(),
                     rngs=rngs or self.rngs)

  def all_reduce(self, group=None) -> "EvalState":
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
      packed = torch.stack([self.num, self.sum_correct, self.sum_loss])
      dist.all_reduce(packed, group=group)
      return EvalState(num=packed[0], sum_correct=packed[1], sum_loss=packed[2], rngs=self.rngs)
    return self


@torch.no_grad()
def evaluate_step(state: EvalState, model: torch.nn.Module, images, labels, valid,
                  loss_fn: Callable, label_pred_fn: Callable) -> EvalState:
  logits, _ = model(images)
  valid = valid.to(logits.device).float()
  loss = loss_fn(logits, labels).float() * valid
  pred = label_pred_fn(logits)
  onehot_pred = torch.nn.functional.one_hot(pred, labels.shape[-1]).to(labels.dtype)
  correct = valid * (labels * onehot_pred).sum(-1).float()
  return state.update(valid, correct, loss)


def evaluate_dataset(*, model, dataset: Iterable[Mapping[str, Any]], loss_fn, label_pred_fn,
                     device=None, input_dtype=None) -> EvalState:
  was_training = model.training
  model.eval()
  device = device or next(model.parameters()).device
  state = EvalState.zeros(device)
  try:
    for batch in pjit_utils.prefetch_to_device(iter(dataset), size=1, device=device):
      images = batch["image"]
      if input_dtype is not None:
        images = images.to(input_dtype)
      valid = batch.get(VALID_KEY)
      if valid is None:
        valid = torch.ones(images.shape[0], device=device)
      state = evaluate_step(state, model, images, batch["labels"].to(device), valid, loss_fn,
                            label_pred_fn)
  finally:
    model.train(was_training)
  return state.all_reduce()


class EvaluateMultipleDatasets(periodic_actions.PeriodicCallback):
  """Periodic callback evaluating ``model`` on every dataset of ``datasets``."""

  def __init__(self, *, model, datasets: Mapping[str, Any], loss_fn, label_pred_fn,
               metric_writer=None, report_progress=None,
               report_progress_name: str = "eval", input_dtype=None, **kwargs):
    self._model = model
    self._datasets = datasets
    self._loss_fn = loss_fn
    self._pred_fn = label_pred_fn
    self._writer = metric_writer
    self._input_dtype = input_dtype
    callback = self._make_callback_fn(report_progress, report_progress_name)
    super().__init__(callback_fn=callback, **kwargs)
    self.last_metrics: Dict[str, float] = {}

  def _make_callback_fn(self, report_progress, name):
    def callback_fn(step: int, t: Optional[float] = None, **kwargs):
      metrics: Dict[str, float] = {}
      for ds_name, dataset in self._datasets.items():
        t0 = time.time()
        state = evaluate_dataset(model=kwargs.get("model", self._model), dataset=dataset,
                                 loss_fn=self._loss_fn, label_pred_fn=self._pred_fn,
                                 input_dtype=self._input_dtype)
        num = max(float(state.num), 1.0)
        metrics[f"{ds_name}/prec@1"] = float(state.sum_correct) / num
        metrics[f"{ds_name}/loss"] = float(state.sum_loss) / num
        metrics[f"{ds_name}/duration_secs"] = time.time() - t0
        if hasattr(dataset, "reset"):
          dataset.reset()
      metrics.update(kwargs.get("extra_metrics") or {})
      self.last_metrics = metrics
      if self._writer is not None:
        self._writer.write_scalars(step, metrics)
    if report_progress is None:
      return callback_fn
    def timed(step, t=None, **kwargs):
      with report_progress.timed(name):
        callback_fn(step, t, **kwargs)
    return timed
