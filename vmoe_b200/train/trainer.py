"""Training loop pieces: losses, the train step with gradient accumulation, train-state
construction, and ``train_and_evaluate``.

Reference: ``vmoe/train/trainer.py`` — ``accumulate_gradients_and_metrics`` :76-131,
``get_loss_fn`` :441-477, ``get_train_steps_and_epochs`` :480-497, ``train_step`` :648-684,
``train_and_evaluate`` :687-838.
"""
from __future__ import annotations

import functools
import logging
import math
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from vmoe_b200 import models as models_lib
from vmoe_b200.models import naming
from vmoe_b200.ops import losses as losses_ops
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.train import optimizer as optimizer_lib
from vmoe_b200.train.train_state import TrainState
from vmoe_b200.utils import misc

Tensor = torch.Tensor


# ------------------------------------------------------------------------------------ losses
def get_loss_fn(name: str, **kwargs):
  """Returns ``(train_loss_fn, eval_loss_fn, label_pred_fn)`` for a loss name."""
  from vmoe_b200.evaluate import ensemble
  default_pred = lambda logits: logits.argmax(-1)
  table = {
      "softmax_xent": (losses_ops.softmax_xent, losses_ops.softmax_xent, default_pred),
      "sigmoid_xent": (losses_ops.sigmoid_xent, losses_ops.sigmoid_xent, default_pred),
      "ensemble_softmax_xent": (ensemble.ensemble_softmax_xent_train,
                                ensemble.ensemble_softmax_xent_eval,
                                ensemble.label_pred_ensemble_softmax),
      "ensemble_sigmoid_xent": (ensemble.ensemble_sigmoid_xent_train,
                                ensemble.ensemble_sigmoid_xent_eval,
                                ensemble.label_pred_ensemble_sigmoid),
  }
  if name not in table:
    raise ValueError(f"Unknown loss: {name!r}")
  train_fn, eval_fn, pred_fn = table[name]
  train_fn = functools.partial(train_fn, **kwargs)
  eval_fn = functools.partial(eval_fn, **kwargs)
  if name.startswith("ensemble_"):
    pred_fn = functools.partial(pred_fn, **kwargs)
  return train_fn, eval_fn, pred_fn


def get_train_steps_and_epochs(*, train_batch_size: int, train_examples: int,
                               train_steps: Optional[int] = None,
                               train_epochs: Optional[float] = None) -> Tuple[int, float]:
  if (train_steps is None) == (train_epochs is None):
    raise ValueError("You must specify either `train_steps` or `train_epochs`, but not both: "
                     f"train_steps = {train_steps!r}, train_epochs = {train_epochs!r}")
  if train_epochs is not None:
    train_steps = int(math.ceil(train_epochs * train_examples / train_batch_size))
  else:
    train_epochs = train_steps * train_batch_size / train_examples
  return int(train_steps), float(train_epochs)


# ------------------------------------------------------------------------------------ step
def _mean_metrics(metrics: Mapping[str, Any]) -> Dict[str, Any]:
  out: Dict[str, Any] = {}
  for k, v in metrics.items():
    if isinstance(v, Mapping):
      out[k] = _mean_metrics(v)
    elif isinstance(v, torch.Tensor):
      out[k] = v.float().mean()
    else:
      out[k] = v
  return out


def _tree_add(a, b):
  if isinstance(a, Mapping):
    return {k: _tree_add(a[k], b[k]) for k in a}
  return a + b


def _tree_scale(a, s):
  if isinstance(a, Mapping):
    return {k: _tree_scale(v, s) for k, v in a.items()}
  return a * s


def compute_loss_and_metrics(state: TrainState, images: Tensor, labels: Tensor,
                             loss_fn: Callable[[Tensor, Tensor], Tensor]):
  """Forward pass: ``total = mean(loss) + mean(auxiliary_loss)``; all metrics are means."""
  logits, metrics = state.model(images)
  metrics = dict(metrics)
  metrics["main_loss"] = loss_fn(logits, labels).float().mean()
  metrics = _mean_metrics(metrics)
  total = metrics["main_loss"] + metrics.get("auxiliary_loss", 0.0)
  metrics["total_loss"] = total
  return total, metrics


def train_step(state: TrainState, images: Tensor, labels: Tensor,
               loss_fn: Callable[[Tensor, Tensor], Tensor], microsteps: Optional[int] = None,
               summarizer=None) -> Tuple[TrainState, Dict[str, Any]]:
  """One optimizer update; with ``microsteps`` the batch is processed in that many slices
  whose gradients and metrics are averaged (each slice keeps every ``microsteps``-th example,
  as the reference's reshape ``(-1, microsteps, ...)`` does)."""
  state.model.train()
  state.optimizer.zero_grad()
  n = microsteps or 1
  if n > 1 and images.shape[0] % n:
    raise ValueError(f"batch {images.shape[0]} is not divisible by microsteps={n}")
  metrics = None
  for i in range(n):
    im = images if n == 1 else images[i::n]
    lb = labels if n == 1 else labels[i::n]
    total, m = compute_loss_and_metrics(state, im, lb, loss_fn)
    total.backward()
    m = {k: (v.detach() if isinstance(v, torch.Tensor) else v) for k, v in m.items()}
    metrics = m if metrics is None else _tree_add(metrics, _detach_tree(m))
  if n > 1:
    metrics = _tree_scale(metrics, 1.0 / n)
  grads_for_summary = None
  if summarizer is not None:
    grads_for_summary = {key: p.grad.detach().clone() / n for key, _, p in
                         naming.named_flax_parameters(state.model, prefix="")
                         if p.grad is not None}
  norms = state.apply_gradients_and_compute_global_norms(microsteps=n)
  metrics.update({f"global_norm/{k}": v for k, v in norms.items()})
  if summarizer is not None:
    flat = misc.flatten_dict(state.state_dict(), sep="/")
    flat.update({f"params_grads/{k}": v for k, v in grads_for_summary.items()})
    metrics.update(summarizer(flat))
  return state, metrics


def _detach_tree(m):
  if isinstance(m, Mapping):
    return {k: _detach_tree(v) for k, v in m.items()}
  return m.detach() if isinstance(m, torch.Tensor) else m


# ------------------------------------------------------------------------------------ state
def create_train_state(*, model_config: Mapping[str, Any], optimizer_config: Mapping[str, Any],
                       total_steps: int, mesh: Optional[mesh_lib.Mesh] = None,
                       device: Optional[torch.device] = None, seed: int = 0,
                       extra_rng_keys=(), **model_overrides) -> TrainState:
  """Builds the model (same seed on every rank, so replicated weights agree), moves it to the
  device and wraps its parameters in the flat-buffer optimizer."""
  mesh = mesh or mesh_lib.get_mesh()
  torch.manual_seed(seed)
  model = models_lib.create_model(model_config, deterministic=False, mesh=mesh, **model_overrides)
  if device is not None:
    model.to(device)
  opt_kwargs = dict(optimizer_config.to_dict() if hasattr(optimizer_config, "to_dict")
                    else optimizer_config)
  named = [(key, p) for key, _, p in naming.named_flax_parameters(model, prefix="params")]
  opt = optimizer_lib.create_optimizer(named, total_steps=total_steps, mesh=mesh, **opt_kwargs)
  rngs = misc.make_rngs(tuple(extra_rng_keys) + ("dropout", "gating"), seed)
  return TrainState(model=model, optimizer=opt, step=0, rngs=rngs, mesh=mesh)
