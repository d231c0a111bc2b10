"""Few-shot linear probing of frozen representations.

Features (the model output without a classification head) of a few-shot train and test split
are gathered on all ranks; for each number of shots, ``shot`` examples per class are picked
with a seeded permutation and a closed-form L2-regularised least-squares classifier on
standardised features (+ a constant bias feature of 100) is fit on the CPU through one
eigen-decomposition shared by all regularisers. The regulariser is chosen per shot by best
mean rank across datasets (reference: ``vmoe/evaluate/fewshot.py:52-418``).
"""
from __future__ import annotations

import time
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from vmoe_b200.data import input_pipeline, pjit_utils
from vmoe_b200.data.pp_ops import VALID_KEY
from vmoe_b200.train import periodic_actions

BIAS_CONSTANT = 100.0


def _precompute_cache(x: np.ndarray, y: np.ndarray, num_classes: int) -> Dict[str, np.ndarray]:
  x = x.astype(np.float64)
  mean = x.mean(axis=0, keepdims=True)
  std = x.std(axis=0, keepdims=True) + 1e-5
  x = (x - mean) / std
  x = np.pad(x, ((0, 0), (0, 1)), constant_values=BIAS_CONSTANT)
  yy = 2.0 * np.eye(num_classes)[y] - 1.0
  n, d = x.shape
  if n >= d:
    eigs, q = np.linalg.eigh(x.T @ x)
    rhs, lhs = q.T @ (x.T @ yy), q
  else:
    eigs, q = np.linalg.eigh(x @ x.T)
    rhs, lhs = q.T @ yy, x.T @ q
  return {"eigs": eigs, "rhs": rhs, "lhs": lhs, "mean": mean, "std": std}


def _eig_fewshot_acc_fn(cache, x_test: np.ndarray, y_test: np.ndarray, l2_reg: float) -> float:
  x = (x_test.astype(np.float64) - cache["mean"]) / cache["std"]
  x = np.pad(x, ((0, 0), (0, 1)), constant_values=BIAS_CONSTANT)
  scaling = (1.0 / (cache["eigs"] + l2_reg)).reshape(1, -1)
  w = (cache["lhs"] * scaling) @ cache["rhs"]
  return float(np.mean(np.argmax(x @ w, axis=1) == y_test))


def _find_best_l2_reg(all_results, shots, l2_regs):
  best = {}
  for shot in shots:
    ranks = []
    for res in all_results.values():
      accs = [res[shot, l2] for l2 in l2_regs]
      ranks.append(np.argsort(np.argsort(accs)))
    best[shot] = l2_regs[int(np.argmax(np.mean(ranks, axis=0)))]
  return best


def _gather(t: torch.Tensor) -> torch.Tensor:
  if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return torch.cat(out, 0)
  return t


@torch.no_grad()
def _compute_representation(model, iterator, device, input_dtype=None):
  feats, labels = [], []
  for batch in pjit_utils.prefetch_to_device(iter(iterator), size=1, device=device):
    images = batch["image"] if input_dtype is None else batch["image"].to(input_dtype)
    features, _ = model(images)
    valid = batch.get(VALID_KEY)
    valid = torch.ones(images.shape[0], dtype=torch.bool, device=device) if valid is None \
        else valid.to(device).bool()
    f, l, v = _gather(features.float()), _gather(batch["label"].to(device)), _gather(valid)
    feats.append(f[v].cpu().numpy())
    labels.append(l[v].cpu().numpy())
  return np.concatenate(feats, 0), np.concatenate(labels, 0)


def _compute_fewshot_metrics(model, shots, l2_regs, num_classes, tr_iter, te_iter, device,
                             seed: int = 0, input_dtype=None):
  tr_x, tr_y = _compute_representation(model, tr_iter, device, input_dtype)
  te_x, te_y = _compute_representation(model, te_iter, device, input_dtype)
  rng = np.random.default_rng(seed)
  class_indices = [rng.permutation(np.where(tr_y == c)[0]) for c in range(num_classes)]
  results = {}
  for shot in shots:
    idx = np.concatenate([ind[:shot] for ind in class_indices], axis=0)
    cache = _precompute_cache(tr_x[idx], tr_y[idx], num_classes)
    for l2 in l2_regs:
      results[shot, l2] = np.array(_eig_fewshot_acc_fn(cache, te_x, te_y, l2))
  return results


class FewShotPeriodicAction(periodic_actions.PeriodicCallback):
  """Runs few-shot evaluation on ``datasets = {key: (name, train_split, test_split)}``.

  ``model`` must return features (build it with ``num_classes=None``). Extra keyword
  arguments (``batch_size``, ``process`` ...) go to the dataset constructor; per-dataset
  ``num_classes`` comes from ``num_classes`` (a dict by key).
  """

  def __init__(self, *, model, datasets: Mapping[str, Tuple[str, str, str]],
               num_classes: Mapping[str, int], shots: Sequence[int], l2_regs: Sequence[float],
               metric_writer=None, main_task: Optional[Tuple[str, int]] = None,
               main_task_prefix: str = "0", seed: int = 0, report_progress=None,
               report_progress_name: str = "fewshot", dataset_kwargs: Optional[Mapping] = None,
               every_steps=None, every_secs=None, on_steps=None, input_dtype=None,
               dataset_iterators: Optional[Mapping[str, Tuple[Any, Any]]] = None):
    self._model = model
    self._writer = metric_writer
    self._shots, self._l2 = tuple(shots), tuple(l2_regs)
    self._seed = seed
    self._main_task = main_task
    self._prefix = main_task_prefix
    self._input_dtype = input_dtype
    self._num_classes = dict(num_classes)
    if dataset_iterators is not None:
      self._datasets = dict(dataset_iterators)
    else:
      kw = dict(dataset_kwargs or {})
      self._datasets = {
          key: (input_pipeline.get_dataset(variant="fewshot", name=name, split=tr, **kw),
                input_pipeline.get_dataset(variant="fewshot", name=name, split=te, **kw))
          for key, (name, tr, te) in datasets.items()}
    self.last_metrics: Dict[str, float] = {}

    def callback_fn(step, t=None, **kwargs):
      model_ = kwargs.get("model", self._model)
      was = model_.training
      model_.eval()
      device = next(model_.parameters()).device
      t0 = time.time()
      all_results = {}
      for key, (tr_it, te_it) in self._datasets.items():
        all_results[key] = _compute_fewshot_metrics(
            model_, self._shots, self._l2, self._num_classes[key], tr_it, te_it, device,
            self._seed, self._input_dtype)
        for it in (tr_it, te_it):
          if hasattr(it, "reset"):
            it.reset()
      model_.train(was)
      best_l2 = _find_best_l2_reg(all_results, self._shots, self._l2)
      metrics = {"fewshot/duration_secs": time.time() - t0}
      for key, res in all_results.items():
        for shot in self._shots:
          metrics[f"fewshot/{key}/{shot}shot"] = float(res[shot, best_l2[shot]])
      if self._main_task is not None:
        key, shot = self._main_task
        metrics[f"{self._prefix}/{key}/{shot}shot"] = float(all_results[key][shot, best_l2[shot]])
      self.last_metrics = metrics
      if self._writer is not None:
        self._writer.write_scalars(step, metrics)

    if report_progress is not None:
      inner = callback_fn
      def callback_fn(step, t=None, **kwargs):  # noqa: F811
        with report_progress.timed(report_progress_name):
          inner(step, t, **kwargs)
    super().__init__(callback_fn=callback_fn, every_steps=every_steps, every_secs=every_secs,
                     on_steps=on_steps)
