"""Losses and predictions for efficient ensembles of experts (E^3).

Logits arrive as ``(B*M, C)`` with the M members of one example adjacent (the model repeats,
not tiles, its inputs). Training uses the plain cross-entropy on labels repeated M times; the
evaluation loss is the negative log of the member-averaged probability; the prediction is the
argmax of that average (reference: ``vmoe/evaluate/ensemble.py:56-160``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from vmoe_b200.utils.misc import multiply_no_nan


def _repeat_labels(labels: torch.Tensor, ensemble_size: int) -> torch.Tensor:
  return labels.repeat_interleave(ensemble_size, dim=0)


def ensemble_softmax_xent_train(logits, labels, ensemble_size: int):
  lab = _repeat_labels(labels, ensemble_size).float()
  return -(lab * F.log_softmax(logits.float(), dim=-1)).sum(-1)


def ensemble_sigmoid_xent_train(logits, labels, ensemble_size: int):
  lab = _repeat_labels(labels, ensemble_size).float()
  return F.binary_cross_entropy_with_logits(logits.float(), lab, reduction="none").sum(-1)


def _member_view(logits, ensemble_size):
  return logits.float().reshape(-1, ensemble_size, logits.shape[-1])


def ensemble_softmax_xent_eval(logits, labels, ensemble_size: int):
  """-sum_c y_c log(mean_m softmax(logits_m)_c)."""
  logp = F.log_softmax(_member_view(logits, ensemble_size), dim=-1)
  log_mean = torch.logsumexp(logp, dim=1) - math.log(ensemble_size)
  return -multiply_no_nan(labels.float(), log_mean).sum(-1)


def ensemble_sigmoid_xent_eval(logits, labels, ensemble_size: int):
  """Binary cross-entropy on the member-averaged per-class probabilities."""
  x = _member_view(logits, ensemble_size)
  log_p = torch.logsumexp(F.logsigmoid(x), dim=1) - math.log(ensemble_size)
  log_not_p = torch.logsumexp(F.logsigmoid(-x), dim=1) - math.log(ensemble_size)
  lab = labels.float()
  return -(lab * log_p + (1.0 - lab) * log_not_p).sum(-1)


def label_pred_ensemble_softmax(logits, ensemble_size: int):
  logp = F.log_softmax(_member_view(logits, ensemble_size), dim=-1)
  return torch.logsumexp(logp, dim=1).argmax(-1)


def label_pred_ensemble_sigmoid(logits, ensemble_size: int):
  x = _member_view(logits, ensemble_size)
  return torch.logsumexp(F.logsigmoid(x), dim=1).argmax(-1)
