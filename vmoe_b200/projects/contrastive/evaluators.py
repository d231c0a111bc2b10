"""Retrieval and zero-shot classification evaluators for two-tower models.

The reference wraps ``big_vision``'s evaluators and raises ``NotImplementedError`` when that
package is missing (``vmoe/projects/contrastive/evaluators.py:57-59,126-128``). Here both are
computed directly from the towers' embeddings on in-memory datasets: retrieval reports
recall@k in both directions, zero-shot embeds one prompt set per class.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Mapping, Sequence

import torch

from vmoe_b200.train import periodic_actions


@torch.no_grad()
def _embed(model, iterator, device, which: str):
  zs = []
  for batch in iterator:
    if which == "image":
      z, _ = model(torch.as_tensor(batch["image"]).to(device), None)
    else:
      z, _ = model(None, torch.as_tensor(batch["text"]).to(device))
    zs.append(z.float().cpu())
  return torch.cat(zs, 0)


def recall_at_k(sim: torch.Tensor, ks: Sequence[int] = (1, 5, 10)) -> Dict[str, float]:
  """``sim (N, N)``: similarity of query i to candidate j, ground truth on the diagonal."""
  n = sim.shape[0]
  ranks = (sim > sim.diagonal().unsqueeze(1)).sum(dim=1)
  return {f"recall@{k}": float((ranks < k).float().mean()) for k in ks if k <= n}


def retrieval_metrics(model, dataset: Iterable[Mapping[str, Any]], device) -> Dict[str, float]:
  batches = list(dataset)
  zi = _embed(model, batches, device, "image")
  zt = _embed(model, batches, device, "text")
  sim = zi @ zt.t()
  out = {f"img2txt/{k}": v for k, v in recall_at_k(sim).items()}
  out.update({f"txt2img/{k}": v for k, v in recall_at_k(sim.t()).items()})
  return out


def zeroshot_metrics(model, dataset: Iterable[Mapping[str, Any]], class_texts: torch.Tensor,
                     device) -> Dict[str, float]:
  """``class_texts (C, L)``: one tokenised prompt per class; batches hold image and label."""
  zc, _ = model(None, class_texts.to(device))
  correct = total = 0
  for batch in dataset:
    z, _ = model(torch.as_tensor(batch["image"]).to(device), None)
    pred = (z.float() @ zc.float().t()).argmax(-1).cpu()
    label = torch.as_tensor(batch["label"])
    correct += int((pred == label).sum())
    total += int(label.numel())
  return {"accuracy": correct / max(total, 1)}


def make_hook(kind: str, *, state, writer, progress, first_step, train_steps, dataset=None,
              class_texts=None, every_steps=None, every_secs=None, on_steps=None, **_):
  if dataset is None:
    raise NotImplementedError(
        f"The {kind} evaluator needs an in-memory `dataset` (and `class_texts` for zeroshot); "
        "the big_vision dataset readers the reference relies on are not available here.")
  device = next(state.model.parameters()).device
  def callback(step, t=None, **kw):
    was = state.model.training
    state.model.eval()
    with progress.timed(kind):
      if kind == "retrieval":
        metrics = retrieval_metrics(state.model, dataset, device)
      else:
        metrics = zeroshot_metrics(state.model, dataset, class_texts, device)
    state.model.train(was)
    writer.write_scalars(step, {f"{kind}/{k}": v for k, v in metrics.items()})
  return periodic_actions.PeriodicCallback(
      callback_fn=callback, every_steps=every_steps, every_secs=every_secs,
      on_steps=set(on_steps or []) | {first_step, train_steps})
