"""PGD adversarial attacks and routing-change statistics.

``stateless_attack_pgd`` takes ``num_updates`` signed-gradient ascent steps of size
``max_epsilon / num_updates`` on the images. ``AttackState`` accumulates, over batches, the
number of images, prediction changes, correct predictions and losses before/after the attack
and, per router, the intersection-over-union of the experts selected before and after
(reference: ``vmoe/projects/adversarial_attacks/attacks.py:23-191``).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Iterable, Optional, Tuple

import torch


def stateless_attack_pgd(images: torch.Tensor, loss_of: Callable[[torch.Tensor], Tuple[torch.Tensor, Any]],
                         *, max_epsilon: float, num_updates: int,
                         generator: Optional[torch.Generator] = None) -> torch.Tensor:
  """``loss_of(x)`` returns ``(scalar loss, aux)``; gradients are taken w.r.t. ``x`` only."""
  del generator  # randomness of the model (router noise) comes from its own streams
  delta = max_epsilon / num_updates
  x = images.detach()
  for _ in range(num_updates):
    x = x.clone().requires_grad_(True)
    with torch.enable_grad():
      loss, _ = loss_of(x)
      (dx,) = torch.autograd.grad(loss, x)
    x = (x + delta * torch.sign(dx.to(x.dtype))).detach()
  return x


def sum_intersection_over_union(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
  """``a, b``: (batch, tokens, experts) combine weights; sum over examples of the mean (over
  tokens) IoU of the expert sets selected in ``a`` and ``b``."""
  assert a.dim() == 3, f"a.ndim = {a.dim()}"
  assert a.shape == b.shape, f"a.shape = {tuple(a.shape)} vs. b.shape = {tuple(b.shape)}"
  num_tokens = a.shape[1]
  a, b = (a > 0).float(), (b > 0).float()
  inter = (a * b).sum(-1)
  union = (a + b).sum(-1) - inter
  iou = torch.where(union > 0, inter / union.clamp_min(1e-30), torch.zeros_like(union))
  return iou.sum() / num_tokens


@dataclasses.dataclass
class AttackState:
  max_updates: int
  num_images: torch.Tensor
  num_changes: torch.Tensor
  num_correct: torch.Tensor  # (2,) before / after
  sum_loss: torch.Tensor     # (2,) before / after
  sum_iou_experts: Dict[str, torch.Tensor]

  @classmethod
  def create(cls, max_updates: int, router_keys: Iterable[str], device="cpu") -> "AttackState":
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)
    return cls(max_updates=max_updates, num_images=z((), dt=torch.int64),
               num_changes=z((), dt=torch.int64), num_correct=z(2, dt=torch.int64), sum_loss=z(2),
               sum_iou_experts={k: z(()) for k in router_keys})

  def update(self, **kwargs) -> "AttackState":
    new = {}
    for k, v in kwargs.items():
      cur = getattr(self, k)
      if isinstance(cur, dict):
        new[k] = {kk: cur[kk] + v[kk] for kk in cur}
      else:
        new[k] = cur + v
    return dataclasses.replace(self, **new)


def stateful_attack(attack_state: AttackState, x, y, valid, *, stateless_attack_fn,
                    compute_loss_predict_correct_cw_fn):
  """Attacks one batch and updates the statistics. Returns ``(new_state, x_adv, loss_before,
  loss_after, pred_before, pred_after, cw_before, cw_after)``."""
  assert x.dim() >= 1
  batch = x.shape[0]

  def mask(a):
    if valid is None:
      return a
    v = valid.reshape((batch,) + (1,) * max(a.dim() - valid.dim(), 0)).to(a.device)
    return a * v.to(a.dtype)

  x_0 = x
  x_m = stateless_attack_fn(x_0, y)
  l_0, y_0, c_0, cw_0 = compute_loss_predict_correct_cw_fn(x_0, y)
  l_m, y_m, c_m, cw_m = compute_loss_predict_correct_cw_fn(x_m, y)
  l_0, y_0, c_0, l_m, y_m, c_m = map(mask, (l_0, y_0, c_0, l_m, y_m, c_m))
  cw_0 = {k: mask(v) for k, v in cw_0.items()}
  cw_m = {k: mask(v) for k, v in cw_m.items()}
  num_images = torch.as_tensor(batch) if valid is None else valid.sum().long()
  new_state = attack_state.update(
      num_images=num_images.to(attack_state.num_images.device),
      num_changes=(y_m != y_0).sum().long(),
      num_correct=torch.stack([c_0.sum(), c_m.sum()]).long(),
      sum_loss=torch.stack([l_0.sum(), l_m.sum()]).float(),
      sum_iou_experts={k: sum_intersection_over_union(cw_0[k], cw_m[k]) for k in cw_0})
  return new_state, x_m, l_0, l_m, y_0, y_m, cw_0, cw_m
