"""V-MoE with ensemble routing (E^3): tokens are repeated ``ensemble_size`` times before the
first MoE block and each copy is routed inside its own subset of experts; the output has
``batch * ensemble_size`` rows with the members of an example adjacent (reference:
``vmoe/nn/vit_moe_ensemble.py:37-132``)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from vmoe_b200.models import ensemble_routing, vit_moe


class MlpMoeWithNoisyTopExpertsPerItemEnsembleRouter(vit_moe.MlpMoeBlock):

  def __init__(self, *args, ensemble_size: Optional[int] = None, **kwargs):
    self.ensemble_size = int(ensemble_size or 1)
    super().__init__(*args, **kwargs)

  def create_router(self, hidden_size, num_experts, router, dtype):
    kwargs = dict(num_experts=num_experts, **(router or {}))
    kwargs.pop("name", None)
    return ensemble_routing.NoisyTopExpertsPerItemEnsembleRouter(
        hidden_size=hidden_size, dtype=dtype, exchange=self.exchange,
        ensemble_size=self.ensemble_size, **kwargs)

  def forward(self, inputs, residual=None):
    tokens = inputs.shape[1]
    x = ensemble_routing.reshape_to_group_size_representation(inputs, self.group_size,
                                                              self.ensemble_size)
    out, metrics = super().forward(x, residual=None)
    out = ensemble_routing.reshape_from_group_size_representation(out, tokens, self.ensemble_size)
    if residual is not None:
      out = out + residual
    return out, metrics


class EncoderMoeEnsemble(vit_moe.EncoderMoe):

  def __init__(self, *args, moe: Optional[Dict[str, Any]] = None, **kwargs):
    self.ensemble_size = int(dict(moe or {}).get("ensemble_size") or 1)
    super().__init__(*args, moe=moe,
                     moe_block_cls=MlpMoeWithNoisyTopExpertsPerItemEnsembleRouter, **kwargs)

  def forward(self, inputs):
    assert inputs.dim() == 3, f"Expected ndim = 3, but got shape {tuple(inputs.shape)}"
    x = self.add_position_emb(inputs)
    if self.training and self.dropout_rate > 0:
      x = torch.nn.functional.dropout(x, self.dropout_rate, True)
    metrics: Dict[str, Any] = {}
    first = True
    for block in range(self.num_layers):
      if block in self.moe_layers and first:
        x = x.repeat_interleave(self.ensemble_size, dim=0)
        first = False
      out = getattr(self, f"encoderblock_{block}")(x)
      if isinstance(out, tuple):
        x, metrics[f"encoderblock_{block}"] = out
      else:
        x = out
    encoded = self.encoder_norm(x)
    aux = [m["auxiliary_loss"] for m in metrics.values()]
    metrics["auxiliary_loss"] = sum(aux) if aux else torch.zeros((), device=x.device)
    return encoded, metrics


class VisionTransformerMoeEnsemble(vit_moe.VisionTransformerMoe):
  encoder_cls = EncoderMoeEnsemble
