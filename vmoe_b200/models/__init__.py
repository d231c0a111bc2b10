"""Model registry: names used in ``config.model.name`` -> classes (reference:
``vmoe/nn/models.py:17-20``), and construction from a config."""
from __future__ import annotations

from typing import Any, Mapping, Optional

from vmoe_b200.utils.misc import parse_call


def registry():
  from vmoe_b200.models import vit_moe
  reg = {"VisionTransformerMoe": vit_moe.VisionTransformerMoe}
  try:
    from vmoe_b200.models import vit_moe_ensemble
    reg["VisionTransformerMoeEnsemble"] = vit_moe_ensemble.VisionTransformerMoeEnsemble
  except ImportError:
    pass
  try:
    from vmoe_b200.models import external
    reg["VisionTransformer"] = external.VisionTransformer
    reg["MlpMixer"] = external.MlpMixer
  except ImportError:
    pass
  return reg


def _plain(obj):
  if hasattr(obj, "to_dict"):
    return obj.to_dict()
  if isinstance(obj, Mapping):
    return {k: _plain(v) for k, v in obj.items()}
  return obj


def create_model(config: Mapping[str, Any], deterministic: bool = False, **overrides):
  """Builds ``config.name`` with the remaining keys as keyword arguments."""
  kwargs = _plain(config)
  name = kwargs.pop("name")
  cls, args, kw2 = parse_call(name, registry())
  kwargs.update(kw2)
  kwargs.update(overrides)
  return cls(*args, deterministic=deterministic, **kwargs)
