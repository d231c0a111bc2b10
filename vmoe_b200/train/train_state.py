"""Training state: model + optimizer + step counter + named RNG streams.

Counterpart of the reference's Flax ``TrainState`` (``vmoe/train/train_state.py:25-44``): the
state dict has the keys ``step / params / opt_state / rngs`` and
``apply_gradients_and_compute_global_norms`` returns the global L2 norms of gradients,
updates and new parameters.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Mapping, Optional

import torch

from vmoe_b200.models import naming
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.parallel import reduce as reduce_lib
from vmoe_b200.train.optimizer import Optimizer


@dataclasses.dataclass
class TrainState:
  model: torch.nn.Module
  optimizer: Optional[Optimizer]
  step: int = 0
  rngs: Optional[Dict[str, torch.Generator]] = None
  mesh: Optional[mesh_lib.Mesh] = None

  def apply_gradients_and_compute_global_norms(self, microsteps: int = 1,
                                               extra: Optional[torch.Tensor] = None):
    """All-reduces the accumulated gradients, applies the optimizer and bumps the step.

    ``extra``: per-rank scalars (1-D tensor) to average over all ranks together with the norm
    reduction; the averages are left in ``self.optimizer.last_extra``."""
    mesh = self.mesh or mesh_lib.get_mesh()
    reduce_lib.reduce_gradients(self.optimizer, mesh)
    norms = self.optimizer.step(grad_div=float(mesh.world_size * max(1, microsteps)), extra=extra)
    self.step += 1
    return norms

  # ------------------------------------------------------------------ (de)serialisation
  def params_dict(self) -> Dict[str, torch.Tensor]:
    return {key: p.data for key, _, p in naming.named_flax_parameters(self.model, prefix="")}

  def state_dict(self) -> Dict[str, Any]:
    out: Dict[str, Any] = {"step": self.step, "params": self.params_dict()}
    if self.optimizer is not None:
      out["opt_state"] = self.optimizer.state_dict()
    if self.rngs:
      out["rngs"] = {k: g.get_state() for k, g in self.rngs.items()}
    return out

  def load_state_dict(self, state: Mapping[str, Any]) -> None:
    self.step = int(state.get("step", 0))
    params = state.get("params", {})
    with torch.no_grad():
      for key, _, p in naming.named_flax_parameters(self.model, prefix=""):
        if key in params:
          p.data.copy_(torch.as_tensor(params[key]).to(p.device, p.dtype).reshape(p.shape))
    if self.optimizer is not None:
      if "opt_state" in state:
        st = dict(state["opt_state"])
        strip = lambda d: {k[len("params/"):] if k.startswith("params/") else k: v
                           for k, v in d.items()}
        # Optimizer entries are keyed by 'params/<path>'; accept bare paths too.
        for name in ("mu", "nu"):
          if name in st:
            st[name] = {("params/" + k if not k.startswith("params/") else k): v
                        for k, v in st[name].items()}
        self.optimizer.load_state_dict(st)
      self.optimizer.sync_shadows()
    if self.rngs and "rngs" in state:
      for k, s in state["rngs"].items():
        if k in self.rngs:
          self.rngs[k].set_state(torch.as_tensor(s, dtype=torch.uint8))
