"""Rebuilds a model from a config and a sharded checkpoint, and extracts routing decisions.

Counterpart of ``vmoe/projects/adversarial_attacks/restore.py:38-176``. The reference captures
Flax "intermediates" of the router modules; here forward hooks on the router modules collect
the dispatcher that each router returns, and ``get_combine_weights`` turns every supported
dispatcher (einsum, indices, fused top-k, with or without the bf16 wrapper) into a
``(tokens, experts)`` matrix of combine weights.
"""
from __future__ import annotations

import contextlib
import functools
import logging
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from vmoe_b200 import moe
from vmoe_b200.models import routing
from vmoe_b200.models import ensemble_routing
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.utils import misc

SUPPORTED_ROUTERS = (
    routing.NoisyTopExpertsPerItemRouter,
    routing.NoisyTopItemsPerExpertRouter,
    ensemble_routing.NoisyTopExpertsPerItemEnsembleRouter,
)


def router_filter(module: torch.nn.Module, _=None) -> bool:
  return isinstance(module, SUPPORTED_ROUTERS)


def router_modules(model: torch.nn.Module) -> Dict[str, torch.nn.Module]:
  """Routers of ``model`` keyed by their module path with '/' separators."""
  return {name.replace(".", "/"): m for name, m in model.named_modules() if router_filter(m)}


@contextlib.contextmanager
def capture_dispatchers(model: torch.nn.Module):
  """Context manager yielding a dict that maps router path -> dispatcher of the last call."""
  captured: Dict[str, Any] = {}
  handles = []
  for key, module in router_modules(model).items():
    def hook(_, __, output, key=key):
      captured[key] = output[0] if isinstance(output, tuple) else output
    handles.append(module.register_forward_hook(hook))
  try:
    yield captured
  finally:
    for h in handles:
      h.remove()


def _dispatcher_combine_weights(dispatcher) -> torch.Tensor:
  if isinstance(dispatcher, moe.Bfloat16Dispatcher):
    dispatcher = dispatcher.dispatcher
  if isinstance(dispatcher, moe.EinsumDispatcher):
    return dispatcher.combine_weights.float().sum(dim=3)  # (G, S, E, C) -> (G, S, E)
  if isinstance(dispatcher, moe.DenseEinsumDispatcher):
    return dispatcher.combine_weights.float()
  if hasattr(dispatcher, "indices") and hasattr(dispatcher, "combine_weights"):
    # Indices form (also the fused top-k dispatcher): (G, S, K) -> (G, S, E).
    expert = dispatcher.indices[..., 0].long()
    e = dispatcher.num_experts
    valid = (expert >= 0) & (expert < e)
    one_hot = torch.nn.functional.one_hot(expert.clamp(0, e - 1), e).float()
    one_hot = one_hot * valid.unsqueeze(-1).float()
    return (one_hot * dispatcher.combine_weights.float().unsqueeze(-1)).sum(dim=2)
  raise TypeError(f"Unknown dispatcher type: {type(dispatcher)}")


def get_combine_weights(captured: Mapping[str, Any]) -> Dict[str, torch.Tensor]:
  """``{router path: (num_tokens, E) combine weights}`` from captured dispatchers."""
  out = {}
  for key, dispatcher in captured.items():
    cw = _dispatcher_combine_weights(dispatcher)
    out[key] = cw.reshape(-1, cw.shape[-1]).detach()
  return out


def compute_loss_predict_cw_fn(x: torch.Tensor, y: torch.Tensor, *, model: torch.nn.Module,
                               loss_fn: Callable[..., torch.Tensor]):
  """Per-example loss, top-1 prediction, correctness and per-router combine weights
  ``(batch, tokens, E)`` (``restore.py:38-52`` of the reference project)."""
  batch = x.shape[0]
  with torch.no_grad(), capture_dispatchers(model) as captured:
    logits, metrics = model(x)
    loss = loss_fn(logits, y, metrics)
  logits = logits.float()
  pred = logits.argmax(dim=-1)
  one_hot = torch.nn.functional.one_hot(pred, logits.shape[-1]).to(logits.dtype)
  labels = y if y.dim() == logits.dim() else torch.nn.functional.one_hot(
      y.long(), logits.shape[-1]).to(logits.dtype)
  correct = (one_hot * labels.to(logits.dtype)).sum(dim=-1)
  cws = {k: m.reshape(batch, -1, m.shape[1]) for k, m in get_combine_weights(captured).items()}
  return loss, pred, correct, cws


def create_mesh(num_expert_partitions: int) -> mesh_lib.Mesh:
  """Logical mesh with at most ``world size`` expert partitions (``restore.py:55-64``)."""
  import torch.distributed as dist
  world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
  if num_expert_partitions > world:
    logging.error(
        "The value of num_expert_partitions is %d, but the current number of devices is %d. "
        "Setting num_expert_partitions to %d", num_expert_partitions, world, world)
    num_expert_partitions = world
  return mesh_lib.get_auto_logical_mesh(num_expert_partitions)


def get_loss_fn(name: str, **kwargs):
  """Per-example loss ``fn(logits, labels)``: 'softmax_xent' or 'sigmoid_xent' (sum over
  classes)."""
  def softmax_xent(logits, labels, **kw):
    del kw
    logp = torch.log_softmax(logits.float(), dim=-1)
    if labels.dim() < logits.dim():
      return -logp.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1)
    return -(labels.float() * logp).sum(dim=-1)

  def sigmoid_xent(logits, labels, **kw):
    del kw
    z = logits.float()
    y = labels.float()
    return (torch.clamp_min(z, 0) - z * y + torch.log1p(torch.exp(-z.abs()))).sum(dim=-1)

  table = {"softmax_xent": softmax_xent, "sigmoid_xent": sigmoid_xent}
  if name not in table:
    raise ValueError(f"Unknown loss: name={name!r}")
  return functools.partial(table[name], **kwargs)


def get_loss_including_auxiliary_fn(name: str, *, attack_auxiliary_loss: bool = False, **kwargs):
  """``fn(logits, labels, metrics)``; adds the mean auxiliary loss when asked to attack it."""
  loss_fn = get_loss_fn(name, **kwargs)

  def fn(logits, labels, metrics):
    loss = loss_fn(logits, labels)
    if attack_auxiliary_loss:
      loss = loss + torch.as_tensor(metrics["auxiliary_loss"]).float().mean()
    return loss

  return fn


def restore_from_config(config: Mapping[str, Any], checkpoint_prefix: str,
                        image_shape: Tuple[int, int, int, int], mesh: mesh_lib.Mesh,
                        device: Optional[torch.device] = None):
  """Builds ``config.model`` in eval mode and fills it from the sharded checkpoint
  ``checkpoint_prefix`` (``.index`` + ``.data-*``); every rank reads only the expert blocks it
  owns. Returns ``(model, loss_fn, router_keys, extra_rng_keys)``
  (``restore.py:126-172`` of the reference project)."""
  from vmoe_b200 import models as models_lib
  from vmoe_b200.checkpoints import flax_layout
  from vmoe_b200.checkpoints import partitioned
  get = (lambda k, d=None: config.get(k, d)) if hasattr(config, "get") else (lambda k, d=None: d)
  model = models_lib.create_model(config["model"], deterministic=True, mesh=mesh,
                                  image_size=image_shape[1])
  if device is not None:
    model.to(device)
  model.eval()
  _, specs = flax_layout.to_flax(model)
  # Checkpoints hold either a bare parameter tree or a train state with a 'params' entry; the
  # shardings handed to the restore must mirror the structure of the index.
  flat_index = misc.flatten_dict(partitioned.read_index(checkpoint_prefix)["index"], sep="/")
  flat_specs = misc.flatten_dict(specs, sep="/")
  has_params = any(k.startswith("params/") for k in flat_index)
  shardings = misc.unflatten_dict({
      k: flat_specs.get(k[len("params/"):] if has_params else k) for k in flat_index}, sep="/")
  tree = partitioned.restore_checkpoint(checkpoint_prefix, shardings=shardings, mesh=mesh)
  params = tree["params"] if has_params else tree
  flax_layout.from_flax(model, params, mesh=mesh)
  loss_kwargs = dict(get("loss") or {"name": "softmax_xent"})
  loss_fn = get_loss_including_auxiliary_fn(**loss_kwargs)
  router_keys = set(router_modules(model).keys())
  extra_rng_keys = tuple(get("extra_rng_keys", ()) or ())
  return model, loss_fn, router_keys, extra_rng_keys
