"""Training loop pieces: losses, the train step with gradient accumulation, train-state
construction, and ``train_and_evaluate``.

Reference: ``vmoe/train/trainer.py`` — ``accumulate_gradients_and_metrics`` :76-131,
``get_loss_fn`` :441-477, ``get_train_steps_and_epochs`` :480-497, ``train_step`` :648-684,
``train_and_evaluate`` :687-838.
"""
from __future__ import annotations

import contextlib

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
    reducer = getattr(state.optimizer, "grad_reducer", None)
    if reducer is not None and i == n - 1:
      reducer.begin()  # gradients are complete after this backward: reduce them as they appear
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
  # The metrics are means over this rank's examples; the logged values are means over the global
  # batch (``vmoe/train/trainer.py:663-666``). They ride in the optimizer's one small
  # all-reduce instead of getting collectives of their own.
  flat_metrics = misc.flatten_dict(metrics, sep="\x00")
  keys = [k for k, v in flat_metrics.items() if isinstance(v, torch.Tensor) and v.dim() == 0
          and v.is_floating_point()]
  mesh = state.mesh or mesh_lib.get_mesh()
  extra = None
  if keys and mesh is not None and mesh.world_size > 1:
    extra = torch.stack([flat_metrics[k].detach().float() for k in keys])
  norms = state.apply_gradients_and_compute_global_norms(microsteps=n, extra=extra)
  if extra is not None and state.optimizer.last_extra is not None:
    for k, v in zip(keys, state.optimizer.last_extra.unbind(0)):
      flat_metrics[k] = v
    metrics = misc.unflatten_dict(flat_metrics, sep="\x00")
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
  from vmoe_b200.parallel import grad_allreduce
  opt.grad_reducer = grad_allreduce.maybe_create(opt, mesh, model)
  rngs = misc.make_rngs(tuple(extra_rng_keys) + ("dropout", "gating"), seed)
  return TrainState(model=model, optimizer=opt, step=0, rngs=rngs, mesh=mesh)


# ------------------------------------------------------------------------------------ mixup
def mixup(generator: Optional[torch.Generator], tree, *, concentration: float,
          shape: Tuple[int, ...] = (1, 2), roll_axis: int = 0):
  """Mixes every array of ``tree`` with rolled copies of itself using Dirichlet weights.

  ``shape[:-1]`` must broadcast against the leading dims of the arrays and ``shape[-1]`` is
  the number of examples mixed together. Weights are sorted in decreasing order so that the
  un-rolled example keeps the largest one; the same weights are used for all arrays.
  """
  arrays = list(tree) if isinstance(tree, (tuple, list)) else [tree]
  if len(shape) < 2:
    raise ValueError(f"Mixup 'shape' has length {len(shape)}, but it must have length >= 2.")
  batch_ndim = len(shape) - 1
  for i, x in enumerate(arrays):
    try:
      torch.broadcast_shapes(tuple(x.shape[:batch_ndim]), tuple(shape[:-1]))
    except RuntimeError:
      raise ValueError(
          f"Mixup with inconsistent shapes. The shape of the {i}-th array is "
          f"{tuple(x.shape)}, but the first {batch_ndim} dims must be broadcastable to "
          f"{tuple(shape[:-1])}") from None
    if tuple(x.shape[:batch_ndim]) != tuple(arrays[0].shape[:batch_ndim]):
      raise ValueError(
          f"Mixup with inconsistent shapes. The shape of the {i}-th array is "
          f"{tuple(x.shape)}, but the first {batch_ndim} dims must be equal to "
          f"{tuple(arrays[0].shape[:batch_ndim])}")
  if not 0 <= roll_axis < batch_ndim:
    raise ValueError(
        f"Mixup 'roll_axis' must be an integer in [0, {batch_ndim}), but got roll_axis = {roll_axis}")
  if concentration <= 0.0:
    raise ValueError(
        f"Mixup 'concentration' must be greater than 0, but got concentration = {concentration}")
  # Dirichlet(alpha) = normalised Gamma(alpha, 1) samples (drawn on the CPU generator).
  gamma = torch._standard_gamma(torch.full(tuple(shape), float(concentration)),
                                generator=generator)
  alpha = gamma / gamma.sum(-1, keepdim=True).clamp_min(1e-30)
  alpha = torch.sort(alpha, dim=-1, descending=True).values
  alpha = torch.movedim(alpha, -1, 0)  # (size, *batch dims)
  def mix(x):
    from vmoe_b200.ops import elementwise
    if (roll_axis == batch_ndim - 1 and not x.requires_grad and
        elementwise.mixup_supported(x, shape[-1])):
      # One kernel instead of `size` rolled copies: the weights depend only on the dims up to
      # and including the rolled one.
      full = alpha.expand((alpha.shape[0],) + tuple(x.shape[:batch_ndim])).contiguous()
      return elementwise.mixup_rows(x, full, roll_axis)
    a = alpha.to(device=x.device, dtype=x.dtype if x.is_floating_point() else torch.float32)
    a = a.reshape(tuple(a.shape) + (1,) * (x.dim() - batch_ndim))
    return sum(a[i] * torch.roll(x, -i, dims=roll_axis) for i in range(shape[-1]))
  out = [mix(x) for x in arrays]
  return type(tree)(out) if isinstance(tree, (tuple, list)) else out[0]


def wrap_train_step_with_mixup(train_step_fn, *, concentration: Optional[float] = None,
                               granularity: str = "device", size: int = 2):
  """Applies mixup to ``(images, labels)`` before ``train_step_fn``.

  ``granularity``: 'batch' / 'device' share one set of weights per process batch (each
  process drives one device), 'example' samples weights per example. Mixing partners are
  taken by rolling inside the local batch, so no cross-device traffic is needed. Uses the
  state's RNG stream named 'mixup'.
  """
  if concentration is None or concentration == 0.0:
    return train_step_fn
  if granularity not in ("batch", "device", "example"):
    raise ValueError(f"Unknown granularity: {granularity!r}")

  def new_train_step_fn(state, images, labels, *args, **kwargs):
    if not state.rngs or "mixup" not in state.rngs:
      raise ValueError('Mixup requires an RNG stream with the name "mixup", but only these '
                       f"were given: {sorted((state.rngs or {}).keys())}")
    imgs, labs = images.unsqueeze(0), labels.unsqueeze(0)
    shape = (1, imgs.shape[1], size) if granularity == "example" else (1, 1, size)
    imgs, labs = mixup(state.rngs["mixup"], (imgs, labs.float()), concentration=concentration,
                       shape=shape, roll_axis=1)
    return train_step_fn(state, imgs[0], labs[0], *args, **kwargs)

  return new_train_step_fn


# ------------------------------------------------------------------------------------ PGD training
def wrap_train_step_with_adversarial_attack(train_step_fn, loss_fn, *, max_epsilon: float,
                                            num_updates: int,
                                            attack_auxiliary_loss: bool = True):
  """Adversarial training: images are replaced by PGD adversarial examples (``num_updates``
  signed-gradient steps of size ``max_epsilon / num_updates``) before the normal step
  (reference: ``vmoe/train/trainer.py:841-886``)."""
  from vmoe_b200.projects.adversarial_attacks import attacks

  def new_train_step_fn(state, images, labels, *args, **kwargs):
    def loss_of(x):
      logits, metrics = state.model(x)
      loss = loss_fn(logits, labels).float().sum()
      if attack_auxiliary_loss:
        loss = loss + metrics["auxiliary_loss"].float().mean()
      return loss, None
    was = state.model.training
    adv = attacks.stateless_attack_pgd(images, loss_of, max_epsilon=max_epsilon,
                                       num_updates=num_updates,
                                       generator=(state.rngs or {}).get("adversarial"))
    state.model.train(was)
    return train_step_fn(state, adv.detach(), labels, *args, **kwargs)

  return new_train_step_fn


def check_device_status(state: TrainState) -> None:
  """Raises ``failure.DeviceWaitTimeout`` if a kernel of the peer-memory paths (expert exchange,
  gradient all-reduce) recorded a wait that ran out since the last check, and
  ``symm.BufferOverrun`` if the canary words around a peer-written region changed. Reading the status
  words synchronises with the device, so the training loop calls this only every
  ``check_device_status_every_steps`` steps."""
  from vmoe_b200.parallel import failure
  reducer = getattr(state.optimizer, "grad_reducer", None) if state.optimizer else None
  if reducer is not None:
    failure.check_status(reducer.status, "gradient all-reduce")
    reducer.buf.check_guards("gradient all-reduce buffer")
  try:
    from vmoe_b200.ops import moe_ops
  except Exception:  # pylint: disable=broad-except
    return
  for comm in getattr(moe_ops, "_LAYER_COMMS", {}).values():
    failure.check_status(comm.status, "expert exchange")
    comm.check_guards()


def create_checkpoint_manager(*, workdir: str, every_steps: Optional[int] = None,
                              keep_last: int = 1, keep_steps_multiple_of: Optional[int] = None,
                              wait_seconds: Optional[int] = 300, mesh=None,
                              **kwargs) -> "CheckpointManager":
  """Factory with the reference's name (``vmoe/train/trainer.py:134-165``)."""
  return CheckpointManager(workdir=workdir, every_steps=every_steps, keep_last=keep_last,
                           keep_steps_multiple_of=keep_steps_multiple_of,
                           wait_seconds=wait_seconds, mesh=mesh, **kwargs)


def restore_or_create_train_state(*, ckpt_manager: "CheckpointManager", model_config,
                                  optimizer_config, total_steps: int, mesh=None, device=None,
                                  seed: int = 0, extra_rng_keys=(), initialization=None,
                                  **model_overrides) -> TrainState:
  """Creates the train state, then restores the latest checkpoint of ``ckpt_manager`` into it if
  there is one; otherwise applies the optional fine-tuning ``initialization`` (kwargs of
  ``initialize_train_state_from_checkpoint``). Mirrors ``vmoe/train/trainer.py:371-438``."""
  state = create_train_state(model_config=model_config, optimizer_config=optimizer_config,
                             total_steps=total_steps, mesh=mesh, device=device, seed=seed,
                             extra_rng_keys=extra_rng_keys, **model_overrides)
  if ckpt_manager.restore(state) is None and initialization:
    initialize_train_state_from_checkpoint(state=state, mesh=mesh, **dict(initialization))
  return state


def accumulate_gradients_and_metrics(state: TrainState, images: Tensor, labels: Tensor,
                                     loss_fn, microsteps: Optional[int] = None):
  """Runs forward + backward over ``microsteps`` slices of the batch, leaving the summed
  gradients in the parameters' ``.grad`` buffers (not yet reduced over ranks, not yet divided
  by the number of slices: the optimizer does both); returns the averaged metrics
  (``vmoe/train/trainer.py:76-131``)."""
  state.model.train()
  state.optimizer.zero_grad()
  n = microsteps or 1
  if n > 1 and images.shape[0] % n:
    raise ValueError(f"batch {images.shape[0]} is not divisible by microsteps={n}")
  metrics = None
  for i in range(n):
    total, m = compute_loss_and_metrics(state, images if n == 1 else images[i::n],
                                        labels if n == 1 else labels[i::n], loss_fn)
    total.backward()
    m = _detach_tree(m)
    metrics = m if metrics is None else _tree_add(metrics, m)
  return _tree_scale(metrics, 1.0 / n) if n > 1 else metrics


def make_train_cost_fn(flops_per_device: Optional[float], seconds_per_device: Optional[float],
                       num_devices: int = 1) -> Callable[[int], Dict[str, float]]:
  """Returns ``fn(step) -> {'flops': ..., 'device_seconds': ...}``: the total training cost up
  to ``step`` over all devices (``vmoe/train/trainer.py:539-553`` of the reference)."""

  def fn(step: int) -> Dict[str, float]:
    out: Dict[str, float] = {}
    if flops_per_device is not None:
      out["flops"] = flops_per_device * step * num_devices
    if seconds_per_device is not None:
      out["device_seconds"] = seconds_per_device * step * num_devices
    return out

  return fn


def override_base_config(base, override):
  """Returns ``base`` updated (recursively) with the keys of ``override``."""
  from vmoe_b200.utils.config_dict import ConfigDict
  out = ConfigDict(base.to_dict() if hasattr(base, "to_dict") else dict(base), type_safe=False)
  if override:
    out.update(override.to_dict() if hasattr(override, "to_dict") else dict(override))
  return out


# ------------------------------------------------------------------------------------ checkpoints
class CheckpointReadError(RuntimeError):
  """A checkpoint that was asked for by step exists but cannot be read."""


class CheckpointManager:
  """Train-state checkpoints ``<workdir>/ckpt/ckpt_<step>.{index,data-*}`` in the sharded
  format, saved asynchronously every ``every_steps`` steps; keeps the last ``keep_last``
  steps plus those that are multiples of ``keep_steps_multiple_of`` (the reference drives
  Orbax with the same options, ``vmoe/train/trainer.py:134-165``)."""

  def __init__(self, *, workdir: str, every_steps: Optional[int] = None, keep_last: int = 1,
               keep_steps_multiple_of: Optional[int] = None, wait_seconds: Optional[int] = 300,
               mesh: Optional[mesh_lib.Mesh] = None, num_shards: Optional[int] = None):
    import os
    from vmoe_b200.checkpoints import base as ckpt_base
    self.dir = os.path.join(workdir, "ckpt")
    self.prefix = os.path.join(self.dir, "ckpt")
    self.every_steps = every_steps
    self.keep_last = keep_last
    self.keep_multiple = keep_steps_multiple_of
    self.wait_seconds = wait_seconds
    self.mesh = mesh or mesh_lib.get_mesh()
    self.num_shards = num_shards
    self._pending = None
    self._pending_step = None
    self._pool = ckpt_base.ThreadPool(8)
    if self.mesh.rank == 0:
      os.makedirs(self.dir, exist_ok=True)
    from vmoe_b200.parallel import multihost_utils
    multihost_utils.sync_devices("checkpoints:create_dir")

  def should_save(self, step: int) -> bool:
    return bool(self.every_steps) and step % self.every_steps == 0

  def all_steps(self):
    from vmoe_b200.checkpoints import base as ckpt_base
    return list(ckpt_base.iterate_complete_steps_for_prefix(self.prefix, suffixes=(".index", ".data")))

  def latest_step(self) -> Optional[int]:
    steps = self.all_steps()
    return max(steps) if steps else None

  def wait_until_finished(self):
    """Waits for the save in flight. Older checkpoints are deleted only now, once the new one
    is completely on disk on every rank: until then they are the only restorable state, and a
    write that fails (the exception propagates from here) must leave them in place."""
    if self._pending is not None:
      pending, step = self._pending, self._pending_step
      self._pending = self._pending_step = None
      pending.get(self.wait_seconds)
      from vmoe_b200.parallel import multihost_utils
      if multihost_utils.all_ranks_ok(True):
        self._cleanup(step)

  def save(self, step: int, state: TrainState, force: bool = False, last_seen_index=None) -> bool:
    if not (force or self.should_save(step)):
      return False
    from vmoe_b200.checkpoints import partitioned
    self.wait_until_finished()
    tree, specs = train_state_to_tree(state)
    tree["dataset_iterator"] = {"last_seen_index": np.asarray(-1 if last_seen_index is None
                                                              else last_seen_index)}
    specs["dataset_iterator"] = {"last_seen_index": None}
    self._pending = partitioned.save_checkpoint(
        f"{self.prefix}_{step}", tree, shardings=specs, mesh=self.mesh,
        num_shards=self.num_shards, thread_pool=self._pool)
    self._pending_step = step
    return True

  def _cleanup(self, current: int):
    if self.mesh.rank != 0:
      return
    import glob, os
    steps = sorted(set(self.all_steps()) - {current})
    keep = set(steps[-max(self.keep_last - 1, 0):]) if self.keep_last > 1 else set()
    for s in steps:
      if s in keep or (self.keep_multiple and s % self.keep_multiple == 0):
        continue
      for f in glob.glob(f"{glob.escape(self.prefix)}_{s}.*"):
        try:
          os.remove(f)
        except OSError:
          pass

  def close(self):
    self.wait_until_finished()
    self._pool.close()
    self._pool.join()

  def restore(self, state: TrainState, step: Optional[int] = None) -> Optional[int]:
    """Restores ``step`` (raises if it cannot be read) or, without ``step``, the newest
    checkpoint that every rank can read: a step whose files are truncated or corrupted is
    reported and skipped, and the one before it is tried, so that a job restarted after a
    crash in the middle of a save resumes from the last good step. Returns the restored step
    or None."""
    from vmoe_b200.checkpoints import partitioned
    from vmoe_b200.parallel import multihost_utils
    candidates = [step] if step is not None else sorted(self.all_steps(), reverse=True)
    _, specs = train_state_to_tree(state)
    specs["dataset_iterator"] = {"last_seen_index": None}
    for candidate in candidates:
      tree, error = None, None
      try:
        tree = partitioned.restore_checkpoint(f"{self.prefix}_{candidate}", shardings=specs,
                                              mesh=self.mesh, thread_pool=self._pool)
      except Exception as e:  # pylint: disable=broad-except
        error = e
      if multihost_utils.all_ranks_ok(error is None):
        load_train_state_from_tree(state, tree)
        return candidate
      if step is not None:
        raise CheckpointReadError(
            f"checkpoint {self.prefix}_{candidate} cannot be read"
            + (f": {type(error).__name__}: {error}" if error is not None
               else " on another rank")) from error
      logging.error("Skipping checkpoint step %d (%s); trying the previous one.", candidate,
                    f"{type(error).__name__}: {error}" if error is not None
                    else "unreadable on another rank")
    return None


import numpy as np  # noqa: E402  (used by the checkpoint helpers below)


def train_state_to_tree(state: TrainState):
  """``(tree, specs)`` in Flax layout: ``step / params / opt_state / rngs`` with local blocks
  of expert-sharded leaves and a matching tree of partition specs."""
  from vmoe_b200.checkpoints import flax_layout
  params, specs = flax_layout.to_flax(state.model)
  tree = {"step": np.asarray(state.step), "params": params}
  spec_tree = {"step": None, "params": specs}
  if state.optimizer is not None:
    opt = state.optimizer
    mu, nu = _moments_to_flax(state, opt)
    tree["opt_state"] = {"count": np.asarray(opt.step_count), "mu": mu,
                         "hyperparams": {"learning_rate": np.asarray(opt.last_learning_rate,
                                                                     dtype=np.float32)}}
    spec_tree["opt_state"] = {"count": None, "mu": specs, "hyperparams": {"learning_rate": None}}
    if nu is not None:
      tree["opt_state"]["nu"] = nu
      spec_tree["opt_state"]["nu"] = specs
    if opt.name == "big_vision_adafactor":
      af, af_specs = _adafactor_to_tree(opt)
      tree["opt_state"]["adafactor"] = af
      spec_tree["opt_state"]["adafactor"] = af_specs
  if state.rngs:
    tree["rngs"] = {k: g.get_state().numpy() for k, g in state.rngs.items()}
    spec_tree["rngs"] = {k: None for k in state.rngs}
  return tree, spec_tree


def _adafactor_to_tree(opt):
  """Second-moment accumulators of big_vision Adafactor (``v`` or the factored ``v_row`` /
  ``v_col``), keyed by the parameter's path, in this package's own array layout. Accumulators
  of expert-sharded parameters that keep the leading expert axis are saved as local blocks."""
  from vmoe_b200.utils.misc import unflatten_dict
  flat, specs = {}, {}
  for b in opt.buckets.values():
    for key, p in b.entries:
      for name, v in opt.af_state[id(p)].items():
        flat[f"{key}/{name}"] = v.detach().cpu().numpy().copy()
        keeps_expert_axis = v.dim() >= 1 and p.dim() >= 1 and v.shape[0] == p.shape[0] and (
            name == "v" or _adafactor_keeps_axis0(opt, p, name))
        specs[f"{key}/{name}"] = ("expert",) if (getattr(p, "expert_sharded", False) and
                                                 keeps_expert_axis) else None
  return unflatten_dict(flat, sep="/"), unflatten_dict(specs, sep="/")


def _adafactor_keeps_axis0(opt, p, name: str) -> bool:
  from vmoe_b200.train.optimizer import _factored_dims
  dims = _factored_dims(p.shape, opt.af["min_dim_size_to_factor"])
  if dims is None:
    return True
  d1, d0 = dims
  return (d0 if name == "v_row" else d1) != 0


def _moments_to_flax(state, opt):
  """Optimizer moments in the same Flax layout as the parameters they belong to."""
  from vmoe_b200.checkpoints import flax_layout
  out = []
  for which in ("mu", "nu"):
    if which == "nu" and opt.name != "adam":
      out.append(None)
      continue
    saved = {}
    for b in opt.buckets.values():
      flat = getattr(b, which)
      for i, (_, p) in enumerate(b.entries):
        saved[id(p)] = p.data
        p.data = b.view_of(flat, i)
    try:
      tree, _ = flax_layout.to_flax(state.model)
    finally:
      for b in opt.buckets.values():
        for _, p in b.entries:
          p.data = saved[id(p)]
    out.append(tree)
  return out


def load_train_state_from_tree(state: TrainState, tree) -> None:
  from vmoe_b200.checkpoints import flax_layout
  state.step = int(np.asarray(tree.get("step", 0)))
  flax_layout.from_flax(state.model, tree["params"], mesh=state.mesh)
  opt = state.optimizer
  if opt is not None and "opt_state" in tree:
    st = tree["opt_state"]
    opt.step_count = int(np.asarray(st.get("count", state.step)))
    for which in ("mu", "nu"):
      if which not in st or (which == "nu" and opt.name != "adam"):
        continue
      saved = {}
      for b in opt.buckets.values():
        flat = getattr(b, which)
        for i, (_, p) in enumerate(b.entries):
          saved[id(p)] = p.data
          p.data = b.view_of(flat, i)
      try:
        flax_layout.from_flax(state.model, st[which], mesh=state.mesh)
      finally:
        for b in opt.buckets.values():
          for _, p in b.entries:
            p.data = saved[id(p)]
    if opt.name == "big_vision_adafactor" and "adafactor" in st:
      from vmoe_b200.utils.misc import flatten_dict
      flat = flatten_dict(st["adafactor"], sep="/")
      for b in opt.buckets.values():
        for key, p in b.entries:
          for name, v in opt.af_state[id(p)].items():
            if f"{key}/{name}" in flat:
              src = torch.as_tensor(np.asarray(flat[f"{key}/{name}"]))
              if (src.shape != v.shape and getattr(p, "expert_sharded", False) and
                  state.mesh is not None and src.dim() >= 1 and v.dim() >= 1 and
                  src.shape[0] == v.shape[0] * state.mesh.num_partitions):
                el = v.shape[0]   # a full array: keep this rank's experts
                src = src[state.mesh.expert_rank * el:(state.mesh.expert_rank + 1) * el]
              v.copy_(src.to(device=v.device, dtype=v.dtype))
  if opt is not None:
    opt.sync_shadows()
  if state.rngs and "rngs" in tree:
    for k, v in tree["rngs"].items():
      if k in state.rngs:
        state.rngs[k].set_state(torch.as_tensor(np.asarray(v), dtype=torch.uint8))


# ------------------------------------------------------------------------------------ loop
def _image_size_from_spec(spec) -> Optional[int]:
  shape = spec.get("image", (None,))[0] if spec else None
  return int(shape[1]) if shape is not None and len(shape) == 4 else None


def create_evaluation_hook(*, base_model_config, writer, progress_hook, datasets, loss_fn,
                           label_pred_fn, first_step, train_steps, extra_rng_keys=(),
                           model_overrides=None, state=None, every_steps=None, every_secs=None,
                           on_steps=None, **kwargs):
  """Evaluation hook; ``model_overrides`` (e.g. a different capacity factor) build a second,
  deterministic model that shares the training model's parameters."""
  from vmoe_b200.evaluate import evaluator
  on_steps = set(on_steps or []) | {first_step, train_steps}
  model = state.model
  if model_overrides:
    cfg = override_base_config(base_model_config, model_overrides)
    model = models_lib.create_model(cfg, deterministic=True, mesh=state.mesh,
                                    image_size=getattr(state.model, "image_size", 224))
    model.to(next(state.model.parameters()).device)
    _share_parameters(state.model, model)
  datasets = {k: v for k, v in datasets.items() if k != "train"}
  return evaluator.EvaluateMultipleDatasets(
      model=model, datasets=datasets, loss_fn=loss_fn, label_pred_fn=label_pred_fn,
      metric_writer=writer, report_progress=progress_hook, every_steps=every_steps,
      every_secs=every_secs, on_steps=on_steps,
      input_dtype=None)


def _share_parameters(src: torch.nn.Module, dst: torch.nn.Module) -> None:
  src_params = dict(src.named_parameters())
  for name, p in dst.named_parameters():
    if name in src_params and src_params[name].shape == p.shape:
      p.data = src_params[name].data
      sp = src_params[name]
      if hasattr(sp, "_bf16_shadow"):
        p._bf16_shadow = sp._bf16_shadow
        p._shadow_version = p._version
    p.requires_grad_(False)


@contextlib.contextmanager
def _step_annotation(name: str, step: int):
  """NVTX range ``<name> <step>`` around a step (visible in Nsight / torch profiler traces); the
  counterpart of ``jax.profiler.StepTraceAnnotation`` (``vmoe/train/trainer.py:822``)."""
  on = torch.cuda.is_available()
  if on:
    torch.cuda.nvtx.range_push(f"{name} {step}")
  try:
    yield
  finally:
    if on:
      torch.cuda.nvtx.range_pop()


def create_progress_hook(*, writer, first_step, train_steps, **kwargs):
  from vmoe_b200.train import periodic_actions
  on_steps = set(kwargs.pop("on_steps", None) or []) | {first_step, train_steps}
  return periodic_actions.ReportProgress(num_train_steps=train_steps, writer=writer,
                                         on_steps=on_steps, **kwargs)


def create_profile_hook(*, workdir, **kwargs):
  from vmoe_b200.train import periodic_actions
  all_processes = kwargs.pop("all_processes", False)
  hook = periodic_actions.Profile(logdir=workdir, **kwargs)
  return hook if all_processes else periodic_actions.SingleProcessPeriodicAction(hook)


def initialize_train_state_from_checkpoint(*, state: TrainState, name: str, mesh=None,
                                           **kwargs) -> None:
  """Runs ``initialize_from_{vmoe,vit,orbax}`` on the Flax-layout view of ``state`` and loads
  the result back (``kwargs``: prefix/filepath/directory, rules, axis_resources_regexes,
  raise_if_* switches)."""
  from vmoe_b200 import initialization
  fns = {"initialize_from_vmoe": initialization.initialize_from_vmoe,
         "initialize_from_vit": initialization.initialize_from_vit,
         "initialize_from_orbax": initialization.initialize_from_orbax}
  if name not in fns:
    raise ValueError(f"Unknown initialization function: {name!r}")
  target, _ = train_state_to_tree(state)
  target.pop("rngs", None)
  new_tree = fns[name](target=target, mesh=mesh or state.mesh, **kwargs)
  load_train_state_from_tree(state, new_tree)


def train_and_evaluate(config, workdir: str, mesh: Optional[mesh_lib.Mesh] = None, writer=None):
  """Trains a model and evaluates it periodically (the ``main`` of ``vmoe_b200.app``)."""
  import time
  from vmoe_b200.data import input_pipeline, pjit_utils
  from vmoe_b200.parallel import multihost_utils
  from vmoe_b200.train.tree_summarizer import TreeSummarizer
  from vmoe_b200.utils import metric_writers
  mesh = mesh or mesh_lib.get_mesh()
  writer = writer or metric_writers.create_default_writer(workdir, just_logging=mesh.rank > 0)
  device = (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
            else torch.device("cpu"))
  datasets = input_pipeline.get_datasets(config.dataset)
  if "train" not in datasets:
    raise KeyError(f'You must have a "train" variant of the dataset. Available: {list(datasets)}')
  train_batch_size = config.dataset.train.batch_size
  train_steps, train_epochs = get_train_steps_and_epochs(
      train_steps=config.get("train_steps"), train_epochs=config.get("train_epochs"),
      train_batch_size=train_batch_size,
      train_examples=input_pipeline.get_data_num_examples(config.dataset.train))
  logging.info("Training for %d steps (%g epochs)", train_steps, train_epochs)
  spec = datasets["train"].peek_spec()
  image_size = _image_size_from_spec(spec) or 224

  opt_cfg = config.optimizer.to_dict() if hasattr(config.optimizer, "to_dict") else dict(config.optimizer)
  extra_rng_keys = tuple(config.get("extra_rng_keys", ()) or ())
  if config.get("mixup") and "mixup" not in extra_rng_keys:
    extra_rng_keys += ("mixup",)
  state = create_train_state(model_config=config.model, optimizer_config=opt_cfg,
                             total_steps=train_steps, mesh=mesh, device=device,
                             seed=config.get("seed", 0), extra_rng_keys=extra_rng_keys,
                             image_size=image_size)
  ckpt_cfg = dict(config.get("save_checkpoint", {}) or {})
  ckpt_manager = CheckpointManager(workdir=workdir, mesh=mesh, **ckpt_cfg)
  restored = ckpt_manager.restore(state)
  if restored is None and config.get("initialization"):
    init_cfg = config.initialization.to_dict() if hasattr(config.initialization, "to_dict") \
        else dict(config.initialization)
    initialize_train_state_from_checkpoint(state=state, mesh=mesh, **init_cfg)
  init_step = state.step
  logging.info("Initial step = %d", init_step)

  loss_cfg = dict(config.get("loss", {"name": "softmax_xent"}))
  train_loss_fn, eval_loss_fn, label_pred_fn = get_loss_fn(**loss_cfg)
  summarizer = None
  if config.get("summarize_arrays"):
    sa = dict(config.summarize_arrays)
    summarizer = TreeSummarizer(**sa)
  step_fn = train_step
  if config.get("adversarial"):
    step_fn = wrap_train_step_with_adversarial_attack(step_fn, train_loss_fn,
                                                      **dict(config.adversarial))
  if config.get("mixup"):
    mix = dict(config.mixup)
    mix.pop("partition_spec", None)
    step_fn = wrap_train_step_with_mixup(step_fn, **mix)
  microsteps = config.get("microsteps")

  progress_hook = create_progress_hook(writer=writer, first_step=init_step + 1,
                                       train_steps=train_steps,
                                       **dict(config.get("report_progress", {}) or {}))
  eval_cfg = dict(config.get("evaluate", {}) or {})
  eval_cfg.pop("seed", None)
  evaluation_hook = create_evaluation_hook(
      base_model_config=config.model, writer=writer, progress_hook=progress_hook,
      datasets=datasets, loss_fn=eval_loss_fn, label_pred_fn=label_pred_fn,
      first_step=init_step + 1, train_steps=train_steps, extra_rng_keys=extra_rng_keys,
      state=state, **eval_cfg)
  profile_hook = None
  if config.get("profile"):
    profile_hook = create_profile_hook(workdir=workdir, **dict(config.profile))
  fewshot_hook = None
  if config.get("fewshot"):
    from vmoe_b200.evaluate import fewshot as fewshot_lib
    fs = dict(config.fewshot)
    fs_model_cfg = override_base_config(config.model, {"num_classes": None})
    fs_model = models_lib.create_model(fs_model_cfg, deterministic=True, mesh=mesh,
                                       image_size=image_size).to(device)
    _share_parameters(state.model, fs_model)
    fewshot_hook = fewshot_lib.FewShotPeriodicAction(
        model=fs_model, metric_writer=writer, report_progress=progress_hook, **fs)

  dtype = getattr(state.model, "dtype", None)
  def batches():
    it = iter(datasets["train"])
    while True:
      yield next(it)
  # ``dataset.train.device_value_range = (vmin, vmax)``: the pipeline delivers uint8 images
  # (its ``process`` string leaves ``value_range`` out) and they are mapped to [vmin, vmax] on
  # the GPU after the copy; multi-hot / one-hot labels may arrive as uint8 as well.
  transforms, dtypes = None, None
  dvr = config.dataset.train.get("device_value_range")
  if dvr:
    transforms = {"image": pjit_utils.value_range_on_device(float(dvr[0]), float(dvr[1]))}
    dtypes = {"labels": torch.float32}
  tr_iter = pjit_utils.prefetch_to_device(
      batches(), size=int(config.dataset.train.get("prefetch_device", 2) or 2), device=device,
      dtypes=dtypes, transforms=transforms)

  status_every = int(config.get("check_device_status_every_steps", 100) or 100)
  # Optional host-side failure detection (``config.heartbeat = {every_steps, timeout_seconds}``).
  heartbeat = None
  hb_cfg = config.get("heartbeat")
  if hb_cfg and mesh.world_size > 1:
    from vmoe_b200.parallel import failure
    heartbeat = failure.Heartbeat()
    heartbeat_every = int(hb_cfg.get("every_steps", 1) or 1)
    heartbeat_timeout = float(hb_cfg.get("timeout_seconds", 60.0))
  multihost_utils.sync_devices("training:start")
  if init_step == 0 and ckpt_cfg.get("every_steps"):
    ckpt_manager.save(0, state, force=True)
  t_start = time.time()
  metrics = {}
  train_cost_fn = None
  for step in range(init_step + 1, train_steps + 1):
    batch = next(tr_iter)
    if train_cost_fn is None:
      try:
        flops, secs = misc.get_flops_and_seconds_per_device(state.model, batch["image"])
      except Exception as e:  # pylint: disable=broad-except
        logging.warning("Could not estimate the cost of a training step: %r", e)
        flops = secs = None
      train_cost_fn = make_train_cost_fn(flops, secs, mesh.world_size)
      costs = {k: v for k, v in (("train/step_flops_per_device", flops),
                                 ("train/step_seconds_per_device", secs)) if v is not None}
      if costs:
        writer.write_scalars(step, costs)
    if profile_hook is not None:
      profile_hook(step)
    with _step_annotation("train", step):
      _, metrics = step_fn(state, batch["image"], batch["labels"], train_loss_fn,
                           microsteps=microsteps, summarizer=summarizer)
    progress_hook(step, scalar_metrics={**train_cost_fn(step),
                                        "train": {k: v for k, v in metrics.items()
                                                  if not isinstance(v, Mapping)}})
    if heartbeat is not None:
      # Every rank publishes the step it reached; a rank that stopped or left is named here, on
      # the host, before this rank launches kernels that would wait for it.
      heartbeat.beat(step)
      if step % heartbeat_every == 0:
        heartbeat.check(step, timeout_s=heartbeat_timeout)
    if step % status_every == 0 or ckpt_manager.should_save(step):
      # Also before every save: a bounded wait that ran out means this step applied gradients
      # or expert rows that were incomplete, and such a state must not become a restore point.
      check_device_status(state)
    with progress_hook.timed("ckpt", wait_jax_async_dispatch=False):
      ckpt_manager.save(step, state)
    evaluation_hook(step)
    if fewshot_hook is not None:
      fewshot_hook(step)
  ckpt_manager.wait_until_finished()
  if ckpt_cfg.get("every_steps") and train_steps > init_step and ckpt_manager.latest_step() != train_steps:
    check_device_status(state)
    ckpt_manager.save(train_steps, state, force=True)
    ckpt_manager.wait_until_finished()
  ckpt_manager.close()
  multihost_utils.sync_devices("training:completed")
  logging.info("Training completed in %.1f s.", time.time() - t_start)
  writer.flush()
  return state, metrics
