"""Runs a PGD attack over a whole dataset against a restored V-MoE / ViT model.

Counterpart of ``vmoe/projects/adversarial_attacks/lib.py:44-235``: restores the model from a
sharded checkpoint, attacks every batch, accumulates the statistics of ``attacks.AttackState``
(error and loss before/after, prediction changes, per-router routing changes), optionally
stores the processed examples of each process in a compressed ``.npz`` file, and writes
``pgd_state.npz`` plus the summary scalars.
"""
from __future__ import annotations

import collections
import io
import logging
import math
import os
from typing import Any, Mapping, Optional

import numpy as np
import torch
import torch.distributed as dist

from vmoe_b200.data import input_pipeline
from vmoe_b200.data import pjit_utils
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.projects.adversarial_attacks import attacks
from vmoe_b200.projects.adversarial_attacks import restore
from vmoe_b200.train import periodic_actions

VALID_KEY = input_pipeline.VALID_KEY


def savez_compressed(filepath: str, **data) -> None:
  """``np.savez_compressed`` through an in-memory buffer (works on non-seekable targets)."""
  outdir = os.path.dirname(filepath)
  if outdir:
    os.makedirs(outdir, exist_ok=True)
  buffer = io.BytesIO()
  np.savez_compressed(buffer, **data)
  with open(filepath, "wb") as fp:
    fp.write(buffer.getvalue())


def _to_numpy(v):
  if isinstance(v, torch.Tensor):
    return v.detach().float().cpu().numpy() if v.dtype == torch.bfloat16 else v.detach().cpu().numpy()
  return np.asarray(v)


class ExampleStorage:
  """Keeps the arrays given to ``store`` and writes them, concatenated over steps, to one
  ``.npz`` file. Device tensors are moved to the host every ``transfer_every_steps`` steps."""

  def __init__(self, filepath: str, transfer_every_steps: int = 1):
    self._filepath = filepath
    self._transfer_every_steps = transfer_every_steps
    self._data = collections.defaultdict(list)
    self._temp = collections.defaultdict(list)

  def _transfer(self):
    for key, values in self._temp.items():
      self._data[key].extend(_to_numpy(v) for v in values)
      self._temp[key] = []

  @property
  def filepath(self) -> str:
    return self._filepath

  def store(self, step: int, **arrays):
    for key, value in arrays.items():
      self._temp[key].append(value)
    if step % self._transfer_every_steps == 0:
      self._transfer()

  def write(self):
    self._transfer()
    if self._data:
      savez_compressed(self._filepath, **{
          key: np.concatenate(values, axis=0) for key, values in self._data.items()})


def get_dataset(config: Mapping[str, Any]) -> input_pipeline.DatasetIterator:
  kwargs = dict(config.to_dict() if hasattr(config, "to_dict") else config)
  kwargs.pop("prefetch_device", None)
  # The variant name only matters in that it is not "train".
  return input_pipeline.get_dataset(variant="adversarial", **kwargs)


def _process_index_count():
  if dist.is_available() and dist.is_initialized():
    return dist.get_rank(), dist.get_world_size()
  return 0, 1


def _allreduce_state(state: attacks.AttackState) -> attacks.AttackState:
  """Sums the statistics over processes (each one attacked its own slice of the data)."""
  if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
    return state
  for t in [state.num_images, state.num_changes, state.num_correct, state.sum_loss,
            *state.sum_iou_experts.values()]:
    dist.all_reduce(t)
  return state


def run_pgd_attack(config, workdir: str, mesh: Optional[mesh_lib.Mesh] = None, writer=None):
  """Runs PGD on an entire dataset, using a model restored from a checkpoint
  (``lib.py:98-235`` of the reference project)."""
  del mesh
  dataset = get_dataset(config.dataset)
  spec = dataset.peek_spec()
  image_shape = (config.dataset.batch_size,) + tuple(spec["image"][0][1:])
  num_examples = input_pipeline.get_data_num_examples(config.dataset)
  num_steps = int(math.ceil(num_examples / config.dataset.batch_size))
  report_progress = periodic_actions.ReportProgress(
      num_train_steps=num_steps, writer=writer, on_steps=[], every_secs=60.0)
  if config.restore.get("from") != "checkpoint":
    raise ValueError(f"config.restore.from = {config.restore.get('from')!r} is not supported.")
  mesh = restore.create_mesh(config.get("num_expert_partitions", 1))
  mesh_lib.set_mesh(mesh)
  device = (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
            else torch.device("cpu"))
  model, loss_fn, router_keys, _ = restore.restore_from_config(
      config, config.restore.prefix, image_shape, mesh, device=device)
  process_index, process_count = _process_index_count()
  example_storage = None
  if config.get("store_examples"):
    kwargs = dict(config.store_examples.to_dict())
    prefix = kwargs.pop("prefix", os.path.join(workdir, "examples"))
    example_storage = ExampleStorage(
        filepath=f"{prefix}-{process_index:03d}-of-{process_count:03d}", **kwargs)
  dataset_iter = pjit_utils.prefetch_to_device(
      dataset, size=config.dataset.get("prefetch_device") or 1, device=device)
  state = attacks.AttackState.create(max_updates=config.num_updates, router_keys=router_keys,
                                     device=device)

  def loss_of(images, labels):
    logits, metrics = model(images)
    return loss_fn(logits, labels, metrics).sum(), None

  def stateless_attack_fn(images, labels):
    return attacks.stateless_attack_pgd(
        images, lambda x: loss_of(x, labels), max_epsilon=config.max_epsilon,
        num_updates=config.num_updates)

  def compute_fn(images, labels):
    return restore.compute_loss_predict_cw_fn(images, labels, model=model, loss_fn=loss_fn)

  for step, batch in enumerate(dataset_iter, 1):
    report_progress(step)
    x_0, y = batch["image"].float(), batch["labels"]
    valid = batch.get(VALID_KEY)
    state, x_m, l_0, l_m, y_0, y_m, cw_0, cw_m = attacks.stateful_attack(
        state, x_0, y, valid, stateless_attack_fn=stateless_attack_fn,
        compute_loss_predict_correct_cw_fn=compute_fn)
    if example_storage:
      extra = {} if valid is None else {"valid": valid}
      example_storage.store(
          step=step, x_0=x_0, y_0=y_0, l_0=l_0, x_m=x_m, y_m=y_m, l_m=l_m, y=y, **extra,
          **{f"cw_0/{k}": v for k, v in cw_0.items()},
          **{f"cw_m/{k}": v for k, v in cw_m.items()})
  state = _allreduce_state(state)
  num_images = max(int(state.num_images), 1)
  num_correct = _to_numpy(state.num_correct)
  sum_loss = _to_numpy(state.sum_loss)
  sum_iou = {k: float(v) for k, v in state.sum_iou_experts.items()}
  if process_index == 0:
    state_filepath = os.path.join(workdir, "pgd_state.npz")
    logging.info("Saving PGDState to %r...", state_filepath)
    savez_compressed(state_filepath, num_images=_to_numpy(state.num_images),
                     num_changes=_to_numpy(state.num_changes), num_correct=num_correct,
                     sum_loss=sum_loss,
                     **{f"sum_iou_experts/{k}": np.asarray(v) for k, v in sum_iou.items()})
  if writer is not None:
    writer.write_scalars(0, {"error": 1 - num_correct[0] / num_images,
                             "loss": sum_loss[0] / num_images})
    writer.write_scalars(config.num_updates, {
        "error": 1 - num_correct[1] / num_images,
        "loss": sum_loss[1] / num_images,
        "prediction_changes": int(state.num_changes) / num_images,
        **{f"routing_changes/{k}": 1 - v / num_images for k, v in sum_iou.items()}})
  if example_storage:
    logging.info("Saving examples to %r...", example_storage.filepath)
    example_storage.write()
  return state
