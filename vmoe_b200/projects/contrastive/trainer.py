"""Contrastive training: the sigmoid (SigLIP) loss and the two-tower train step / loop.

``sigmoid_loss(logits)``: ``-sum_n log sigmoid(z_mn * logits_mn)`` with ``z = 2 I - 1``, one
value per image. Every rank contrasts its local images with its local texts (reference:
``vmoe/projects/contrastive/trainer.py:214-357``).
"""
from __future__ import annotations

from typing import Callable, Mapping, Optional

import torch
import torch.nn.functional as F

from vmoe_b200.models import naming
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.train import optimizer as optimizer_lib
from vmoe_b200.train import trainer as base_trainer
from vmoe_b200.train.train_state import TrainState
from vmoe_b200.utils import misc


def sigmoid_loss(logits: torch.Tensor) -> torch.Tensor:
  if logits.dim() < 2 or logits.shape[-1] != logits.shape[-2]:
    raise ValueError(f"Last two dims of logits must be equal, but got logits.shape={tuple(logits.shape)}")
  n = logits.shape[-1]
  z = 2.0 * torch.eye(n, dtype=logits.dtype, device=logits.device) - 1.0
  return -F.logsigmoid(logits * z).sum(dim=-1)


def train_step(state: TrainState, images, texts, loss_fn: Callable[[torch.Tensor], torch.Tensor],
               microsteps: Optional[int] = None, summarizer=None):
  state.model.train()
  state.optimizer.zero_grad()
  n = microsteps or 1
  metrics = None
  for i in range(n):
    im = images if n == 1 else images[i::n]
    tx = texts if n == 1 else texts[i::n]
    logits, m = state.model(im, tx)
    m = dict(m)
    m["main_loss"] = loss_fn(logits).float().mean()
    m = base_trainer._mean_metrics(m)
    # Auxiliary losses live under 'img' / 'txt'; only a top-level entry is added to the loss.
    total = m["main_loss"] + m.get("auxiliary_loss", 0.0)
    m["total_loss"] = total
    total.backward()
    m = base_trainer._detach_tree(m)
    metrics = m if metrics is None else base_trainer._tree_add(metrics, m)
  if n > 1:
    metrics = base_trainer._tree_scale(metrics, 1.0 / n)
  norms = state.apply_gradients_and_compute_global_norms(microsteps=n)
  metrics.update({f"global_norm/{k}": v for k, v in norms.items()})
  if summarizer is not None:
    flat = misc.flatten_dict(state.state_dict(), sep="/")
    metrics.update(summarizer(flat))
  return state, metrics


def create_train_state(*, model_config, optimizer_config, total_steps: int, mesh=None,
                       device=None, seed: int = 0, **model_overrides) -> TrainState:
  from vmoe_b200.projects.contrastive import models
  mesh = mesh or mesh_lib.get_mesh()
  torch.manual_seed(seed)
  cfg = model_config.to_dict() if hasattr(model_config, "to_dict") else dict(model_config)
  cfg.pop("name", None)
  model = models.TwoTower(mesh=mesh, **cfg, **model_overrides)
  if device is not None:
    model.to(device)
  opt_kwargs = dict(optimizer_config.to_dict() if hasattr(optimizer_config, "to_dict")
                    else optimizer_config)
  named = [(key, p) for key, _, p in naming.named_flax_parameters(model, prefix="params")]
  opt = optimizer_lib.create_optimizer(named, total_steps=total_steps, mesh=mesh, **opt_kwargs)
  return TrainState(model=model, optimizer=opt, step=0, rngs=misc.make_rngs(("dropout", "gating"), seed),
                    mesh=mesh)


def train_and_evaluate(config, workdir: str, mesh=None, writer=None):
  """Contrastive training loop; batches need ``image`` and ``text`` entries."""
  import time
  from vmoe_b200.data import input_pipeline, pjit_utils
  from vmoe_b200.utils import metric_writers
  mesh = mesh or mesh_lib.get_mesh()
  writer = writer or metric_writers.create_default_writer(workdir, just_logging=mesh.rank > 0)
  device = (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
            else torch.device("cpu"))
  datasets = input_pipeline.get_datasets(config.dataset)
  train_steps, _ = base_trainer.get_train_steps_and_epochs(
      train_steps=config.get("train_steps"), train_epochs=config.get("train_epochs"),
      train_batch_size=config.dataset.train.batch_size,
      train_examples=input_pipeline.get_data_num_examples(config.dataset.train))
  spec = datasets["train"].peek_spec()
  state = create_train_state(model_config=config.model, optimizer_config=config.optimizer,
                             total_steps=train_steps, mesh=mesh, device=device,
                             seed=config.get("seed", 0),
                             image_size=base_trainer._image_size_from_spec(spec) or 224)
  ckpt = base_trainer.CheckpointManager(workdir=workdir, mesh=mesh,
                                        **dict(config.get("save_checkpoint", {}) or {}))
  ckpt.restore(state)
  progress = base_trainer.create_progress_hook(
      writer=writer, first_step=state.step + 1, train_steps=train_steps,
      **dict(config.get("report_progress", {}) or {}))
  hooks = []
  for name in ("retrieval", "zeroshot"):
    if config.get(name):
      from vmoe_b200.projects.contrastive import evaluators
      hooks.append(evaluators.make_hook(name, state=state, writer=writer, progress=progress,
                                        first_step=state.step + 1, train_steps=train_steps,
                                        **dict(config[name])))
  def batches():
    it = iter(datasets["train"])
    while True:
      yield next(it)
  it = pjit_utils.prefetch_to_device(batches(), size=2, device=device)
  metrics = {}
  for step in range(state.step + 1, train_steps + 1):
    batch = next(it)
    _, metrics = train_step(state, batch["image"], batch["text"], sigmoid_loss,
                            microsteps=config.get("microsteps"))
    progress(step, scalar_metrics={"train": {k: v for k, v in metrics.items()
                                             if not isinstance(v, Mapping)}})
    ckpt.save(step, state)
    for h in hooks:
      h(step)
  ckpt.close()
  writer.flush()
  return state, metrics
