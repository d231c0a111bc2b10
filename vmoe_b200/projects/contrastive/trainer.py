"""Contrastive training: the sigmoid (SigLIP) loss and the two-tower train step / loop.

``sigmoid_loss(logits)``: ``-sum_n log sigmoid(z_mn * logits_mn)`` with ``z = 2 I - 1``, one
value per image. As in the reference, where the step is jitted over the global batch
(``vmoe/projects/contrastive/trainer.py:214-264``), every image is contrasted with the texts of
the WHOLE global batch: each rank all-gathers the text embeddings (an autograd-aware
collective whose backward sums the gradients that all ranks computed for a rank's texts) and
evaluates its rows of the global logits matrix, one source rank's block of columns at a time.
"""
from __future__ import annotations

from typing import Callable, Mapping, Optional

import torch
import torch.distributed as dist
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


class _AllGatherRows(torch.autograd.Function):
  """``(n, d)`` on every rank -> ``(world, n, d)``. Backward: the sum over ranks of the
  gradients for this rank's block (every rank used every block)."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    world = dist.get_world_size(group)
    out = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(out, x.contiguous(), group=group)
    return torch.stack(out, 0)

  @staticmethod
  def backward(ctx, grad):
    grad = grad.contiguous()
    dist.all_reduce(grad, group=ctx.group)
    return grad[dist.get_rank(ctx.group)], None


def global_sigmoid_loss(zimg: torch.Tensor, ztxt: torch.Tensor, scale: torch.Tensor,
                        bias: Optional[torch.Tensor], group=None) -> torch.Tensor:
  """Per-image SigLIP loss of this rank's images against the texts of all ranks (``(n,)``).

  ``zimg``, ``ztxt``: this rank's normalised embeddings ``(n, d)``; the global batch is the
  concatenation over ranks, so the positive of local image ``i`` is text ``i`` of this rank.
  One ``(n, n)`` block of logits is alive at a time."""
  if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
    logits = zimg @ ztxt.t() * scale
    return sigmoid_loss(logits if bias is None else logits + bias)
  rank = dist.get_rank(group)
  blocks = _AllGatherRows.apply(ztxt, group)           # (world, n, d)
  n = zimg.shape[0]
  eye = torch.eye(n, dtype=zimg.dtype, device=zimg.device)
  loss = zimg.new_zeros(n)
  for src in range(blocks.shape[0]):
    logits = zimg @ blocks[src].t() * scale
    if bias is not None:
      logits = logits + bias
    z = (2.0 * eye - 1.0) if src == rank else -torch.ones_like(eye)
    loss = loss - F.logsigmoid(logits * z).sum(dim=-1)
  return loss


def train_step(state: TrainState, images, texts, loss_fn: Callable[[torch.Tensor], torch.Tensor],
               microsteps: Optional[int] = None, summarizer=None):
  """One update. With several ranks and ``loss_fn is sigmoid_loss`` the loss is taken over the
  global batch (``global_sigmoid_loss``); any other ``loss_fn`` sees the rank's own logits."""
  state.model.train()
  state.optimizer.zero_grad()
  n = microsteps or 1
  mesh = state.mesh or mesh_lib.get_mesh()
  use_global = (loss_fn is sigmoid_loss and mesh is not None and mesh.world_size > 1 and
                dist.is_available() and dist.is_initialized())
  metrics = None
  for i in range(n):
    im = images if n == 1 else images[i::n]
    tx = texts if n == 1 else texts[i::n]
    if use_global:
      zimg, ztxt, scale, bias, m = state.model.embed_pair(im, tx)
      per_image = global_sigmoid_loss(zimg, ztxt, scale, bias, mesh.world_group)
    else:
      logits, m = state.model(im, tx)
      per_image = loss_fn(logits)
    m = dict(m)
    m["main_loss"] = per_image.float().mean()
    m = base_trainer._mean_metrics(m)
    # Auxiliary losses live under 'img' / 'txt'; only a top-level entry is added to the loss.
    total = m["main_loss"] + m.get("auxiliary_loss", 0.0)
    m["total_loss"] = total
    reducer = getattr(state.optimizer, "grad_reducer", None)
    if reducer is not None and i == n - 1:
      reducer.begin()
    total.backward()
    m = base_trainer._detach_tree(m)
    metrics = m if metrics is None else base_trainer._tree_add(metrics, m)
  if n > 1:
    metrics = base_trainer._tree_scale(metrics, 1.0 / n)
  grads_for_summary = None
  if summarizer is not None:
    grads_for_summary = {key: p.grad.detach().clone() / n for key, _, p in
                         naming.named_flax_parameters(state.model, prefix="")
                         if p.grad is not None}
  flat_metrics = misc.flatten_dict(metrics, sep="\x00")
  keys = [k for k, v in flat_metrics.items() if isinstance(v, torch.Tensor) and v.dim() == 0
          and v.is_floating_point()]
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
  # Restore the latest checkpoint of this run or, failing that, initialise from another
  # checkpoint (``vmoe/projects/contrastive/trainer.py:299-311``).
  if ckpt.restore(state) is None and config.get("initialization"):
    init_cfg = config.initialization.to_dict() if hasattr(config.initialization, "to_dict") \
        else dict(config.initialization)
    base_trainer.initialize_train_state_from_checkpoint(state=state, mesh=mesh, **init_cfg)
  init_step = state.step
  summarizer = None
  if config.get("summarize_arrays"):
    from vmoe_b200.train.tree_summarizer import TreeSummarizer
    summarizer = TreeSummarizer(**dict(config.summarize_arrays))
  progress = base_trainer.create_progress_hook(
      writer=writer, first_step=init_step + 1, train_steps=train_steps,
      **dict(config.get("report_progress", {}) or {}))
  profile_hook = None
  if config.get("profile"):
    profile_hook = base_trainer.create_profile_hook(workdir=workdir, **dict(config.profile))
  fewshot_hook = create_fewshot_hook(state=state, writer=writer, progress_hook=progress,
                                     first_step=init_step + 1, train_steps=train_steps,
                                     **dict(config.get("fewshot", {}) or {}))
  hooks = []
  for name in ("retrieval", "zeroshot"):
    if config.get(name):
      from vmoe_b200.projects.contrastive import evaluators
      hooks.append(evaluators.make_hook(name, state=state, writer=writer, progress=progress,
                                        first_step=init_step + 1, train_steps=train_steps,
                                        **dict(config[name])))
  def batches():
    it = iter(datasets["train"])
    while True:
      yield next(it)
  it = pjit_utils.prefetch_to_device(batches(), size=2, device=device)
  metrics = {}
  for step in range(init_step + 1, train_steps + 1):
    batch = next(it)
    if profile_hook is not None:
      profile_hook(step)
    _, metrics = train_step(state, batch["image"], batch["text"], sigmoid_loss,
                            microsteps=config.get("microsteps"), summarizer=summarizer)
    progress(step, scalar_metrics={"train": {k: v for k, v in metrics.items()
                                             if not isinstance(v, Mapping)}})
    ckpt.save(step, state)
    if fewshot_hook is not None:
      fewshot_hook(step)
    for h in hooks:
      h(step)
  ckpt.close()
  writer.flush()
  return state, metrics


class _ImageFeatures(torch.nn.Module):
  """The image tower as a feature extractor for the few-shot evaluator: ``model(images)`` ->
  (normalised image embeddings, metrics), sharing the two-tower model's parameters."""

  def __init__(self, two_tower):
    super().__init__()
    self.two_tower = two_tower

  def forward(self, images):
    return self.two_tower(images, None)


def create_fewshot_hook(*, state: TrainState, writer, progress_hook, first_step: int,
                        train_steps: int, **kwargs):
  """Few-shot evaluation of the image tower every so often; no keyword arguments = no hook
  (``vmoe/projects/contrastive/trainer.py:67-99``)."""
  if not kwargs:
    return None
  from vmoe_b200.evaluate import fewshot as fewshot_lib
  on_steps = set(kwargs.pop("on_steps", None) or []) | {first_step, train_steps}
  return fewshot_lib.FewShotPeriodicAction(
      model=_ImageFeatures(state.model), metric_writer=writer, report_progress=progress_hook,
      report_progress_name="fewshot", on_steps=sorted(on_steps), **kwargs)
