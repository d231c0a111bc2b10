"""End-to-end training loop on CPU: train, evaluate, checkpoint, resume, mixup, microsteps."""
import os

import torch

from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.train import trainer
from vmoe_b200.utils.config_dict import ConfigDict


class _Writer:
  def __init__(self):
    self.scalars = {}

  def write_scalars(self, step, scalars):
    self.scalars.setdefault(step, {}).update(scalars)

  def write_hparams(self, hparams):
    pass

  def write_texts(self, step, texts):
    pass

  def flush(self):
    pass


def _config(train_steps, **extra):
  config = common.get_base_config()
  pp = 'value_range(-1,1)|onehot(5, inkey="label", outkey="labels")|keep("image", "labels")'
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = ConfigDict(dict(
      name="synthetic", split="train", batch_size=8, image_size=16, num_classes=5,
      num_train_examples=64, process=pp, shuffle_buffer=16), type_safe=False)
  config.dataset.val = ConfigDict(dict(
      name="synthetic", split="validation", batch_size=8, image_size=16, num_classes=5,
      num_eval_examples=12, process=pp), type_safe=False)
  config.train_steps = train_steps
  config.loss = ConfigDict({"name": "softmax_xent"})
  config.optimizer = ConfigDict({"name": "sgd", "momentum": 0.9, "learning_rate": 0.01},
                                type_safe=False)
  config.model = ConfigDict({
      "name": "VisionTransformerMoe", "num_classes": 5, "patch_size": (8, 8), "hidden_size": 16,
      "classifier": "token", "representation_size": None,
      "encoder": {"num_layers": 2, "num_heads": 2, "mlp_dim": 32, "dropout_rate": 0.0,
                  "attention_dropout_rate": 0.0,
                  "moe": {"num_experts": 2, "layers": (1,), "group_size": 10,
                          "router": {"num_selected_experts": 1, "noise_std": 1.0,
                                     "importance_loss_weight": 0.01, "load_loss_weight": 0.01,
                                     "dispatcher": {"name": "einsum", "capacity_factor": 2.0,
                                                    "batch_priority": False}}}}},
      type_safe=False)
  config.save_checkpoint.every_steps = 2
  config.report_progress.every_steps = 1
  config.evaluate.every_steps = 2
  config.extra_rng_keys = ("dropout", "gating")
  for k, v in extra.items():
    setattr(config, k, v)
  return config


def test_train_evaluate_checkpoint_and_resume(tmp_path):
  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  writer = _Writer()
  state, metrics = trainer.train_and_evaluate(_config(4), str(tmp_path), mesh=mesh, writer=writer)
  assert state.step == 4 and torch.isfinite(torch.as_tensor(metrics["total_loss"]))
  assert any("val/loss" in s or any(k.startswith("val") for k in s) for s in writer.scalars.values())
  files = os.listdir(os.path.join(str(tmp_path), "ckpt"))
  assert any(f.startswith("ckpt_4.index") for f in files), files
  # A second run with more steps resumes from step 4 instead of starting over.
  writer2 = _Writer()
  state2, _ = trainer.train_and_evaluate(_config(6), str(tmp_path), mesh=mesh, writer=writer2)
  assert state2.step == 6
  assert min(writer2.scalars) >= 5


def test_microsteps_and_mixup_run(tmp_path):
  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  config = _config(2, microsteps=2,
                   mixup=ConfigDict({"concentration": 0.2, "granularity": "example", "size": 2},
                                    type_safe=False))
  config.extra_rng_keys = ("dropout", "gating", "mixup")
  state, metrics = trainer.train_and_evaluate(config, str(tmp_path), mesh=mesh, writer=_Writer())
  assert state.step == 2 and torch.isfinite(torch.as_tensor(metrics["total_loss"]))


def test_device_value_range_option(tmp_path):
  """``dataset.train.device_value_range``: the pipeline leaves the images uint8 (no
  ``value_range`` in its process string) and the prefetcher maps them behind the copy."""
  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  config = _config(2)
  pp = 'onehot(5, inkey="label", outkey="labels")|keep("image", "labels")'
  config.dataset.train.process = pp
  config.dataset.train.device_value_range = (-1.0, 1.0)
  seen = {}
  orig = trainer.train_step

  def spy(state, images, labels, *a, **k):
    seen["dtype"], seen["min"], seen["max"] = images.dtype, float(images.min()), float(images.max())
    return orig(state, images, labels, *a, **k)

  trainer.train_step = spy
  try:
    state, metrics = trainer.train_and_evaluate(config, str(tmp_path), mesh=mesh, writer=_Writer())
  finally:
    trainer.train_step = orig
  assert state.step == 2 and torch.isfinite(torch.as_tensor(metrics["total_loss"]))
  assert seen["dtype"] == torch.float32 and -1.0 - 1e-6 <= seen["min"] < seen["max"] <= 1.0 + 1e-6
