"""The training loop on a GPU with the CUDA kernels: train, evaluate, checkpoint, resume and
mixup / micro-steps on a small V-MoE (the CPU counterpart is ``tests/test_trainer_e2e.py``)."""
import os

import pytest
import torch

from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.train import trainer
from vmoe_b200.utils.config_dict import ConfigDict

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
  pytest.skip("needs a GPU", allow_module_level=True)


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


def _config(train_steps, optimizer="adam", **extra):
  config = common.get_base_config()
  pp = 'value_range(-1,1)|onehot(10, inkey="label", outkey="labels")|keep("image", "labels")'
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = ConfigDict(dict(
      name="synthetic", split="train", batch_size=16, image_size=64, num_classes=10,
      num_train_examples=256, process=pp, shuffle_buffer=32), type_safe=False)
  config.dataset.val = ConfigDict(dict(
      name="synthetic", split="validation", batch_size=16, image_size=64, num_classes=10,
      num_eval_examples=40, process=pp), type_safe=False)
  config.train_steps = train_steps
  config.loss = ConfigDict({"name": "softmax_xent"})
  opt = {"name": optimizer, "learning_rate": 1e-3}
  if optimizer == "adam":
    opt["weight_decay"] = 0.1
  config.optimizer = ConfigDict(opt, type_safe=False)
  # ViT-S/32 with 8 experts in the last two odd blocks; 64-pixel images give 4 patches + class
  # token, groups of 8 images.
  model = common.get_vmoe_config("ViT-S/32, E=8, K=2, Last 2", 64, 10)
  model.encoder.dtype = "bfloat16"
  model.encoder.moe.router.dispatcher.batch_priority = True
  config.model = model
  config.save_checkpoint.every_steps = 3
  config.report_progress.every_steps = 1
  config.evaluate.every_steps = 3
  config.extra_rng_keys = ("dropout", "gating")
  for k, v in extra.items():
    setattr(config, k, v)
  return config


@pytest.mark.parametrize("optimizer", ["adam", "big_vision_adafactor"])
def test_train_evaluate_checkpoint_and_resume_on_the_kernels(tmp_path, optimizer):
  from vmoe_b200.ops import _lib
  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  writer = _Writer()
  _lib.reset_launch_count()
  state, metrics = trainer.train_and_evaluate(_config(6, optimizer), str(tmp_path), mesh=mesh,
                                              writer=writer)
  assert _lib.reset_launch_count() > 100, "the CUDA kernels did not run"
  assert state.step == 6 and torch.isfinite(torch.as_tensor(metrics["total_loss"]))
  assert any(any(k.startswith("val") for k in s) for s in writer.scalars.values())
  files = os.listdir(os.path.join(str(tmp_path), "ckpt"))
  assert any(f.startswith("ckpt_6.index") for f in files), files
  # A second run with more steps resumes from step 6 instead of starting over.
  writer2 = _Writer()
  state2, metrics2 = trainer.train_and_evaluate(_config(8, optimizer), str(tmp_path), mesh=mesh,
                                                writer=writer2)
  assert state2.step == 8 and min(writer2.scalars) >= 7
  assert torch.isfinite(torch.as_tensor(metrics2["total_loss"]))


def test_microsteps_and_mixup_on_the_kernels(tmp_path):
  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  config = _config(3, microsteps=2,
                   mixup=ConfigDict({"concentration": 0.2, "granularity": "example", "size": 2},
                                    type_safe=False))
  config.extra_rng_keys = ("dropout", "gating", "mixup")
  state, metrics = trainer.train_and_evaluate(config, str(tmp_path), mesh=mesh, writer=_Writer())
  assert state.step == 3 and torch.isfinite(torch.as_tensor(metrics["total_loss"]))
