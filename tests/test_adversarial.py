"""PGD attack project: attack arithmetic, routing-change statistics, dispatcher capture and the
end-to-end ``run_pgd_attack`` on a tiny V-MoE restored from a sharded checkpoint (CPU)."""
import os

import numpy as np
import pytest
import torch

from vmoe_b200 import moe
from vmoe_b200 import models as models_lib
from vmoe_b200.checkpoints import flax_layout
from vmoe_b200.checkpoints import partitioned
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.projects.adversarial_attacks import attacks
from vmoe_b200.projects.adversarial_attacks import lib
from vmoe_b200.projects.adversarial_attacks import restore
from vmoe_b200.utils.config_dict import ConfigDict


def test_pgd_moves_by_epsilon_in_sign_direction():
  w = torch.tensor([1.0, -2.0, 0.5])
  x = torch.zeros(4, 3)
  out = attacks.stateless_attack_pgd(x, lambda v: ((v * w).sum(), None), max_epsilon=0.3,
                                     num_updates=3)
  np.testing.assert_allclose(out.numpy(), np.tile([0.3, -0.3, 0.3], (4, 1)), atol=1e-6)


def test_sum_intersection_over_union():
  a = torch.tensor([[[1., 0, 1, 0], [0, 1, 0, 0]]])
  b = torch.tensor([[[1., 1, 0, 0], [0, 1, 0, 0]]])
  # token 0: |{0}| / |{0,1,2}| = 1/3, token 1: 1 -> mean over 2 tokens.
  assert float(attacks.sum_intersection_over_union(a, b)) == pytest.approx((1 / 3 + 1) / 2)


def test_combine_weights_from_dispatchers():
  g, s, e, c = 2, 3, 4, 2
  cw = torch.rand(g, s, e, c)
  ein = moe.EinsumDispatcher(combine_weights=cw)
  out = restore.get_combine_weights({"r": moe.Bfloat16Dispatcher(ein)})["r"]
  np.testing.assert_allclose(out.numpy(), cw.sum(3).reshape(-1, e).numpy(), rtol=1e-6)
  idx = torch.tensor([[[[0, 0], [3, 1]], [[1, 0], [2, 0]], [[3, 0], [0, 1]]]] * g)
  w = torch.rand(g, s, 2)
  ind = moe.ExpertIndicesDispatcher(indices=idx, combine_weights=w, num_experts=e, capacity=c)
  out = restore.get_combine_weights({"r": ind})["r"].reshape(g, s, e)
  assert float(out[0, 0, 0]) == pytest.approx(float(w[0, 0, 0]))
  assert float(out[0, 0, 3]) == pytest.approx(float(w[0, 0, 1]))
  assert float(out[0, 1, 0]) == 0.0


def _tiny_config(tmp, prefix):
  config = ConfigDict(type_safe=False)
  config.dataset = ConfigDict({
      "name": "synthetic", "split": "validation", "image_size": 16, "num_classes": 5,
      "num_eval_examples": 6, "batch_size": 4,
      "process": 'value_range(-1,1)|onehot(5, inkey="label", outkey="labels")|keep("image", "labels")',
  }, type_safe=False)
  config.num_updates = 2
  config.max_epsilon = 0.1
  config.restore = ConfigDict({"from": "checkpoint", "prefix": prefix})
  config.loss = ConfigDict({"name": "softmax_xent", "attack_auxiliary_loss": True})
  config.model = ConfigDict({
      "name": "VisionTransformerMoe", "num_classes": 5, "patch_size": (8, 8), "hidden_size": 16,
      "classifier": "token", "representation_size": None,
      "encoder": {"num_layers": 2, "num_heads": 2, "mlp_dim": 32, "dropout_rate": 0.0,
                  "attention_dropout_rate": 0.0,
                  "moe": {"num_experts": 2, "layers": (1,), "group_size": 5,
                          "router": {"num_selected_experts": 1, "noise_std": 0.0,
                                     "importance_loss_weight": 0.01,
                                     "dispatcher": {"name": "einsum", "capacity_factor": 2.0,
                                                    "batch_priority": False}}}},
  }, type_safe=False)
  config.num_expert_partitions = 1
  config.store_examples = ConfigDict({"transfer_every_steps": 1})
  return config


class _Writer:
  def __init__(self):
    self.scalars = {}

  def write_scalars(self, step, scalars):
    self.scalars[step] = dict(scalars)


def test_run_pgd_attack_end_to_end(tmp_path):
  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  prefix = os.path.join(str(tmp_path), "ckpt")
  config = _tiny_config(str(tmp_path), prefix)
  torch.manual_seed(0)
  model = models_lib.create_model(config.model, deterministic=True, mesh=mesh, image_size=16)
  params, specs = flax_layout.to_flax(model)
  res = partitioned.save_checkpoint(prefix, params, shardings=specs, mesh=mesh)
  if res is not None:
    res.get()
  writer = _Writer()
  state = lib.run_pgd_attack(config, str(tmp_path), writer=writer)
  assert int(state.num_images) == 6  # 2 of the 8 batch slots are padding
  saved = np.load(os.path.join(str(tmp_path), "pgd_state.npz"))
  assert int(saved["num_images"]) == 6
  assert saved["sum_loss"][1] >= saved["sum_loss"][0]  # the attack ascends the loss
  assert set(writer.scalars) == {0, 2}
  assert any(k.startswith("routing_changes/") for k in writer.scalars[2])
  examples = np.load(os.path.join(str(tmp_path), "examples-000-of-001"))
  assert examples["x_0"].shape == examples["x_m"].shape
  assert np.abs(examples["x_m"] - examples["x_0"]).max() <= 0.1 + 1e-5
