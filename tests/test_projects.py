"""Project configs and the E^3 demo helpers (CPU)."""
import math

import torch

from vmoe_b200.notebooks import demo_eee_cifar100 as demo
from vmoe_b200.projects.soft_moe.configs import pretrain_laion


def test_laion_config_variants():
  cfg = pretrain_laion.get_config("soft-b16")
  assert cfg.model.name.endswith("contrastive.models.TwoTower")
  assert cfg.model.image.encoder.moe.num_experts == 128
  assert cfg.model.image.encoder.moe.router.name == "SoftRouter"
  assert cfg.model.text.num_classes == cfg.model.image.hidden_size == 768
  assert cfg.num_expert_partitions == 128
  assert cfg.optimizer.learning_rate.warmup_steps == 20_000
  vit = pretrain_laion.get_config("vit-s14")
  assert vit.num_expert_partitions == 1 and vit.params_axis_resources == []
  syn = pretrain_laion.get_config("ec-l16,synthetic")
  assert syn.dataset.train.name == "synthetic_text" and "fewshot" not in syn


def test_ensemble_log_probs_averages_member_probabilities():
  torch.manual_seed(0)
  logits = torch.randn(6, 5)  # 3 images x 2 members
  out = demo.ensemble_log_probs(logits, 2)
  p = torch.softmax(logits.reshape(3, 2, 5), -1).mean(1)
  assert torch.allclose(out.exp(), p, atol=1e-6)
  assert math.isclose(float(out.exp().sum(-1)[0]), 1.0, rel_tol=1e-5)


def test_demo_model_config_group_size():
  cfg = demo.model_config(batch_size=1024, num_devices=8)
  assert cfg["encoder"]["moe"]["group_size"] == (1024 // 8) * 17 * 2
