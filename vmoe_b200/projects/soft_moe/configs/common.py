"""Shared pieces of the Soft MoE configs: ViT Ti/S/B/L/H tables (gap classifier, QK
LayerNorm), the experts-choose baseline, the soft-router model, Adam + rsqrt schedule
(reference: ``vmoe/projects/soft_moe/configs/common.py:38-264``)."""
import math
from typing import Optional

from vmoe_b200.configs import common_fewshot
from vmoe_b200.configs.vmoe_paper.common import get_base_config, get_data_config  # noqa: F401
from vmoe_b200.utils.config_dict import ConfigDict

get_fewshot_config = common_fewshot.get_fewshot


def get_optimizer_rsqrt_config() -> ConfigDict:
  return ConfigDict({
      "name": "adam", "b1": 0.9, "b2": 0.999, "mu_dtype": "float32",
      "weight_decay": (("head/kernel", 3.0), (".*/kernel", 0.03)),
      "gradient_clip": {"global_norm": 1.0},
      "learning_rate": {"schedule": "big_vision_rsqrt", "peak_value": 1e-3,
                        "warmup_steps": 10_000, "cooldown_steps": 50_000, "timescale": 100_000},
  }, type_safe=False)


def get_vit_config(variant: str, patch_size: int, num_classes: Optional[int]) -> ConfigDict:
  i = ["Ti", "S", "B", "L", "H"].index(variant)
  return ConfigDict({
      "name": "VisionTransformerMoe",
      "num_classes": num_classes,
      "patch_size": (patch_size, patch_size),
      "hidden_size": [192, 384, 768, 1024, 1280][i],
      "classifier": "gap",
      "head_bias_init": -math.log(num_classes) if num_classes else 0.0,
      "encoder": {
          "num_layers": [12, 12, 12, 24, 32][i], "mlp_dim": [768, 1536, 3072, 4096, 5120][i],
          "num_heads": [3, 6, 12, 16, 16][i], "dropout_rate": 0.0,
          "attention_dropout_rate": 0.0, "attention_qk_norm": True, "moe": {"layers": ()},
      },
  }, type_safe=False)


def get_vmoe_experts_choose_config(variant, patch_size, num_classes, *, image_size, num_experts,
                                   last_n, capacity_factor: float = 1.0) -> ConfigDict:
  config = get_vit_config(variant, patch_size, num_classes)
  config.encoder.moe = ConfigDict({
      "layers": tuple(range(config.encoder.num_layers))[-last_n:],
      "num_experts": num_experts,
      "group_size": (image_size // patch_size) ** 2,
      "split_rngs": False,
      "router": {
          "name": "NoisyTopItemsPerExpertRouter", "noise_std": 1.0,
          "dispatcher": {"name": "einsum", "bfloat16": True, "capacity_factor": capacity_factor,
                         "capacity_ceil_or_round": "round", "capacity_multiple_of": 1,
                         "partition_spec": (("expert", "replica"),)},
      },
  }, type_safe=False)
  return config


def get_vmoe_soft_router_config(variant, patch_size, num_classes, *, image_size, num_experts,
                                last_n, capacity_factor: Optional[float] = 1.0,
                                num_slots: Optional[int] = None) -> ConfigDict:
  config = get_vit_config(variant, patch_size, num_classes)
  config.encoder.moe = ConfigDict({
      "layers": tuple(range(config.encoder.num_layers))[-last_n:],
      "num_experts": num_experts,
      "group_size": (image_size // patch_size) ** 2,
      "split_rngs": False,
      "router": {"name": "SoftRouter", "capacity_factor": capacity_factor, "num_slots": num_slots,
                 "partition_spec": (("expert", "replica"),), "compute_similarity_metrics": True},
  }, type_safe=False)
  return config
