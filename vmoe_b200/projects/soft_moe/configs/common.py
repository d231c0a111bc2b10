"""Shared pieces of the Soft MoE configs: ViT Ti/S/B/L/H tables (gap classifier, QK
LayerNorm), the experts-choose baseline, the soft-router model, Adam + rsqrt schedule
(reference: ``vmoe/projects/soft_moe/configs/common.py:38-264``)."""
import math
from typing import Optional

from vmoe_b200.configs import common_fewshot
from vmoe_b200.configs.vmoe_paper.common import get_base_config, get_data_config  # noqa: F401
from vmoe_b200.utils.config_dict import ConfigDict

get_fewshot_config = common_fewshot.get_fewshot


def get_adam_config() -> ConfigDict:
  return ConfigDict({
      "name": "adam", "b1": 0.9, "b2": 0.999, "mu_dtype": "float32",
      "weight_decay": (("head/kernel", 3.0), (".*/kernel", 0.03)),
      "gradient_clip": {"global_norm": 1.0},
  }, type_safe=False)


def get_optimizer_linear_config() -> ConfigDict:
  """Adam with linear decay, as in "Scaling Vision Transformers"."""
  config = get_adam_config()
  config.learning_rate = ConfigDict({"schedule": "warmup_linear_decay", "peak_value": 8e-4,
                                     "end_value": 0.0, "warmup_steps": 10_000}, type_safe=False)
  return config


def get_optimizer_rsqrt_config() -> ConfigDict:
  """Adam with the reciprocal-square-root schedule of the ViT-22B paper."""
  config = get_adam_config()
  config.learning_rate = ConfigDict({
      "schedule": "big_vision_rsqrt", "peak_value": 1e-3, "warmup_steps": 10_000,
      "cooldown_steps": 50_000, "timescale": 10_000}, type_safe=False)
  return config


def get_imagenet_config(batch_size: int, resize_hi: int = 256, resize_lo: int = 224,
                        randaug: str = "", data_dir: Optional[str] = None) -> ConfigDict:
  """Dataset variants for training / evaluating on ImageNet: train, val, test, v2, real."""
  randaug = f"|{randaug}" if randaug and randaug[0] != "|" else randaug
  pp_common = lambda inkey: (f'value_range(-1,1)|onehot(1000, inkey="{inkey}", outkey="labels")|'
                             'keep("image", "labels")')
  pp_train = f'decode_jpeg_and_inception_crop({resize_lo})|flip_lr{randaug}|{pp_common("label")}'
  pp_eval1 = f'decode|resize_small({resize_hi})|central_crop({resize_lo})|{pp_common("label")}'
  pp_eval2 = (f'decode|resize_small({resize_hi})|central_crop({resize_lo})|'
              f'ignore_no_labels(labels_key="real_label")|{pp_common("real_label")}')
  ev = lambda name, split, pp: {"name": name, "split": split, "process": pp,
                                "batch_size": batch_size, "data_dir": data_dir, "cache": "batched"}
  return ConfigDict({
      "train": {"name": "imagenet2012", "split": "train[:99%]", "process": pp_train,
                "batch_size": batch_size, "data_dir": data_dir, "cache": "loaded",
                "shuffle_buffer": 250_000},
      "val": ev("imagenet2012", "train[99%:]", pp_eval1),
      "test": ev("imagenet2012", "validation", pp_eval1),
      "v2": ev("imagenet_v2", "test", pp_eval1),
      "real": ev("imagenet2012_real", "validation", pp_eval2),
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
