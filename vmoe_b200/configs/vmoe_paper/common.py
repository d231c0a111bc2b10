"""Shared pieces of the V-MoE paper configs: base options, dataset blocks, the optimizer and
the model factory driven by a description string such as
``'ViT-B/16, E=8, K=2, Every 2, 300 Epochs'``.

Values follow the reference (``vmoe/configs/vmoe_paper/common.py:33-256``): S/B/L/H = hidden
512/768/1024/1280, layers 8/12/24/32, MLP 2048/3072/4096/5120, heads 8/12/16/16; ``Every n``
puts MoE layers at ``n-1, 2n-1, ...``; ``Last n`` takes the last n odd layers; the routing
group is 8 images' worth of tokens.
"""
from __future__ import annotations

import math
import re
from typing import Optional

from vmoe_b200.utils.config_dict import ConfigDict

DESCRIPTIONS_REGEX = re.compile(
    r"^ViT-(?P<variant>.)/(?P<patch>[0-9]+), "
    r"E=(?P<num_experts>[0-9]+), "
    r"K=(?P<k>[0-9]+), "
    r"(?P<where>Every|Last) (?P<where_num>[0-9]+)"
    r"(?:, (?P<epochs>[0-9]+) Epochs)?$")

VARIANTS = ["S", "B", "L", "H"]


def _match(description: str):
  m = DESCRIPTIONS_REGEX.match(description)
  if not m:
    raise ValueError(f"Description {description!r} doesn't match the regex.")
  return m


def flatten_dict(config, prefix=""):
  if isinstance(config, ConfigDict):
    config = config.to_dict()
  flat = {}
  for k, v in config.items():
    if isinstance(v, dict):
      flat.update(flatten_dict(v, prefix=f"{prefix}{k}."))
    else:
      flat[f"{prefix}{k}"] = v
  return flat


def get_base_config() -> ConfigDict:
  config = ConfigDict()
  config.save_checkpoint = ConfigDict()
  config.save_checkpoint.every_steps = 1_000
  config.save_checkpoint.keep_last = 1
  config.save_checkpoint.wait_seconds = 300
  config.report_progress = ConfigDict(type_safe=False)
  config.report_progress.every_secs = 60.0
  config.report_progress.every_steps = 250
  config.evaluate = ConfigDict(type_safe=False)
  config.evaluate.every_steps = 1_000
  config.profile = ConfigDict()
  config.profile.all_processes = False
  config.profile.num_profile_steps = 5
  config.profile.first_profile = 10
  config.profile.every_secs = 3600.0
  config.seed = 0
  return config


def get_data_config(name: str, split: str, process: str, batch_size: int,
                    shuffle_buffer: Optional[int] = None, cache: Optional[str] = None,
                    data_dir: Optional[str] = None) -> ConfigDict:
  config = ConfigDict(type_safe=False)
  config.name = name
  config.split = split
  config.process = process
  config.batch_size = batch_size
  config.prefetch = "autotune"
  config.prefetch_device = 2
  if shuffle_buffer:
    config.shuffle_buffer = shuffle_buffer
  if cache:
    config.cache = cache
  if data_dir:
    config.data_dir = data_dir
  return config


def get_mixup_concentration(aug: str) -> float:
  return {"light0": 0.0, "light1": 0.2, "medium1": 0.2, "medium2": 0.5, "strong1": 0.5,
          "strong2": 0.8, "extreme1": 0.5, "extreme2": 0.8}[aug]


def get_mixup_config(aug: str) -> ConfigDict:
  config = ConfigDict()
  config.granularity = "device"
  config.size = 2
  config.concentration = get_mixup_concentration(aug)
  return config


def get_num_epochs(description: str) -> int:
  m = _match(description)
  if m.group("epochs") is None:
    raise ValueError(f"Description {description!r} has no number of epochs.")
  return int(m.group("epochs"))


def get_optimizer_config(description: str) -> ConfigDict:
  m = _match(description)
  variant, patch = m.group("variant"), int(m.group("patch"))
  config = ConfigDict(type_safe=False)
  config.name = "adam"
  config.b1 = 0.9
  config.b2 = 0.999
  config.mu_dtype = "float32"
  config.weight_decay = 0.1
  config.learning_rate = ConfigDict()
  config.learning_rate.schedule = "warmup_linear_decay"
  config.learning_rate.peak_value = {
      ("S", 32): 1e-3, ("B", 32): 8e-4, ("B", 16): 8e-4, ("L", 32): 6e-4, ("L", 16): 4e-4,
      ("H", 14): 3e-4}.get((variant, patch), 4e-4)
  config.learning_rate.end_value = 1e-5
  config.learning_rate.warmup_steps = 10_000
  config.gradient_clip = ConfigDict({"global_norm": 10.0 if variant == "H" else None},
                                    type_safe=False)
  return config


def get_randaug(aug: str) -> str:
  l, m = {"light0": (2, 0), "light1": (2, 10), "medium1": (2, 15), "medium2": (2, 15),
          "strong1": (2, 20), "strong2": (2, 20), "extreme1": (4, 15), "extreme2": (4, 20)}[aug]
  return f"randaug({l}, {m})"


def get_vmoe_config(description: str, image_size: int, num_classes: int) -> ConfigDict:
  """Model config for a canonical architecture description."""
  m = _match(description)
  variant_idx = VARIANTS.index(m.group("variant"))
  patch_size = int(m.group("patch"))
  num_experts = int(m.group("num_experts"))
  k = int(m.group("k"))
  where, where_num = m.group("where"), int(m.group("where_num"))
  # Routing groups: the tokens of 8 images (the smallest per-device batch assumed).
  num_tokens = (image_size // patch_size) ** 2 + 1
  group_size = 8 * num_tokens

  config = ConfigDict()
  config.name = "VisionTransformerMoe"
  config.num_classes = num_classes
  config.patch_size = (patch_size, patch_size)
  config.hidden_size = [512, 768, 1024, 1280][variant_idx]
  config.classifier = "token"
  config.representation_size = config.hidden_size
  config.head_bias_init = -math.log(num_classes)
  config.encoder = ConfigDict()
  config.encoder.num_layers = [8, 12, 24, 32][variant_idx]
  config.encoder.mlp_dim = [2048, 3072, 4096, 5120][variant_idx]
  config.encoder.num_heads = [8, 12, 16, 16][variant_idx]
  config.encoder.dropout_rate = 0.0
  config.encoder.attention_dropout_rate = 0.0
  config.encoder.moe = ConfigDict()
  config.encoder.moe.num_experts = num_experts
  if where == "Every":
    config.encoder.moe.layers = tuple(range(where_num - 1, config.encoder.num_layers, where_num))
  else:
    config.encoder.moe.layers = tuple(range(1, config.encoder.num_layers, 2))[-where_num:]
  config.encoder.moe.dropout_rate = 0.0
  config.encoder.moe.split_rngs = False
  config.encoder.moe.group_size = group_size
  config.encoder.moe.router = ConfigDict()
  config.encoder.moe.router.num_selected_experts = k
  config.encoder.moe.router.noise_std = 1.0  # the effective std is 1 / num_experts
  config.encoder.moe.router.importance_loss_weight = 0.005
  config.encoder.moe.router.load_loss_weight = 0.005
  config.encoder.moe.router.dispatcher = ConfigDict()
  config.encoder.moe.router.dispatcher.name = "einsum"
  config.encoder.moe.router.dispatcher.bfloat16 = True
  config.encoder.moe.router.dispatcher.capacity_factor = 1.05
  config.encoder.moe.router.dispatcher.partition_spec = (("expert", "replica"),)
  config.encoder.moe.router.dispatcher.batch_priority = False
  return config
