"""Standard few-shot evaluation settings (reference: ``vmoe/configs/common_fewshot.py``)."""
from typing import Optional

from vmoe_b200.utils.config_dict import ConfigDict


def get_fewshot(*, batch_size: int, resize_resolution: int = 256, target_resolution: int = 224,
                every_steps: Optional[int] = 25_000, seeds_per_step: int = 1) -> ConfigDict:
  config = ConfigDict(type_safe=False)
  config.datasets = {
      "birds": ("caltech_birds2011", "train", "test"),
      "caltech": ("caltech101", "train", "test"),
      "cars": ("cars196:2.1.0", "train", "test"),
      "cifar100": ("cifar100", "train", "test"),
      "col_hist": ("colorectal_histology", "train[:2000]", "train[2000:]"),
      "dtd": ("dtd", "train", "test"),
      "imagenet": ("imagenet2012_subset/10pct", "train", "validation"),
      "pets": ("oxford_iiit_pet", "train", "test"),
      "uc_merced": ("uc_merced", "train[:1000]", "train[1000:]"),
  }
  config.batch_size = batch_size
  config.process = (f"decode|resize({resize_resolution})|central_crop({target_resolution})|"
                    'value_range(-1, 1)|keep("image", "label")')
  config.cache = "loaded"
  config.shots = [1, 5, 10, 25]
  config.l2_regs = [2.0 ** i for i in range(-10, 20)]
  config.main_task = ("imagenet", 10)
  config.model_overrides = ConfigDict({"num_classes": None}, type_safe=False)
  if every_steps:
    config.every_steps = every_steps
  if seeds_per_step:
    config.seeds_per_step = seeds_per_step
  return config
