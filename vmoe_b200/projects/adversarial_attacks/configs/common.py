"""Config helpers of "On the Adversarial Robustness of Mixture of Experts": the ILSVRC2012
fine-tuning base (SGD momentum 0.9, peak lr 0.03, cosine decay, clip 10), the dense ViT
family including the B+/B++/B+++ sizes interpolated between B and L, and V-MoE models whose
auxiliary loss switches to the GShard loss when there are only two experts
(``vmoe/projects/adversarial_attacks/configs/common.py:17-137``)."""
import math
import re

from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.utils.config_dict import ConfigDict

IMAGENET_BATCH_SIZE = 1024
IMAGENET_NUM_CLASSES = 1000
IMAGENET_IMAGE_SIZE = 384

flatten_dict = common.flatten_dict

_VIT_VARIANTS = ["S", "B", "B+", "B++", "B+++", "L", "H"]
_VIT_HIDDEN = [512, 768, 832, 896, 960, 1024, 1280]
_VIT_LAYERS = [8, 12, 15, 18, 21, 24, 32]
_VIT_MLP = [2048, 3072, 3328, 3584, 3840, 4096, 5120]
_VIT_HEADS = [8, 12, 13, 14, 15, 16, 16]


def get_num_epochs(description: str) -> int:
  match = re.match(r".*, ([0-9]+) Epochs$", description)
  if not match:
    raise ValueError(f"The number of epochs can't be parsed from {description!r}.")
  return int(match.group(1))


def get_base_finetune_config(batch_size: int = IMAGENET_BATCH_SIZE,
                             image_size: int = IMAGENET_IMAGE_SIZE,
                             num_classes: int = IMAGENET_NUM_CLASSES) -> ConfigDict:
  config = common.get_base_config()
  config.evaluate.every_steps = 100
  config.dataset = ConfigDict(type_safe=False)
  pp_common = (f'value_range(-1,1)|onehot({num_classes}, inkey="label", outkey="labels")|'
               'keep("image", "labels")')
  config.dataset.train = common.get_data_config(
      name="imagenet2012", split="train[:99%]", batch_size=batch_size,
      process=f"decode_jpeg_and_inception_crop({image_size})|flip_lr|{pp_common}",
      shuffle_buffer=50_000, cache=None)
  config.dataset.val = common.get_data_config(
      name="imagenet2012", split="train[99%:]", batch_size=batch_size,
      process=f"decode|resize({image_size})|{pp_common}", shuffle_buffer=None, cache="batched")
  config.dataset.test = common.get_data_config(
      name="imagenet2012", split="validation", batch_size=batch_size,
      process=f"decode|resize({image_size})|{pp_common}", shuffle_buffer=None, cache="batched")
  config.dataset.test_real = common.get_data_config(
      name="imagenet2012_real", split="validation", batch_size=batch_size,
      process=(f"decode|resize({image_size})|value_range(-1,1)|"
               f'onehot({num_classes}, inkey="real_label", outkey="labels")|'
               'keep("image", "labels")'),
      shuffle_buffer=None, cache="batched")
  config.loss = ConfigDict({"name": "softmax_xent"})
  config.train_steps = 10_000
  config.optimizer = ConfigDict({
      "name": "sgd",
      "momentum": 0.9,
      "accumulator_dtype": "float32",
      "learning_rate": {"schedule": "warmup_cosine_decay", "peak_value": 0.03,
                        "end_value": 1e-5, "warmup_steps": 500},
      "gradient_clip": {"global_norm": 10.0},
  }, type_safe=False)
  return config


def get_vit_config(description: str, num_classes: int) -> ConfigDict:
  match = re.match(r"^ViT-(?P<variant>[^/]+)/(?P<patch>[0-9]+)", description)
  if not match:
    raise ValueError(f"Description {description!r} doesn't match the regex.")
  idx = _VIT_VARIANTS.index(match.group("variant"))
  patch = int(match.group("patch"))
  config = ConfigDict(type_safe=False)
  config.name = "VisionTransformer"
  config.num_classes = num_classes
  config.patches = ConfigDict({"size": (patch, patch)})
  config.hidden_size = _VIT_HIDDEN[idx]
  config.classifier = "token"
  config.representation_size = config.hidden_size
  config.head_bias_init = -math.log(num_classes)
  config.transformer = ConfigDict()
  config.transformer.num_layers = _VIT_LAYERS[idx]
  config.transformer.mlp_dim = _VIT_MLP[idx]
  config.transformer.num_heads = _VIT_HEADS[idx]
  config.transformer.dropout_rate = 0.0
  config.transformer.attention_dropout_rate = 0.0
  return config


def get_vmoe_config(description: str, num_classes: int, image_size: int) -> ConfigDict:
  config = common.get_vmoe_config(description, image_size=image_size, num_classes=num_classes)
  # With two experts the load loss of the V-MoE paper can produce NaNs; use GShard's instead.
  router = config.encoder.moe.router
  if config.encoder.moe.num_experts > 2:
    router.importance_loss_weight = 0.005
    router.load_loss_weight = 0.005
    router.gshard_loss_weight = 0.0
  else:
    router.importance_loss_weight = 0.0
    router.load_loss_weight = 0.0
    router.gshard_loss_weight = 0.01
  return config
