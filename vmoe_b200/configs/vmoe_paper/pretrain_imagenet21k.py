"""Pre-training of V-MoE S/32 ... H/14 on ImageNet-21k (https://arxiv.org/abs/2106.05974).

``get_config('synthetic')`` swaps the TFDS datasets for synthetic ones of the same shape so the
config runs offline; ``get_config('ViT-L/16, E=32, K=2, Every 2, 300 Epochs')`` selects another
architecture (reference: ``vmoe/configs/vmoe_paper/pretrain_imagenet21k.py``)."""
from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.utils.config_dict import ConfigDict

NUM_CLASSES = 21_843
DEFAULT_DESCRIPTION = "ViT-B/16, E=8, K=2, Every 2, 300 Epochs"


def get_config(arg: str = "") -> ConfigDict:
  synthetic = "synthetic" in arg
  description = arg.replace("synthetic", "").strip(" ;,") or DEFAULT_DESCRIPTION
  config = common.get_base_config()
  pp_common = f'value_range(-1,1)|onehot({NUM_CLASSES})|keep("image", "labels")'
  config.dataset = ConfigDict(type_safe=False)
  train = common.get_data_config(
      name="imagenet21k", split="full[102400:]", batch_size=4096, shuffle_buffer=250_000,
      process=f"decode_jpeg_and_inception_crop(224)|flip_lr|randaug(2,20)|{pp_common}")
  val = common.get_data_config(
      name="imagenet21k", split="full[:102400]", batch_size=4096, cache="batched",
      process=f"decode|resize_small(256)|central_crop(224)|{pp_common}")
  if synthetic:
    for d, split in ((train, "train"), (val, "validation[:8192]")):
      d.name, d.split = "synthetic", split
      d.num_classes, d.multi_label, d.image_size = NUM_CLASSES, True, 224
      d.process = f"flip_lr|{pp_common}"
  config.dataset.train, config.dataset.val = train, val
  config.loss = ConfigDict({"name": "sigmoid_xent"})
  config.description = description
  config.model = common.get_vmoe_config(description, 224, NUM_CLASSES)
  config.optimizer = common.get_optimizer_config(description)
  config.train_epochs = common.get_num_epochs(description)
  config.mixup = ConfigDict({"concentration": 0.5, "size": 2})
  config.num_expert_partitions = config.model.encoder.moe.num_experts
  config.params_axis_resources = [("Moe/Mlp/.*", ("expert",))]
  config.extra_rng_keys = ("dropout", "gating", "mixup")
  return config


def get_hyper(hyper):
  return hyper.product([])
