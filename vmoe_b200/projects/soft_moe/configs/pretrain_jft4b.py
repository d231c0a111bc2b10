"""Soft MoE paper pre-training: ``get_config('soft-b16')``, ``'ec-l16'``, ``'vit-s14'`` ...
(model type - backbone). Default experts: 128 (S/16, B/16, L/16) or 256 (S/14, H/14) in the
last 6 / 6 / 12 / 16 blocks, one slot per expert (reference:
``vmoe/projects/soft_moe/configs/pretrain_jft4b.py``). The dataset is not public; append
``,synthetic`` to run on synthetic data of the same shape."""
from vmoe_b200.projects.soft_moe.configs import common
from vmoe_b200.utils.config_dict import ConfigDict

DATASET = "jft4b"
NUM_CLASSES = 29_593
BATCH_SIZE = 4096
PP_COMMON = f'value_range(-1,1)|onehot({NUM_CLASSES})|keep("image", "labels")'


def get_default_moe_num_experts_and_last_n(variant: str, patch_size: int):
  num_experts = {("S", 16): 128, ("S", 14): 256, ("B", 16): 128, ("L", 16): 128,
                 ("H", 14): 256}[(variant, patch_size)]
  return num_experts, {"S": 6, "B": 6, "L": 12, "H": 16}[variant]


def get_config(model: str = "soft-s16") -> ConfigDict:
  synthetic = model.endswith(",synthetic")
  model = model.split(",")[0]
  model_type, backbone = model.split("-")
  patch_size, variant = int(backbone[1:]), backbone[0].upper()
  config = common.get_base_config()
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = common.get_data_config(
      name=DATASET, split="full[16384:]", batch_size=BATCH_SIZE,
      process=f"decode_jpeg_and_inception_crop(224)|flip_lr|{PP_COMMON}")
  config.dataset.val = common.get_data_config(
      name=DATASET, split="full[:16384]", batch_size=BATCH_SIZE, cache="batched",
      process=f"decode|resize_small(256)|central_crop(224)|{PP_COMMON}")
  if synthetic:
    for d, split in ((config.dataset.train, "train"), (config.dataset.val, "validation[:8192]")):
      d.name, d.split, d.num_classes, d.multi_label = "synthetic", split, NUM_CLASSES, True
      d.process = PP_COMMON
  else:
    config.fewshot = common.get_fewshot_config(batch_size=BATCH_SIZE, resize_resolution=256,
                                               target_resolution=224)
  config.loss = ConfigDict({"name": "sigmoid_xent"})
  config.optimizer = common.get_optimizer_rsqrt_config()
  if model_type == "vit":
    config.model = common.get_vit_config(variant, patch_size, NUM_CLASSES)
  elif model_type == "ec":
    e, last_n = get_default_moe_num_experts_and_last_n(variant, patch_size)
    config.model = common.get_vmoe_experts_choose_config(
        variant, patch_size, NUM_CLASSES, image_size=224, num_experts=e, last_n=last_n,
        capacity_factor=1.0)
  elif model_type == "soft":
    e, last_n = get_default_moe_num_experts_and_last_n(variant, patch_size)
    config.model = common.get_vmoe_soft_router_config(
        variant, patch_size, NUM_CLASSES, image_size=224, num_experts=e, last_n=last_n,
        capacity_factor=None, num_slots=1)
    config.model.encoder.moe.router.compute_similarity_metrics = False
    config.optimizer.weight_decay = tuple(config.optimizer.weight_decay) + (
        (".*/Moe/Router/scale", 0.03),)
  else:
    raise ValueError(f"Unknown model type: {model_type!r}")
  config.train_steps = 2_000_000 if variant == "H" else 4_000_000
  if model_type == "vit":
    config.num_expert_partitions = 1
    config.params_axis_resources = []
  else:
    config.num_expert_partitions = config.model.encoder.moe.num_experts
    config.params_axis_resources = [("Moe/Mlp/.*", ("expert",))]
  config.extra_rng_keys = ("dropout", "gating")
  config.summarize_arrays = ConfigDict({
      "rules": ["opt_state/.*/hyperparams/learning_rate", "params/.*/Moe/Router/scale"],
      "max_summary_values": 1}, type_safe=False)
  config.save_checkpoint.keep_last = 2
  config.save_checkpoint.keep_steps_multiple_of = 50_000
  return config


def get_hyper(hyper, model="soft-s16"):
  del model
  return hyper.product([])
