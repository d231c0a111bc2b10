"""Shared builder of the three fine-tuning configs of the V-MoE paper: a released checkpoint is
mapped onto a model at a new resolution / label space with initialization rules (head dropped,
position embeddings resized), then trained with SGD momentum 0.9, gradient clipping and cosine
decay. Every value below is the one of the reference's ``vmoe/configs/vmoe_paper/*_ft_*.py``
file of the same name; the three config files next to this one select a variant.
"""
from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.utils.config_dict import ConfigDict

BATCH_SIZE = 1024

_VARIANTS = {
    # vmoe_s32_last2_ilsvrc2012_randaug_light1_ft_ilsvrc2012.py
    "s32_ilsvrc2012": dict(
        description="ViT-S/32, E=8, K=2, Last 2, 300 Epochs",
        prefix="gs://vmoe_checkpoints/vmoe_s32_last2_ilsvrc2012_randaug_light1",
        dataset="imagenet2012", num_classes=1000, image_size=384, train_steps=10_000,
        train_split="train[:99%]", val_split="train[99%:]", test_split="validation",
        train_decode="decode_jpeg_and_inception_crop({size})", imagenet_extras=True,
        peak_value=0.003, warmup_steps=500, evaluate_every_steps=None,
        drop_pre_logits=True, explicit_prefetch=True),
    # vmoe_b16_imagenet21k_randaug_strong_ft_ilsvrc2012.py
    "b16_ilsvrc2012": dict(
        description="ViT-B/16, E=8, K=2, Every 2, 300 Epochs",
        prefix="gs://vmoe_checkpoints/vmoe_b16_imagenet21k_randaug_strong",
        dataset="imagenet2012", num_classes=1000, image_size=384, train_steps=10_000,
        train_split="train[:99%]", val_split="train[99%:]", test_split="validation",
        train_decode="decode_jpeg_and_inception_crop({size})", imagenet_extras=True,
        peak_value=0.003, warmup_steps=500, evaluate_every_steps=None,
        drop_pre_logits=False, explicit_prefetch=False),
    # vmoe_b16_imagenet21k_randaug_strong_ft_cifar10.py
    "b16_cifar10": dict(
        description="ViT-B/16, E=8, K=2, Every 2, 300 Epochs",
        prefix="gs://vmoe_checkpoints/vmoe_b16_imagenet21k_randaug_strong",
        dataset="cifar10", num_classes=10, image_size=128, train_steps=1_000,
        train_split="train[:98%]", val_split="train[98%:]", test_split="test",
        train_decode="decode|inception_crop({size})", imagenet_extras=False,
        peak_value=0.0015, warmup_steps=100, evaluate_every_steps=100,
        drop_pre_logits=False, explicit_prefetch=False),
}


def _data(v, name, split, process, train):
  cfg = common.get_data_config(
      name=name, split=split, process=process, batch_size=BATCH_SIZE,
      shuffle_buffer=50_000 if train else None, cache=None if train else "batched")
  cfg.data_dir = None
  cfg.manual_dir = None
  if v["explicit_prefetch"]:
    cfg.prefetch = 16 if train else 1
    cfg.prefetch_device = 1
  return cfg


def get_config(arg: str = "b16_ilsvrc2012") -> ConfigDict:
  v = _VARIANTS[arg]
  size, classes = v["image_size"], v["num_classes"]
  pp_common = (f'value_range(-1,1)|onehot({classes}, inkey="label", outkey="labels")|'
               'keep("image", "labels")')
  config = common.get_base_config()
  if v["evaluate_every_steps"] is not None:
    config.evaluate.every_steps = v["evaluate_every_steps"]
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = _data(
      v, v["dataset"], v["train_split"],
      f'{v["train_decode"].format(size=size)}|flip_lr|{pp_common}', train=True)
  eval_pp = f"decode|resize({size})|{pp_common}"
  config.dataset.val = _data(v, v["dataset"], v["val_split"], eval_pp, train=False)
  config.dataset.test = _data(v, v["dataset"], v["test_split"], eval_pp, train=False)
  if v["imagenet_extras"]:
    config.dataset.test_real = _data(
        v, "imagenet2012_real", "validation",
        (f"decode|resize({size})|value_range(-1,1)|"
         f'onehot({classes}, inkey="real_label", outkey="labels")|keep("image", "labels")'),
        train=False)
    config.dataset.imagenet_v2 = _data(v, "imagenet_v2", "test", eval_pp, train=False)
  config.loss = ConfigDict({"name": "softmax_xent"})
  config.train_steps = v["train_steps"]
  config.description = v["description"]
  config.model = common.get_vmoe_config(v["description"], size, classes)
  config.model.representation_size = None
  config.model.encoder.moe.router.dispatcher.capacity_factor = 1.5
  rules = [("head", "")]                                    # do not restore the head
  if v["drop_pre_logits"]:
    rules.append(("pre_logits/.*", ""))                     # nor the pre-logits layer
  rules += [("^(.*/pos_embedding)$", r"params/\1", "vit_zoom"),  # resize position embeddings
            ("^(.*)$", r"params/\1")]                            # everything else as is
  config.initialization = ConfigDict({
      "name": "initialize_from_vmoe",
      "prefix": v["prefix"],
      "rules": rules,
      "raise_if_target_unmatched": False,
      "axis_resources_regexes": [("Moe/Mlp/.*", ("expert",))],
  }, type_safe=False)
  config.optimizer = ConfigDict({
      "name": "sgd", "momentum": 0.9, "accumulator_dtype": "float32",
      "learning_rate": {"schedule": "warmup_cosine_decay", "peak_value": v["peak_value"],
                        "end_value": 1e-5, "warmup_steps": v["warmup_steps"]},
      "gradient_clip": {"global_norm": 10.0},
  }, type_safe=False)
  config.num_expert_partitions = config.model.encoder.moe.num_experts
  config.params_axis_resources = [("Moe/Mlp/.*", ("expert",))]
  config.extra_rng_keys = ("dropout", "gating")
  return config


def get_hyper(hyper):
  """Three fine-tuning seeds, as in every ``*_ft_*`` config of the reference."""
  return hyper.sweep("config.seed", list(range(3)))
