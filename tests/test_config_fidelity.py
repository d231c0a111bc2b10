"""Shipped configs against values transcribed (by reading) from the reference's config files
``vmoe/configs/**`` and ``vmoe/projects/soft_moe/configs/common.py``: the entries that decide
what is trained (optimizer, schedule, model, datasets, evaluation cadence, seeds sweep)."""
import importlib

import pytest

from vmoe_b200.utils import misc

CFG = "vmoe_b200.configs.vmoe_paper."

FT_COMMON = {
    "loss.name": "softmax_xent",
    "optimizer.name": "sgd", "optimizer.momentum": 0.9, "optimizer.accumulator_dtype": "float32",
    "optimizer.learning_rate.schedule": "warmup_cosine_decay",
    "optimizer.learning_rate.end_value": 1e-5,
    "optimizer.gradient_clip.global_norm": 10.0,
    "model.representation_size": None,
    "model.encoder.moe.router.dispatcher.capacity_factor": 1.5,
    "model.encoder.moe.router.dispatcher.name": "einsum",
    "model.encoder.moe.router.noise_std": 1.0,
    "model.encoder.moe.router.importance_loss_weight": 0.005,
    "model.encoder.moe.router.load_loss_weight": 0.005,
    "initialization.name": "initialize_from_vmoe",
    "initialization.raise_if_target_unmatched": False,
    "num_expert_partitions": 8, "extra_rng_keys": ("dropout", "gating"),
    "save_checkpoint.every_steps": 1000, "save_checkpoint.keep_last": 1,
    "report_progress.every_secs": 60.0, "report_progress.every_steps": 250,
    "profile.num_profile_steps": 5, "profile.first_profile": 10, "seed": 0,
    "dataset.train.batch_size": 1024, "dataset.train.shuffle_buffer": 50_000,
    "dataset.val.cache": "batched", "dataset.test.cache": "batched",
}

TABLE = {
    "vmoe_b16_imagenet21k_randaug_strong_ft_cifar10": {
        **FT_COMMON,
        "evaluate.every_steps": 100, "train_steps": 1000,
        "description": "ViT-B/16, E=8, K=2, Every 2, 300 Epochs",
        "optimizer.learning_rate.peak_value": 0.0015, "optimizer.learning_rate.warmup_steps": 100,
        "dataset.train.name": "cifar10", "dataset.train.split": "train[:98%]",
        "dataset.val.split": "train[98%:]", "dataset.test.split": "test",
        "dataset.train.process": ('decode|inception_crop(128)|flip_lr|value_range(-1,1)|'
                                  'onehot(10, inkey="label", outkey="labels")|keep("image", "labels")'),
        "dataset.train.prefetch": "autotune", "dataset.train.prefetch_device": 2,
        "model.num_classes": 10, "model.hidden_size": 768, "model.encoder.num_layers": 12,
        "model.encoder.moe.layers": (1, 3, 5, 7, 9, 11), "model.encoder.moe.group_size": 8 * 65,
        "initialization.prefix": "gs://vmoe_checkpoints/vmoe_b16_imagenet21k_randaug_strong",
        "initialization.rules": [("head", ""), ("^(.*/pos_embedding)$", r"params/\1", "vit_zoom"),
                                 ("^(.*)$", r"params/\1")],
    },
    "vmoe_b16_imagenet21k_randaug_strong_ft_ilsvrc2012": {
        **FT_COMMON,
        "evaluate.every_steps": 1000, "train_steps": 10_000,
        "description": "ViT-B/16, E=8, K=2, Every 2, 300 Epochs",
        "optimizer.learning_rate.peak_value": 0.003, "optimizer.learning_rate.warmup_steps": 500,
        "dataset.train.name": "imagenet2012", "dataset.train.split": "train[:99%]",
        "dataset.val.split": "train[99%:]", "dataset.test.split": "validation",
        "dataset.test_real.name": "imagenet2012_real", "dataset.test_real.split": "validation",
        "dataset.test_real.process": ('decode|resize(384)|value_range(-1,1)|'
                                      'onehot(1000, inkey="real_label", outkey="labels")|'
                                      'keep("image", "labels")'),
        "dataset.imagenet_v2.name": "imagenet_v2", "dataset.imagenet_v2.split": "test",
        "dataset.train.process": ('decode_jpeg_and_inception_crop(384)|flip_lr|value_range(-1,1)|'
                                  'onehot(1000, inkey="label", outkey="labels")|'
                                  'keep("image", "labels")'),
        "dataset.train.prefetch": "autotune",
        "model.num_classes": 1000, "model.encoder.moe.group_size": 8 * 577,
        "initialization.prefix": "gs://vmoe_checkpoints/vmoe_b16_imagenet21k_randaug_strong",
    },
    "vmoe_s32_last2_ilsvrc2012_randaug_light1_ft_ilsvrc2012": {
        **FT_COMMON,
        "evaluate.every_steps": 1000, "train_steps": 10_000,
        "description": "ViT-S/32, E=8, K=2, Last 2, 300 Epochs",
        "optimizer.learning_rate.peak_value": 0.003, "optimizer.learning_rate.warmup_steps": 500,
        "dataset.train.prefetch": 16, "dataset.train.prefetch_device": 1,
        "dataset.val.prefetch": 1, "dataset.imagenet_v2.prefetch_device": 1,
        "dataset.test_real.name": "imagenet2012_real",
        "model.hidden_size": 512, "model.encoder.moe.layers": (5, 7),
        "model.encoder.moe.group_size": 8 * 145,
        "initialization.prefix": "gs://vmoe_checkpoints/vmoe_s32_last2_ilsvrc2012_randaug_light1",
        "initialization.rules": [("head", ""), ("pre_logits/.*", ""),
                                 ("^(.*/pos_embedding)$", r"params/\1", "vit_zoom"),
                                 ("^(.*)$", r"params/\1")],
    },
    "vmoe_s32_last2_ilsvrc2012_randaug_light1": {
        "loss.name": "sigmoid_xent", "train_epochs": 300,
        "description": "ViT-S/32, E=8, K=2, Last 2, 300 Epochs",
        "optimizer.name": "adam", "optimizer.b1": 0.9, "optimizer.b2": 0.999,
        "optimizer.weight_decay": [(".*/kernel", 0.1)],
        "optimizer.learning_rate.schedule": "warmup_linear_decay",
        "optimizer.learning_rate.peak_value": 3e-3, "optimizer.learning_rate.end_value": 1e-5,
        "optimizer.learning_rate.warmup_steps": 10_000,
        "optimizer.gradient_clip.global_norm": 1.0,
        "model.encoder.moe.dropout_rate": 0.2, "model.encoder.moe.router.dispatcher.capacity_factor": 1.05,
        "model.representation_size": 512, "model.num_classes": 1000,
        "mixup.concentration": 0.2, "mixup.size": 2, "mixup.granularity": "device",
        "dataset.train.batch_size": 8192, "dataset.train.split": "train[:99%]",
        "dataset.train.process": ('decode_jpeg_and_inception_crop(224)|flip_lr|randaug(2, 10)|'
                                  'value_range(-1,1)|onehot(1000, inkey="label", outkey="labels")|'
                                  'keep("image", "labels")'),
        "dataset.test.split": "validation", "dataset.imagenet_v2.name": "imagenet_v2",
        "dataset.imagenet_real.name": "imagenet2012_real",
        "dataset.imagenet_real.process": ('decode|resize_small(256)|central_crop(224)|value_range(-1,1)|'
                                          'onehot(1000, inkey="real_label", outkey="labels")|'
                                          'keep("image", "labels")'),
        "evaluate.model_overrides.encoder.moe.router.dispatcher.capacity_factor": 4.0,
        "extra_rng_keys": ("dropout", "gating", "mixup"), "num_expert_partitions": 8,
    },
}


def _norm(v):
  if isinstance(v, (list, tuple)):
    return tuple(_norm(x) for x in v)
  return v


@pytest.mark.parametrize("name", sorted(TABLE))
def test_config_values_match_the_reference(name):
  mod = importlib.import_module(CFG + name)
  cfg = mod.get_config()
  flat = misc.flatten_dict(cfg.to_dict(), sep=".")
  # tuples / lists of rules are leaves
  for key, want in TABLE[name].items():
    if key in flat:
      got = flat[key]
    else:
      node = cfg
      for part in key.split("."):
        node = node[part]
      got = node.to_dict() if hasattr(node, "to_dict") else node
    assert _norm(got) == _norm(want), (name, key, got, want)


class _Hyper:
  def sweep(self, key, values):
    return [{key: v} for v in values]

  def product(self, sweeps):
    return sweeps


@pytest.mark.parametrize("name", [n for n in TABLE if "_ft_" in n])
def test_finetune_configs_sweep_three_seeds(name):
  mod = importlib.import_module(CFG + name)
  assert mod.get_hyper(_Hyper()) == [{"config.seed": s} for s in range(3)]


def test_soft_moe_common_helpers_match_the_reference():
  from vmoe_b200.projects.soft_moe.configs import common
  adam = common.get_adam_config()
  assert adam.name == "adam" and adam.b1 == 0.9 and adam.b2 == 0.999 and adam.mu_dtype == "float32"
  assert _norm(adam.weight_decay) == (("head/kernel", 3.0), (".*/kernel", 0.03))
  assert adam.gradient_clip.global_norm == 1.0
  lin = common.get_optimizer_linear_config().learning_rate
  assert (lin.schedule, lin.peak_value, lin.end_value, lin.warmup_steps) == \
      ("warmup_linear_decay", 8e-4, 0.0, 10_000)
  rs = common.get_optimizer_rsqrt_config().learning_rate
  assert (rs.schedule, rs.peak_value, rs.warmup_steps, rs.cooldown_steps, rs.timescale) == \
      ("big_vision_rsqrt", 1e-3, 10_000, 50_000, 10_000)
  inet = common.get_imagenet_config(batch_size=512, randaug="randaug(2, 10)")
  assert sorted(inet.keys()) == ["real", "test", "train", "v2", "val"]
  assert inet.train.split == "train[:99%]" and inet.train.cache == "loaded"
  assert inet.train.shuffle_buffer == 250_000 and inet.val.cache == "batched"
  assert inet.train.process == (
      'decode_jpeg_and_inception_crop(224)|flip_lr|randaug(2, 10)|value_range(-1,1)|'
      'onehot(1000, inkey="label", outkey="labels")|keep("image", "labels")')
  assert inet.real.name == "imagenet2012_real" and "ignore_no_labels" in inet.real.process
  assert inet.v2.name == "imagenet_v2" and inet.v2.split == "test"
