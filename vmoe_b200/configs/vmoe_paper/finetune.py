"""Fine-tuning configs of the V-MoE paper: a released checkpoint is mapped onto a model at a
new resolution / label space with initialization rules (head dropped, position embeddings
resized), then trained with SGD momentum 0.9, gradient clipping and cosine decay.

``get_config('<name>')`` with name in: ``s32_ilsvrc2012`` (S/32 -> ILSVRC2012 @384, 10k steps,
batch 1024), ``b16_ilsvrc2012`` (B/16 I21k -> ILSVRC2012 @384), ``b16_cifar10`` (B/16 I21k ->
CIFAR-10 @128, 1k steps) (reference: the ``*_ft_*.py`` files of ``vmoe/configs/vmoe_paper``).
"""
from vmoe_b200.configs import common_fewshot
from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.utils.config_dict import ConfigDict

_VARIANTS = {
    "s32_ilsvrc2012": dict(desc="ViT-S/32, E=8, K=2, Last 2", ckpt="vmoe_s32_last2_ilsvrc2012_randaug_light1",
                           dataset="imagenet2012", classes=1000, size=384, steps=10_000, batch=1024,
                           train_split="train[:99%]", val_split="train[99%:]", lr=0.03),
    "b16_ilsvrc2012": dict(desc="ViT-B/16, E=8, K=2, Every 2", ckpt="vmoe_b16_imagenet21k_randaug_strong",
                           dataset="imagenet2012", classes=1000, size=384, steps=10_000, batch=1024,
                           train_split="train[:99%]", val_split="train[99%:]", lr=0.003),
    "b16_cifar10": dict(desc="ViT-B/16, E=8, K=2, Every 2", ckpt="vmoe_b16_imagenet21k_randaug_strong",
                        dataset="cifar10", classes=10, size=128, steps=1_000, batch=1024,
                        train_split="train[:98%]", val_split="train[98%:]", lr=0.001),
}


def get_config(arg: str = "b16_ilsvrc2012") -> ConfigDict:
  v = _VARIANTS[arg]
  pp = (f'value_range(-1,1)|onehot({v["classes"]}, inkey="label", outkey="labels")|'
        'keep("image", "labels")')
  config = common.get_base_config()
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = common.get_data_config(
      name=v["dataset"], split=v["train_split"], batch_size=v["batch"], shuffle_buffer=50_000,
      process=f'decode|inception_crop({v["size"]})|flip_lr|{pp}')
  config.dataset.val = common.get_data_config(
      name=v["dataset"], split=v["val_split"], batch_size=v["batch"], cache="batched",
      process=f'decode|resize({v["size"]})|{pp}')
  config.loss = ConfigDict({"name": "softmax_xent"})
  config.description = v["desc"]
  config.model = common.get_vmoe_config(v["desc"], v["size"], v["classes"])
  config.model.representation_size = None
  config.model.head_bias_init = 0.0
  # Routing groups of one image and a generous capacity at fine-tuning time.
  config.model.encoder.moe.router.dispatcher.capacity_factor = 1.5
  config.optimizer = ConfigDict({
      "name": "sgd", "momentum": 0.9, "gradient_clip": {"global_norm": 10.0},
      "learning_rate": {"schedule": "warmup_cosine_decay", "peak_value": v["lr"],
                        "end_value": 1e-5, "warmup_steps": 500},
  }, type_safe=False)
  config.train_steps = v["steps"]
  config.initialization = ConfigDict({
      "name": "initialize_from_vmoe",
      "prefix": f'gs://vmoe_checkpoints/{v["ckpt"]}',
      "rules": [("head", ""), ("^(.*/pos_embedding)$", r"params/\1", "vit_zoom"),
                ("^(.*)$", r"params/\1")],
      "raise_if_target_unmatched": False,
      "axis_resources_regexes": [("Moe/Mlp/.*", ("expert",))],
  }, type_safe=False)
  config.num_expert_partitions = config.model.encoder.moe.num_experts
  config.params_axis_resources = [("Moe/Mlp/.*", ("expert",))]
  config.extra_rng_keys = ("dropout", "gating")
  config.fewshot = None
  config.save_checkpoint.every_steps = 1_000
  config.evaluate.every_steps = 1_000
  return config


get_fewshot = common_fewshot.get_fewshot
