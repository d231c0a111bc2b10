"""Soft MoE paper, contrastive pre-training on LAION-400M: ``get_config('soft-b16')``,
``'ec-l16'``, ``'vit-s14'`` ... (model type - backbone). A two-tower model (the image tower is
the chosen ViT / experts-choice MoE / Soft MoE at 256 px, the text tower a B-size transformer
over 16 sentencepiece tokens) trained with the sigmoid contrastive loss, batch 16384, rsqrt
schedule with 20k warm-up and cool-down steps, 750k steps, plus few-shot, retrieval and
zero-shot evaluation every 10k steps (reference:
``vmoe/projects/soft_moe/configs/pretrain_laion.py``). Append ``,synthetic`` to the model
string to train on synthetic image / token pairs of the same shapes."""
from vmoe_b200.projects.soft_moe.configs import common
from vmoe_b200.utils.config_dict import ConfigDict

BATCH_SIZE = 16_384
DATASET = "laion400m"


def get_default_moe_num_experts_and_last_n(variant: str, patch_size: int):
  num_experts = {("S", 16): 128, ("S", 14): 256, ("B", 16): 128, ("L", 16): 128,
                 ("H", 14): 256}[(variant, patch_size)]
  return num_experts, {"S": 6, "B": 6, "L": 12, "H": 16}[variant]


def tokenize(inkey: str, outkey: str = "text") -> str:
  return (f'tokenize(max_len=16, model="c4_en", eos="sticky", inkey="{inkey}", '
          f'outkey="{outkey}", pad_value=1)')


def get_config(model: str = "soft-s16") -> ConfigDict:
  synthetic = model.endswith(",synthetic")
  model = model.split(",")[0]
  model_type, backbone = model.split("-")
  patch_size, variant = int(backbone[1:]), backbone[0].upper()
  # Soft MoEs benefit from augmentation; ViTs and experts-choice MoEs do worse with it.
  process_str = ("decode|resize(256)" if model_type in ("vit", "ec")
                 else "decode_jpeg_and_inception_crop(256)")
  config = common.get_base_config()
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = common.get_data_config(
      name=DATASET, split="full[16384:]", batch_size=BATCH_SIZE,
      process=(f'{process_str}|value_range(-1,1)|flatten|{tokenize("text")}|'
               'keep("image", "text")'),
      shuffle_buffer=250_000)
  if synthetic:
    d = config.dataset.train
    d.name, d.split, d.image_size, d.text_len, d.vocab_size = "synthetic_text", "train", 256, 16, 32_000
    d.process = 'value_range(-1,1)|keep("image", "text")'
  else:
    config.fewshot = common.get_fewshot_config(
        batch_size=1_024, resize_resolution=292, target_resolution=256, every_steps=10_000,
        seeds_per_step=3)
    config.fewshot.model_overrides = ConfigDict(type_safe=False)
    config.retrieval = ConfigDict({
        "batch_size": 1_024,
        "every_steps": 10_000,
        "datasets": {
            "coco": {"dataset": "coco_captions", "txt_name": ("captions", "text"),
                     "pp_img": "resize(256)|value_range(-1, 1)",
                     "pp_txt": tokenize(inkey="texts", outkey="labels")},
            "flickr": {"dataset": "argus:flickr30k/captions", "txt_name": "texts",
                       "pp_img": "resize(256)|value_range(-1, 1)",
                       "pp_txt": tokenize(inkey="texts", outkey="labels")},
        }}, type_safe=False)
    config.zeroshot = ConfigDict({
        "batch_size": 1_024,
        "every_steps": 10_000,
        "pp_img": "resize(256)|value_range(-1, 1)",
        "pp_txt": tokenize(inkey="texts", outkey="labels"),
        "datasets": {"cifar100": {},
                     "imagenet2012": {"class_names": "clip", "split": "validation"},
                     "oxford_iiit_pet": {}},
    }, type_safe=False)
  config.optimizer = common.get_optimizer_rsqrt_config()
  config.optimizer.weight_decay = ((".*/kernel", 0.1),)
  config.optimizer.learning_rate.warmup_steps = 20_000
  config.optimizer.learning_rate.cooldown_steps = 20_000
  config.train_steps = 750_000
  config.model = ConfigDict({
      "name": "vmoe_b200.projects.contrastive.models.TwoTower",
      "bias_init": -10.0,
      "scale_init": 10.0,
  }, type_safe=False)
  if model_type == "vit":
    config.model.image = common.get_vit_config(variant, patch_size, None)
  elif model_type == "ec":
    e, last_n = get_default_moe_num_experts_and_last_n(variant, patch_size)
    config.model.image = common.get_vmoe_experts_choose_config(
        variant, patch_size, None, image_size=256, num_experts=e, last_n=last_n,
        capacity_factor=1.0)
  elif model_type == "soft":
    e, last_n = get_default_moe_num_experts_and_last_n(variant, patch_size)
    config.model.image = common.get_vmoe_soft_router_config(
        variant, patch_size, None, image_size=256, num_experts=e, last_n=last_n,
        capacity_factor=None, num_slots=1)
    config.model.image.encoder.moe.router.compute_similarity_metrics = False
  else:
    raise ValueError(f"Unknown model type: {model_type!r}")
  # The text encoder is a B-size transformer.
  config.model.text = ConfigDict({
      "vocab_size": 32_000,
      "num_classes": config.model.image.hidden_size,
      "hidden_size": 768,
      "encoder": {"num_layers": 12, "mlp_dim": 3072, "num_heads": 12, "dropout_rate": 0.0,
                  "attention_dropout_rate": 0.0, "attention_qk_norm": True,
                  "moe": {"layers": ()}},
  }, type_safe=False)
  if model_type == "vit":
    config.num_expert_partitions = 1
    config.params_axis_resources = []
  else:
    config.num_expert_partitions = config.model.image.encoder.moe.num_experts
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
