"""E^3 (efficient ensemble of experts) S/32, 2 members x 4 experts in the last two odd blocks,
fine-tuned on CIFAR-100 at 128 px for 2000 steps (reference:
``vmoe/configs/eee_paper/eee_s32_last2_ilsvrc2012_ft_cifar100.py``; 81.31 % test there)."""
from vmoe_b200.utils.config_dict import ConfigDict

BATCH_SIZE = 1024
NUM_CLASSES = 100
IMAGE_SIZE = 128
PATCH_SIZE = 32
NUM_LAYERS = 8
NUM_EXPERTS = 8
NUM_SELECTED_EXPERTS = 1
ENSEMBLE_SIZE = 2
NUM_TOKENS_PER_IMAGE = (IMAGE_SIZE // PATCH_SIZE) ** 2 + 1
NUM_DEVICES = 8
GROUP_SIZE_PER_ENS_MEMBER = (BATCH_SIZE // NUM_DEVICES) * NUM_TOKENS_PER_IMAGE


def get_data_params(name, split, process, shuffle_buffer, cache):
  cfg = ConfigDict(type_safe=False)
  cfg.name, cfg.split, cfg.process, cfg.batch_size = name, split, process, BATCH_SIZE
  cfg.prefetch, cfg.prefetch_device = "autotune", 2
  if shuffle_buffer:
    cfg.shuffle_buffer = shuffle_buffer
  if cache:
    cfg.cache = cache
  return cfg


def get_config(arg: str = "") -> ConfigDict:
  config = ConfigDict(type_safe=False)
  pp = (f'value_range(-1,1)|onehot({NUM_CLASSES}, inkey="label", outkey="labels")|'
        'keep("image", "labels")')
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = get_data_params("cifar100", "train[:98%]",
                                         f"decode|inception_crop({IMAGE_SIZE})|flip_lr|{pp}", 50_000, None)
  config.dataset.val = get_data_params("cifar100", "train[98%:]", f"decode|resize({IMAGE_SIZE})|{pp}", None, "batched")
  config.dataset.test = get_data_params("cifar100", "test", f"decode|resize({IMAGE_SIZE})|{pp}", None, "batched")
  config.loss = ConfigDict({"name": "ensemble_softmax_xent", "ensemble_size": ENSEMBLE_SIZE})
  config.description = "EEE-S/32, K=1, M=2, Last 2"
  config.train_steps = 2_000
  config.initialization = ConfigDict({
      "name": "initialize_from_vmoe",
      "prefix": "gs://vmoe_checkpoints/eee_s32_last2_ilsvrc2012",
      "rules": [("head", ""), ("^(.*/pos_embedding)$", r"params/\1", "vit_zoom"),
                ("^(.*/Moe/Router/dense/.*)$", r"params/\1", "reshape"), ("^(.*)$", r"params/\1")],
      "raise_if_target_unmatched": False,
      "axis_resources_regexes": [("Moe/Mlp/.*", ("expert",))],
  }, type_safe=False)
  config.model = ConfigDict({
      "name": "VisionTransformerMoeEnsemble",
      "num_classes": NUM_CLASSES,
      "patch_size": (PATCH_SIZE, PATCH_SIZE),
      "hidden_size": 512,
      "classifier": "token",
      "representation_size": None,
      "head_bias_init": -10.0,
      "encoder": {
          "num_layers": NUM_LAYERS, "mlp_dim": 2048, "num_heads": 8, "dropout_rate": 0.0,
          "attention_dropout_rate": 0.0,
          "moe": {
              "ensemble_size": ENSEMBLE_SIZE,
              "num_experts": NUM_EXPERTS,
              "group_size": GROUP_SIZE_PER_ENS_MEMBER * ENSEMBLE_SIZE,
              "layers": (5, 7),
              "dropout_rate": 0.0,
              "router": {
                  "num_selected_experts": NUM_SELECTED_EXPERTS, "noise_std": 1e-3,
                  "importance_loss_weight": 0.005, "load_loss_weight": 0.005,
                  "dispatcher": {"name": "einsum", "bfloat16": True, "capacity_factor": 1.5,
                                 "batch_priority": False,
                                 "partition_spec": (("expert", "replica"),)},
              },
          },
      },
  }, type_safe=False)
  config.optimizer = ConfigDict({
      "name": "sgd", "momentum": 0.9, "accumulator_dtype": "float32",
      "learning_rate": {"schedule": "warmup_cosine_decay", "peak_value": 0.003, "end_value": 1e-5,
                        "warmup_steps": 200},
      "gradient_clip": {"global_norm": 10.0},
  }, type_safe=False)
  config.num_expert_partitions = NUM_EXPERTS
  config.params_axis_resources = [("Moe/Mlp/.*", ("expert",))]
  config.extra_rng_keys = ("dropout", "gating")
  config.save_checkpoint = ConfigDict({"every_steps": 500, "keep_last": 1, "wait_seconds": 300})
  config.report_progress = ConfigDict({"every_secs": None, "every_steps": 100}, type_safe=False)
  config.evaluate = ConfigDict({"every_steps": 500}, type_safe=False)
  config.seed = 0
  return config
