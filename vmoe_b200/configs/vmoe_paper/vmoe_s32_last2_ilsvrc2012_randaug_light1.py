"""V-MoE S/32 (8 experts in the last two odd blocks, K=2) trained from scratch on ILSVRC2012
for 300 epochs, batch 8192, RandAugment 'light1' + mixup 0.2 (reference:
``vmoe/configs/vmoe_paper/vmoe_s32_last2_ilsvrc2012_randaug_light1.py``; about 5h50m on
TPUv3-32 there, 76.8 % validation accuracy)."""
from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.utils.config_dict import ConfigDict

NUM_CLASSES = 1_000
BATCH_SIZE = 8192
PP_COMMON = (f'value_range(-1,1)|onehot({NUM_CLASSES}, inkey="label", outkey="labels")|'
             'keep("image", "labels")')


def get_data_params_train(name, split, aug, synthetic=False):
  process = f"decode_jpeg_and_inception_crop(224)|flip_lr|{common.get_randaug(aug)}|{PP_COMMON}"
  cfg = common.get_data_config(name=name, split=split, batch_size=BATCH_SIZE, process=process,
                               shuffle_buffer=50_000)
  cfg.prefetch, cfg.prefetch_device = 16, 1
  if synthetic:
    cfg.name, cfg.split, cfg.num_classes = "synthetic", "train", NUM_CLASSES
    cfg.process = f"flip_lr|{PP_COMMON}"
  return cfg


def get_data_params_eval(name, split, synthetic=False):
  cfg = common.get_data_config(name=name, split=split, batch_size=BATCH_SIZE, cache="batched",
                               process=f"decode|resize_small(256)|central_crop(224)|{PP_COMMON}")
  cfg.prefetch, cfg.prefetch_device = 1, 1
  if synthetic:
    cfg.name, cfg.split, cfg.num_classes = "synthetic", "validation", NUM_CLASSES
    cfg.process = PP_COMMON
  return cfg


def get_config(arg: str = "") -> ConfigDict:
  synthetic = "synthetic" in arg
  config = common.get_base_config()
  config.dataset = ConfigDict(type_safe=False)
  config.dataset.train = get_data_params_train("imagenet2012", "train[:99%]", "light1", synthetic)
  config.dataset.val = get_data_params_eval("imagenet2012", "train[99%:]", synthetic)
  if not synthetic:
    config.dataset.test = get_data_params_eval("imagenet2012", "validation")
    config.dataset.imagenet_v2 = get_data_params_eval("imagenet_v2", "test")
    config.dataset.imagenet_real = common.get_data_config(
        name="imagenet2012_real", split="validation", shuffle_buffer=None, batch_size=BATCH_SIZE,
        cache="batched",
        process=("decode|resize_small(256)|central_crop(224)|value_range(-1,1)|"
                 f'onehot({NUM_CLASSES}, inkey="real_label", outkey="labels")|'
                 'keep("image", "labels")'))
  config.loss = ConfigDict({"name": "sigmoid_xent"})
  config.description = "ViT-S/32, E=8, K=2, Last 2, 300 Epochs"
  config.model = common.get_vmoe_config(config.description, 224, NUM_CLASSES)
  config.model.encoder.moe.dropout_rate = 0.2
  config.optimizer = common.get_optimizer_config(config.description)
  # Different from the standard values of the paper's ImageNet-21k runs.
  config.optimizer.weight_decay = [(".*/kernel", 0.1)]
  config.optimizer.learning_rate.peak_value = 3e-3
  config.optimizer.gradient_clip.global_norm = 1.0
  config.train_epochs = common.get_num_epochs(config.description)
  config.mixup = common.get_mixup_config("light1")
  config.num_expert_partitions = config.model.encoder.moe.num_experts
  config.params_axis_resources = [("Moe/Mlp/.*", ("expert",))]
  config.extra_rng_keys = ("dropout", "gating", "mixup")
  config.evaluate.model_overrides = ConfigDict(
      {"encoder": {"moe": {"router": {"dispatcher": {"capacity_factor": 4.0}}}}}, type_safe=False)
  return config
