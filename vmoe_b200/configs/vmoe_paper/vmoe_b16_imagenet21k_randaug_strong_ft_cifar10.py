"""Fine-tuning config ``vmoe_b16_imagenet21k_randaug_strong_ft_cifar10`` of the V-MoE paper
(``vmoe/configs/vmoe_paper/vmoe_b16_imagenet21k_randaug_strong_ft_cifar10.py``); the settings live in ``finetune.py``."""
from vmoe_b200.configs.vmoe_paper import finetune


def get_config():
  return finetune.get_config("b16_cifar10")


def get_hyper(hyper):
  return finetune.get_hyper(hyper) if hasattr(finetune, "get_hyper") else hyper.product([])
