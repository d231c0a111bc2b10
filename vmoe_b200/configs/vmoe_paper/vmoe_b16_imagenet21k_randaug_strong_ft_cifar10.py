"""Fine-tuning config ``vmoe_b16_imagenet21k_randaug_strong_ft_cifar10`` of the V-MoE paper
(``vmoe/configs/vmoe_paper/vmoe_b16_imagenet21k_randaug_strong_ft_cifar10.py``); the values live in
``finetune.py`` under the variant ``b16_cifar10``."""
from vmoe_b200.configs.vmoe_paper import finetune


def get_config():
  return finetune.get_config("b16_cifar10")


get_hyper = finetune.get_hyper
