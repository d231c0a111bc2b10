"""Fine-tuning config ``vmoe_s32_last2_ilsvrc2012_randaug_light1_ft_ilsvrc2012`` of the V-MoE paper
(``vmoe/configs/vmoe_paper/vmoe_s32_last2_ilsvrc2012_randaug_light1_ft_ilsvrc2012.py``); the settings live in ``finetune.py``."""
from vmoe_b200.configs.vmoe_paper import finetune


def get_config():
  return finetune.get_config("s32_ilsvrc2012")


def get_hyper(hyper):
  return finetune.get_hyper(hyper) if hasattr(finetune, "get_hyper") else hyper.product([])
