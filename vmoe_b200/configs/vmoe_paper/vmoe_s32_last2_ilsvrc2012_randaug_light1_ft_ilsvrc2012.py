"""Fine-tuning config ``vmoe_s32_last2_ilsvrc2012_randaug_light1_ft_ilsvrc2012`` of the V-MoE paper
(``vmoe/configs/vmoe_paper/vmoe_s32_last2_ilsvrc2012_randaug_light1_ft_ilsvrc2012.py``); the values live in
``finetune.py`` under the variant ``s32_ilsvrc2012``."""
from vmoe_b200.configs.vmoe_paper import finetune


def get_config():
  return finetune.get_config("s32_ilsvrc2012")


get_hyper = finetune.get_hyper
