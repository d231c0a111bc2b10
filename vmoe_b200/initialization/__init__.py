"""Initialisation of train states from V-MoE, ViT and Orbax checkpoints."""
from vmoe_b200.initialization.initialization import (initialize_from_orbax, initialize_from_vit,
                                                     initialize_from_vmoe)
from vmoe_b200.initialization.mapping import map_state_dict
