"""Parameter trees of ViT-MoE and its ensemble variant in the checkpoint (Flax) layout, and
forward shapes. Expected trees are those of the reference's tests
(``vmoe/nn/vit_moe_test.py:146-245``, ``vmoe/nn/vit_moe_ensemble_test.py:30-98``)."""
import copy

import pytest
import torch

from vmoe_b200.checkpoints import flax_layout
from vmoe_b200.models import vit_moe
from vmoe_b200.models import vit_moe_ensemble
from vmoe_b200.utils.misc import flatten_dict, unflatten_dict

CONFIG = {
    "num_classes": 4, "patch_size": (2, 2), "hidden_size": 8, "image_size": 4,
    "encoder": {
        "num_layers": 2, "mlp_dim": 16, "num_heads": 2,
        "moe": {
            "layers": (1,), "num_experts": 4, "group_size": 4,
            "router": {
                "num_selected_experts": 1, "noise_std": 1e-3,
                "importance_loss_weight": 0.02, "load_loss_weight": 0.02,
                "dispatcher": {"name": "einsum", "capacity": 2, "batch_priority": False,
                               "bfloat16": False},
            },
        },
        "dropout_rate": 0.0, "attention_dropout_rate": 0.0,
    },
    "classifier": "gap", "representation_size": None,
}
ATTENTION = {
    "key": {"bias": (2, 4), "kernel": (8, 2, 4)},
    "out": {"bias": (8,), "kernel": (2, 4, 8)},
    "query": {"bias": (2, 4), "kernel": (8, 2, 4)},
    "value": {"bias": (2, 4), "kernel": (8, 2, 4)},
}
MLP = {"Dense_0": {"bias": (16,), "kernel": (8, 16)}, "Dense_1": {"bias": (8,), "kernel": (16, 8)}}
MOE = {"Dense_0": {"bias": (4, 16), "kernel": (4, 8, 16)},
       "Dense_1": {"bias": (4, 8), "kernel": (4, 16, 8)}}
NORM = {"bias": (8,), "scale": (8,)}


def _shapes(model):
  flat = flax_layout.flax_shapes(model)
  flat = flatten_dict(flat, sep="/") if any(isinstance(v, dict) for v in flat.values()) else flat
  return unflatten_dict({k: tuple(v[0]) for k, v in flat.items()}, sep="/")


def _expected(router_kernel=(8, 4), learned_posemb=True, seq_len=4):
  encoder = {
      "encoder_norm": NORM,
      "encoderblock_0": {"LayerNorm_0": NORM, "LayerNorm_1": NORM, "SelfAttention": ATTENTION,
                         "Mlp": MLP},
      "encoderblock_1": {"LayerNorm_0": NORM, "LayerNorm_1": NORM, "SelfAttention": ATTENTION,
                         "Moe": {"Mlp": MOE, "Router": {"dense": {"kernel": router_kernel}}}},
  }
  if learned_posemb:
    encoder["posembed_input"] = {"pos_embedding": (1, seq_len, 8)}
  return {"Encoder": encoder, "embedding": {"bias": (8,), "kernel": (2, 2, 3, 8)},
          "head": {"bias": (4,), "kernel": (8, 4)}}


@pytest.mark.parametrize("position_emb", [{}, {"name": "sincos2d"}])
def test_vit_moe_parameter_tree(position_emb):
  config = copy.deepcopy(CONFIG)
  config["encoder"]["position_emb"] = position_emb
  model = vit_moe.VisionTransformerMoe(**config)
  assert _shapes(model) == _expected(learned_posemb=not position_emb)


@pytest.mark.parametrize("classifier, seq_len, extra", [
    ("map", 4, {"MapHead": {"probe": (1, 1, 8), "MultiHeadDotProductAttention": ATTENTION,
                            "LayerNorm": NORM, "Mlp": MLP}}),
    ("gap", 4, {}),
    ("token", 5, {}),
])
def test_classifier_variants(classifier, seq_len, extra):
  config = copy.deepcopy(CONFIG)
  config["classifier"] = classifier
  model = vit_moe.VisionTransformerMoe(**config)
  shapes = _shapes(model)
  assert shapes["Encoder"]["posembed_input"] == {"pos_embedding": (1, seq_len, 8)}
  if classifier == "token":
    assert shapes.pop("cls") == (1, 1, 8)
  expected = _expected(seq_len=seq_len)
  expected.update(extra)
  assert shapes == expected
  logits, metrics = model(torch.randn(16, 4, 4, 3))
  assert logits.shape == (16, 4) and "auxiliary_loss" in metrics


def test_moe_dropout_depends_on_the_seed():
  config = copy.deepcopy(CONFIG)
  config["encoder"]["moe"]["dropout_rate"] = 0.2
  model = vit_moe.VisionTransformerMoe(**config, deterministic=False)
  with torch.no_grad():
    model.head.weight.normal_()
  model.train()
  x = torch.randn(16, 4, 4, 3)
  outs = []
  for seed in (2, 3):
    torch.manual_seed(seed)
    outs.append(model(x)[0])
  assert (outs[0] - outs[1]).abs().sum() > 0.01


@pytest.mark.parametrize("members, router_kernel", [(1, (8, 1, 4)), (2, (8, 2, 2))])
def test_ensemble_parameter_tree(members, router_kernel):
  config = copy.deepcopy(CONFIG)
  config["encoder"]["moe"]["ensemble_size"] = members
  config["encoder"]["moe"]["group_size"] *= members
  model = vit_moe_ensemble.VisionTransformerMoeEnsemble(**config)
  assert _shapes(model) == _expected(router_kernel=router_kernel)


@pytest.mark.parametrize("members, layers, rows", [(2, (1,), 32), (2, (5, 7), 32), (2, (), 16),
                                                   (1, (1,), 16)])
def test_ensemble_forward_shapes(members, layers, rows):
  config = copy.deepcopy(CONFIG)
  if layers:
    config["encoder"]["num_layers"] = max(layers) + 1
  config["encoder"]["moe"]["layers"] = layers
  config["encoder"]["moe"]["ensemble_size"] = members
  config["encoder"]["moe"]["group_size"] *= members
  model = vit_moe_ensemble.VisionTransformerMoeEnsemble(**config)
  logits, metrics = model(torch.randn(16, 4, 4, 3))
  assert logits.shape == (rows, 4) and "auxiliary_loss" in metrics
