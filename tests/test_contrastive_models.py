"""Two-tower model and text tower (reference test: ``vmoe/projects/contrastive/models_test.py``)."""
import math

import pytest
import torch

from vmoe_b200.projects.contrastive import models

OUTPUT_DIM = 32
IMAGE = {"num_classes": OUTPUT_DIM, "patch_size": (4, 4), "hidden_size": 64, "classifier": "gap",
         "encoder": {"num_layers": 2, "mlp_dim": 256, "num_heads": 2},
         "head_kernel_zero_init": True}
TEXT = {"num_classes": OUTPUT_DIM, "hidden_size": 64, "vocab_size": 128,
        "encoder": {"num_layers": 2, "mlp_dim": 256, "num_heads": 2}}


def test_two_tower_parameters_and_outputs():
  batch, size, text_len = 4, 8, 16
  model = models.TwoTower(image=dict(IMAGE), text=dict(TEXT), scale_init=2.0, bias_init=1.0,
                          image_size=size)
  names = {n.split(".")[0] for n, _ in model.named_parameters()}
  assert {"img", "txt", "s", "b"} <= names
  assert model.s.detach().item() == pytest.approx(math.log(2.0)) and model.b.detach().item() == 1.0
  images = torch.zeros(batch, size, size, 3)
  texts = torch.zeros(batch, text_len, dtype=torch.int32)
  logits, _ = model(images, texts)
  assert logits.shape == (batch, batch) and logits.dtype == torch.float32
  # The image head starts at zero, the text head does not.
  zimg, _ = model(images, None)
  assert zimg.shape == (batch, OUTPUT_DIM) and float(zimg.abs().sum()) == 0.0
  ztxt, _ = model(None, texts)
  assert ztxt.shape == (batch, OUTPUT_DIM) and float(ztxt.abs().sum()) > 0.0


@pytest.mark.parametrize("pool_type", ["last", "first", "gap", "gmp", "map"])
def test_text_tower_pooling(pool_type):
  cfg = dict(TEXT)
  model = models.TextTransformer(pool_type=pool_type, max_len=8, **cfg)
  tokens = torch.randint(0, 128, (3, 8), generator=torch.Generator().manual_seed(0))
  out, metrics = model(tokens)
  assert out.shape == (3, OUTPUT_DIM) and "auxiliary_loss" in metrics
  features, _ = models.TextTransformer(pool_type=pool_type, max_len=8,
                                       **{**cfg, "num_classes": None})(tokens)
  assert features.shape == (3, 64)


def test_text_tower_rejects_unknown_pooling_and_2d_position_embeddings():
  with pytest.raises(NotImplementedError):
    models.TextTransformer(pool_type="median", **dict(TEXT))
  cfg = dict(TEXT)
  cfg["encoder"] = dict(cfg["encoder"], position_emb={"name": "sincos2d"})
  with pytest.raises(ValueError):
    models.TextTransformer(**cfg)
