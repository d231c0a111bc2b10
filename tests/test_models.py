"""Model families, routers of the projects, contrastive loss, fine-tune initialisation (CPU)."""
import math
import os

import numpy as np
import pytest
import torch

from vmoe_b200 import models as models_lib
from vmoe_b200.checkpoints import flax_layout, partitioned
from vmoe_b200.initialization import initialization
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.projects.contrastive import models as contrastive_models
from vmoe_b200.projects.contrastive import trainer as contrastive_trainer
from vmoe_b200.projects.soft_moe import router as soft_router
from vmoe_b200.projects.sparsity_constrained_ot import ot_routing


def _mesh():
  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  return mesh


def _vmoe_cfg(**moe):
  base = {"num_experts": 4, "layers": (1,), "group_size": 10,
          "router": {"num_selected_experts": 2, "noise_std": 1.0, "importance_loss_weight": 0.01,
                     "load_loss_weight": 0.01,
                     "dispatcher": {"name": "einsum", "capacity_factor": 2.0,
                                    "batch_priority": True}}}
  base.update(moe)
  return {"name": "VisionTransformerMoe", "num_classes": 7, "patch_size": (8, 8),
          "hidden_size": 32, "classifier": "token", "representation_size": None,
          "encoder": {"num_layers": 2, "num_heads": 4, "mlp_dim": 64, "dropout_rate": 0.0,
                      "attention_dropout_rate": 0.0, "moe": base}}


def test_vit_moe_forward_backward_and_metrics():
  mesh = _mesh()
  torch.manual_seed(0)
  model = models_lib.create_model(_vmoe_cfg(), mesh=mesh, image_size=16)
  model.train()
  logits, metrics = model(torch.rand(4, 16, 16, 3) * 2 - 1)
  assert logits.shape == (4, 7)
  aux = metrics["auxiliary_loss"]
  assert torch.as_tensor(aux).numel() >= 1 and torch.isfinite(torch.as_tensor(aux)).all()
  (logits.sum() + torch.as_tensor(aux).mean()).backward()
  grads = [p.grad for p in model.parameters() if p.requires_grad]
  assert all(g is not None for g in grads)
  assert any(float(g.abs().sum()) > 0 for g in grads)


def test_ensemble_model_repeats_inputs_per_member():
  mesh = _mesh()
  cfg = _vmoe_cfg(ensemble_size=2)
  cfg["name"] = "VisionTransformerMoeEnsemble"
  cfg["encoder"]["moe"]["group_size"] = 20
  cfg["encoder"]["moe"]["router"]["num_selected_experts"] = 1
  model = models_lib.create_model(cfg, deterministic=True, mesh=mesh, image_size=16)
  logits, _ = model(torch.rand(4, 16, 16, 3))
  assert logits.shape == (8, 7)  # batch x members, members of one image adjacent


def test_mlp_mixer_and_dense_vit_return_logits_and_empty_metrics():
  mesh = _mesh()
  mixer = models_lib.create_model(
      {"name": "MlpMixer", "num_classes": 5, "patches": {"size": (8, 8)}, "num_blocks": 2,
       "hidden_dim": 16, "tokens_mlp_dim": 8, "channels_mlp_dim": 32}, mesh=mesh, image_size=16)
  out, metrics = mixer(torch.rand(3, 16, 16, 3))
  assert out.shape == (3, 5) and not metrics
  vit = models_lib.create_model(
      {"name": "VisionTransformer", "num_classes": 5, "patches": {"size": (8, 8)},
       "hidden_size": 16, "classifier": "token", "representation_size": None,
       "transformer": {"num_layers": 2, "mlp_dim": 32, "num_heads": 2, "dropout_rate": 0.0,
                       "attention_dropout_rate": 0.0}}, mesh=mesh, image_size=16)
  out, metrics = vit(torch.rand(3, 16, 16, 3))
  assert out.shape == (3, 5) and not metrics


def test_soft_router_weights_are_convex_combinations():
  torch.manual_seed(0)
  r = soft_router.SoftRouter(num_experts=4, hidden_size=8, num_slots=2,
                             compute_similarity_metrics=True)
  r.eval()
  dispatcher, metrics = r(torch.randn(3, 6, 8))
  inner = dispatcher.dispatcher
  d, c = inner.dispatch_weights, inner.combine_weights
  assert d.shape == c.shape == (3, 6, 4, 2)
  assert torch.allclose(d.sum(dim=1), torch.ones(3, 4, 2), atol=1e-5)       # over tokens
  assert torch.allclose(c.sum(dim=(2, 3)), torch.ones(3, 6), atol=1e-5)     # over slots
  assert float(metrics["auxiliary_loss"]) == 0.0
  assert "mu_similarity_mean" in metrics
  x = torch.randn(3, 6, 8)
  out = dispatcher.combine(dispatcher.dispatch(x))  # identity experts
  assert out.shape == x.shape


def test_ot_plans_have_the_right_marginals():
  torch.manual_seed(0)
  sim = torch.randn(2, 12, 4)
  plan = ot_routing.sinkhorn_plan(sim, maxiter=200)
  assert torch.allclose(plan.sum(-1), torch.ones(2, 12), atol=1e-3)
  assert torch.allclose(plan.sum(-2), torch.full((2, 4), 3.0), atol=1e-2)
  x = torch.randn(5, 7)
  p = ot_routing.projection_simplex(x)
  assert torch.allclose(p.sum(-1), torch.ones(5), atol=1e-5) and (p >= 0).all()
  ps = ot_routing.projection_sparse_simplex(x, 2)
  assert ((ps > 0).sum(-1) <= 2).all() and torch.allclose(ps.sum(-1), torch.ones(5), atol=1e-5)


def test_sigmoid_contrastive_loss_matches_definition():
  torch.manual_seed(0)
  logits = torch.randn(5, 5)
  targets = 2 * torch.eye(5) - 1
  want = -torch.nn.functional.logsigmoid(targets * logits).sum(-1).mean()
  got = contrastive_trainer.sigmoid_loss(logits)
  assert torch.allclose(got.mean(), want, atol=1e-6)


def test_two_tower_logits_shape_and_scale():
  mesh = _mesh()
  image = _vmoe_cfg()
  image.pop("name")
  image["num_classes"] = 12
  text = {"vocab_size": 50, "num_classes": 12, "hidden_size": 16,
          "encoder": {"num_layers": 1, "mlp_dim": 32, "num_heads": 2, "dropout_rate": 0.0,
                      "attention_dropout_rate": 0.0, "moe": {"layers": ()}}}
  model = contrastive_models.TwoTower(image=image, text=text, scale_init=10.0, bias_init=-10.0,
                                      deterministic=True, mesh=mesh, image_size=16)
  logits, metrics = model(torch.rand(4, 16, 16, 3), torch.randint(1, 50, (4, 16)))
  assert logits.shape == (4, 4)
  assert float(metrics["scale"]) == pytest.approx(10.0, rel=1e-5)
  assert float(logits.detach().max()) <= 10.0 - 10.0 + 1e-4  # cosine <= 1 -> s * cos + b <= 0


def test_initialize_from_vmoe_drops_head_and_zooms_position_embedding(tmp_path):
  mesh = _mesh()
  torch.manual_seed(0)
  src = models_lib.create_model(_vmoe_cfg(), mesh=mesh, image_size=16)   # 2x2 patches + cls
  params, specs = flax_layout.to_flax(src)
  prefix = os.path.join(str(tmp_path), "src")
  res = partitioned.save_checkpoint(prefix, {"params": params}, shardings={"params": specs},
                                    mesh=mesh)
  if res is not None:
    res.get()
  cfg = _vmoe_cfg()
  cfg["num_classes"] = 3
  dst = models_lib.create_model(cfg, mesh=mesh, image_size=32)           # 4x4 patches + cls
  before_head = dst.head.weight.detach().clone()
  target, _ = flax_layout.to_flax(dst)
  rules = [("^params/head/.*$", None),
           ("^(.*/pos_embedding)$", r"\1", "vit_zoom"),
           ("^(.*)$", r"\1")]
  new = initialization.initialize_from_vmoe(target={"params": target}, prefix=prefix, rules=rules,
                                            mesh=mesh, raise_if_target_unmatched=False)
  flax_layout.from_flax(dst, new["params"], mesh=mesh)
  assert torch.equal(dst.head.weight, before_head)                        # dropped -> untouched
  assert dst.Encoder.posembed_input.pos_embedding.shape == (1, 17, 32)
  src_cls = src.Encoder.posembed_input.pos_embedding[0, 0]
  assert torch.allclose(dst.Encoder.posembed_input.pos_embedding[0, 0], src_cls, atol=1e-6)
  a = src.Encoder.encoderblock_0.SelfAttention.qkv.weight
  b = dst.Encoder.encoderblock_0.SelfAttention.qkv.weight
  assert torch.allclose(a, b)


def test_forward_flop_count_of_a_tiny_vit_moe():
  from vmoe_b200.utils import misc
  mesh = _mesh()
  model = models_lib.create_model(_vmoe_cfg(), mesh=mesh, image_size=16)
  b, t, h, m, classes = 4, 5, 32, 64, 7
  rows = b * t
  embed = 2 * b * 4 * (8 * 8 * 3) * h
  attn = 2 * (2 * rows * h * 3 * h + 4 * b * 4 * t * t * (h // 4) + 2 * rows * h * h)
  dense_mlp = 2 * rows * 2 * h * m
  # MoE block: 2 groups of 10 tokens, 4 experts, K=2, capacity factor 2 -> C = 10 (-> mult of 4: 12)
  from vmoe_b200 import moe
  cap = moe.compute_capacity(10 * 2, 4, 2.0, "ceil", 4)
  moe_mlp = 2 * (2 * 4 * cap) * 2 * h * m + 2 * rows * h * 4
  head = 2 * b * h * classes
  want = embed + attn + dense_mlp + moe_mlp + head
  got = misc.count_forward_flops(model, torch.rand(b, 16, 16, 3))
  assert got == pytest.approx(want, rel=1e-6), (got, want)
  flops, secs = misc.get_flops_and_seconds_per_device(model, torch.rand(b, 16, 16, 3))
  assert flops == pytest.approx(3 * want) and secs == pytest.approx(flops / 1.418e15)
