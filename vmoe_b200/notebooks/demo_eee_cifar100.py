"""E^3 (efficient ensemble of experts) inference demo on CIFAR-100, as a script.

Builds ``VisionTransformerMoeEnsemble`` (S/32, 8 experts in blocks 5 and 7, two ensemble
members of four experts each) from a plain dict, restores a fine-tuned checkpoint in the
sharded ``.index`` / ``.data-*`` format with ``tree=None``, evaluates the test split and
combines the members by averaging their probabilities: logits come out as
``(batch * members, classes)`` with the members of one image adjacent (inputs are repeated,
not tiled), so they are reshaped to ``(batch, members, classes)``
(counterpart of ``vmoe/notebooks/demo_eee_CIFAR100.ipynb``; the released checkpoint
``eee_s32_last2_ilsvrc2012_ft_cifar100`` reaches 81.26 %).

  python -m vmoe_b200.notebooks.demo_eee_cifar100 --checkpoint <prefix> \
      [--dataset cifar100 --data_dir <dir with the dataset>] [--batch_size 1024]

Without ``--checkpoint`` the model keeps its random initialisation and, without a dataset on
disk, ``--dataset synthetic`` produces random images: the script then only demonstrates the
API.
"""
from __future__ import annotations

import argparse
import math

import torch

NUM_CLASSES = 100
IMAGE_SIZE = 128
PATCH_SIZE = 32
NUM_LAYERS = 8
NUM_EXPERTS = 8
NUM_SELECTED_EXPERTS = 1
ENSEMBLE_SIZE = 2


def model_config(batch_size: int, num_devices: int = 8) -> dict:
  tokens_per_image = (IMAGE_SIZE // PATCH_SIZE) ** 2 + 1
  group_size_per_member = max(batch_size // num_devices, 1) * tokens_per_image
  return {
      "name": "VisionTransformerMoeEnsemble",
      "num_classes": NUM_CLASSES,
      "patch_size": (PATCH_SIZE, PATCH_SIZE),
      "hidden_size": 512,
      "classifier": "token",
      "representation_size": 512,
      "head_bias_init": -10.0,
      "encoder": {
          "num_layers": NUM_LAYERS,
          "num_heads": 8,
          "mlp_dim": 2048,
          "dropout_rate": 0.0,
          "attention_dropout_rate": 0.0,
          "moe": {
              "ensemble_size": ENSEMBLE_SIZE,
              "num_experts": NUM_EXPERTS,
              "group_size": group_size_per_member * ENSEMBLE_SIZE,
              "layers": (5, 7),
              "dropout_rate": 0.0,
              "router": {
                  "num_selected_experts": NUM_SELECTED_EXPERTS,
                  "noise_std": 1.0,  # divided by the number of experts inside the router
                  "importance_loss_weight": 0.005,
                  "load_loss_weight": 0.005,
                  "dispatcher": {
                      "name": "einsum",
                      "bfloat16": True,
                      # A balanced router sends group_size / num_experts tokens to each
                      # expert; 1.5x that leaves slack for imbalance.
                      "capacity_factor": 1.5,
                      "batch_priority": False,
                      "partition_spec": (("expert", "replica"),),
                  },
              },
          },
      },
  }


def ensemble_log_probs(logits: torch.Tensor, ensemble_size: int) -> torch.Tensor:
  """``(batch * members, classes)`` -> log of the member-averaged probabilities."""
  logits = logits.float().reshape(-1, ensemble_size, logits.shape[-1])
  log_p = torch.log_softmax(logits, dim=-1)
  return torch.logsumexp(log_p, dim=1) - math.log(ensemble_size)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--checkpoint", default=None, help="prefix of the .index / .data-* files")
  ap.add_argument("--dataset", default="cifar100")
  ap.add_argument("--data_dir", default=None)
  ap.add_argument("--batch_size", type=int, default=1024)
  ap.add_argument("--max_batches", type=int, default=None)
  args = ap.parse_args()

  from vmoe_b200 import models
  from vmoe_b200.checkpoints import flax_layout, partitioned
  from vmoe_b200.data import input_pipeline
  from vmoe_b200.parallel import mesh as mesh_lib

  mesh = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(mesh)
  device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
  model = models.create_model(model_config(args.batch_size), deterministic=True, mesh=mesh,
                              image_size=IMAGE_SIZE).to(device)
  model.eval()
  if args.checkpoint:
    checkpoint = partitioned.restore_checkpoint(prefix=args.checkpoint, tree=None, mesh=mesh)
    flax_layout.from_flax(model, checkpoint.get("params", checkpoint), mesh=mesh)

  extra = {"data_dir": args.data_dir} if args.data_dir else {}
  if args.dataset.startswith("synthetic"):
    extra.update(image_size=IMAGE_SIZE, num_classes=NUM_CLASSES, num_eval_examples=2048)
  dataset = input_pipeline.get_dataset(
      variant="test", name=args.dataset, split="test" if not extra.get("image_size") else "validation",
      batch_size=args.batch_size,
      process=f'keep("image", "label")|decode|resize({IMAGE_SIZE}, inkey="image")|value_range(-1,1)',
      **extra)
  ncorrect = ntotal = 0
  with torch.no_grad():
    for i, batch in enumerate(dataset):
      if args.max_batches is not None and i >= args.max_batches:
        break
      mask = torch.as_tensor(batch["__valid__"]).to(device)
      images = torch.as_tensor(batch["image"]).to(device)
      labels = torch.as_tensor(batch["label"]).to(device)
      logits, _ = model(images)  # (batch * ENSEMBLE_SIZE, NUM_CLASSES)
      preds = ensemble_log_probs(logits, ENSEMBLE_SIZE).argmax(dim=1)
      ncorrect += int(((preds == labels) & mask.bool()).sum())
      ntotal += int(mask.sum())
  print(f"Test accuracy: {ncorrect / max(ntotal, 1) * 100:.2f}%")


if __name__ == "__main__":
  main()
