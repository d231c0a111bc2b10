"""Dense baselines with the ``(output, metrics)`` interface of the MoE models: a plain Vision
Transformer (a V-MoE without MoE layers) and an MLP-Mixer (reference: ``vmoe/nn/external.py``
wraps the ``vit_jax`` implementations)."""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch
from torch import nn

from vmoe_b200.models import vit_moe


class VisionTransformer(vit_moe.VisionTransformerMoe):
  """ViT: ``transformer`` holds the encoder kwargs (num_layers, mlp_dim, num_heads, ...)."""

  def __init__(self, num_classes: Optional[int], patches: Mapping[str, Any], hidden_size: int,
               transformer: Mapping[str, Any], classifier: str = "token",
               representation_size: Optional[int] = None, deterministic: bool = False,
               head_bias_init: float = 0.0, image_size=224, mesh=None, **kwargs):
    patch = patches["size"] if isinstance(patches, Mapping) else patches
    enc = dict(transformer)
    enc.pop("moe", None)
    super().__init__(num_classes=num_classes, patch_size=tuple(patch), hidden_size=hidden_size,
                     encoder=enc, classifier=classifier, representation_size=representation_size,
                     deterministic=deterministic, head_bias_init=head_bias_init,
                     image_size=image_size, mesh=mesh)

  def forward(self, images):
    out, _ = super().forward(images)
    return out, {}


class _MixerBlock(nn.Module):
  def __init__(self, tokens: int, hidden: int, tokens_mlp_dim: int, channels_mlp_dim: int):
    super().__init__()
    self.LayerNorm_0 = vit_moe.LayerNorm(hidden)
    self.token_mixing = vit_moe.MlpBlock(tokens, tokens_mlp_dim)
    self.LayerNorm_1 = vit_moe.LayerNorm(hidden)
    self.channel_mixing = vit_moe.MlpBlock(hidden, channels_mlp_dim)

  def forward(self, x):
    y = self.LayerNorm_0(x).transpose(1, 2)
    x = x + self.token_mixing(y.contiguous()).transpose(1, 2)
    return self.channel_mixing(self.LayerNorm_1(x), residual=x)


class MlpMixer(nn.Module):
  """MLP-Mixer (https://arxiv.org/abs/2105.01601)."""

  def __init__(self, num_classes: Optional[int], patches: Mapping[str, Any], num_blocks: int,
               hidden_dim: int, tokens_mlp_dim: int, channels_mlp_dim: int,
               deterministic: bool = False, image_size=224, num_channels: int = 3, mesh=None,
               dtype=None):
    super().__init__()
    patch = tuple(patches["size"] if isinstance(patches, Mapping) else patches)
    if isinstance(image_size, int):
      image_size = (image_size, image_size)
    self.patch_size, self.image_size, self.num_channels = patch, tuple(image_size), num_channels
    self.dtype = vit_moe.parse_dtype(dtype)
    tokens = (image_size[0] // patch[0]) * (image_size[1] // patch[1])
    self.stem = vit_moe.Dense(patch[0] * patch[1] * num_channels, hidden_dim)
    self.blocks = nn.ModuleList(
        [_MixerBlock(tokens, hidden_dim, tokens_mlp_dim, channels_mlp_dim) for _ in range(num_blocks)])
    self.pre_head_layer_norm = vit_moe.LayerNorm(hidden_dim)
    self.head = vit_moe.Dense(hidden_dim, num_classes, kernel_init="zeros") if num_classes else None
    self.deterministic = deterministic
    if deterministic:
      self.eval()

  patchify = vit_moe.VisionTransformerMoe.patchify

  def forward(self, images):
    x = self.stem(self.patchify(images))
    for blk in self.blocks:
      x = blk(x)
    x = self.pre_head_layer_norm(x).mean(dim=1)
    if self.head is not None:
      x = self.head(x)
    return x, {}
