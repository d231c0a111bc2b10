"""Two-tower image/text models for contrastive (SigLIP-style) training.

``TextTransformer``: token embedding -> ``EncoderMoe`` (learned position embeddings, optional
MoE blocks) -> pooling (``last | first | gap | gmp | map``) -> optional head.
``TwoTower``: image tower (any model of the registry) and text tower; both outputs are
L2-normalised and ``logits = exp(s) * zimg @ ztxt^T + b`` with learned scalars ``s`` (init
``log(scale_init)``) and ``b`` (reference: ``vmoe/projects/contrastive/models.py:32-186``).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Mapping, Optional

import torch
from torch import nn

from vmoe_b200.models import vit_moe
from vmoe_b200.utils.misc import parse_call


class TextTransformer(nn.Module):

  def __init__(self, vocab_size: int, num_classes: Optional[int], hidden_size: int,
               encoder: Mapping[str, Any], pool_type: str = "last", deterministic: bool = False,
               head_bias_init: float = 0.0, head_kernel_zero_init: bool = False,
               max_len: int = 16, mesh=None):
    super().__init__()
    if pool_type not in ("last", "first", "gap", "gmp", "map"):
      raise NotImplementedError(f"Cannot do pooling {pool_type!r}")
    enc = dict(encoder)
    if dict(enc.get("position_emb") or {}).get("name") == "sincos2d":
      raise ValueError("sincos2d position embeddings are not supproted for text.")
    self.pool_type = pool_type
    self.dtype = vit_moe.parse_dtype(enc.get("dtype"))
    self.Embed_0 = nn.Embedding(vocab_size, hidden_size)
    nn.init.normal_(self.Embed_0.weight, std=1.0 / math.sqrt(hidden_size))
    self.Encoder = vit_moe.EncoderMoe(hidden_size=hidden_size, seq_len=max_len, mesh=mesh, **enc)
    if pool_type == "map":
      self.MapHead = vit_moe.MapHead(hidden_size, enc["mlp_dim"], enc["num_heads"],
                                     qk_norm=enc.get("attention_qk_norm", False))
    self.head = vit_moe.Dense(
        hidden_size, num_classes, kernel_init="zeros" if head_kernel_zero_init else "lecun_normal",
        bias_init=head_bias_init) if num_classes else None
    self.deterministic = deterministic
    if deterministic:
      self.eval()

  def train(self, mode: bool = True):
    return super().train(mode and not self.deterministic)

  def apply_pooling(self, x):
    if self.pool_type == "last":
      return x[:, -1, :]
    if self.pool_type == "first":
      return x[:, 0, :]
    if self.pool_type == "gap":
      return x.mean(dim=1)
    if self.pool_type == "gmp":
      return x.amax(dim=1)
    return self.MapHead(x)

  def forward(self, text: torch.Tensor):
    x = self.Embed_0(text.long())
    if self.dtype is not None:
      x = x.to(self.dtype)
    x, metrics = self.Encoder(x)
    x = self.apply_pooling(x)
    if self.head is not None:
      return self.head(x), metrics
    return x, metrics


def _registry() -> Dict[str, Any]:
  from vmoe_b200 import models as models_lib
  reg = dict(models_lib.registry())
  reg["TextTransformer"] = TextTransformer
  return reg


class TwoTower(nn.Module):

  def __init__(self, image: Mapping[str, Any], text: Mapping[str, Any], scale_init: float = 1.0,
               bias_init: Optional[float] = None, deterministic: bool = False, mesh=None,
               image_size=224, **_):
    super().__init__()
    self.img = self._build(image, "VisionTransformerMoe", deterministic, mesh,
                           image_size=image_size)
    self.txt = self._build(text, "TextTransformer", deterministic, mesh)
    self.s = nn.Parameter(torch.tensor(math.log(scale_init), dtype=torch.float32))
    self.b = nn.Parameter(torch.tensor(float(bias_init))) if bias_init is not None else None
    self.deterministic = deterministic
    self.last_embeddings: Dict[str, torch.Tensor] = {}

  @staticmethod
  def _build(cfg, default_name, deterministic, mesh, **extra):
    cfg = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(cfg)
    cls, args, kwargs = parse_call(cfg.pop("name", default_name), _registry())
    kwargs.update(cfg)
    kwargs.update(extra)
    return cls(*args, deterministic=deterministic, mesh=mesh, **kwargs)

  def embed_pair(self, images: torch.Tensor, texts: torch.Tensor):
    """``(zimg, ztxt, scale, bias, metrics)``: the normalised embeddings of both towers and the
    logit scale / bias, for losses that build their own logits (global-batch contrast)."""
    zimg, mi = self.img(images)
    ztxt, mt = self.txt(texts)
    zimg, ztxt = zimg.float(), ztxt.float()
    zimg = zimg / (zimg.norm(dim=-1, keepdim=True) + 1e-8)
    ztxt = ztxt / (ztxt.norm(dim=-1, keepdim=True) + 1e-8)
    self.last_embeddings["zimg"], self.last_embeddings["ztxt"] = zimg.detach(), ztxt.detach()
    s = torch.exp(self.s)
    return zimg, ztxt, s, self.b, {"img": mi, "txt": mt, "scale": s.detach()}

  def forward(self, images: Optional[torch.Tensor], texts: Optional[torch.Tensor]):
    if images is None and texts is None:
      raise ValueError("You must give at least one of images or texts arrays.")
    zimg = ztxt = None
    metrics: Dict[str, Any] = {}
    if images is not None:
      zimg, metrics["img"] = self.img(images)
      zimg = zimg.float()
      zimg = zimg / (zimg.norm(dim=-1, keepdim=True) + 1e-8)
      self.last_embeddings["zimg"] = zimg.detach()
    if texts is not None:
      ztxt, metrics["txt"] = self.txt(texts)
      ztxt = ztxt.float()
      ztxt = ztxt / (ztxt.norm(dim=-1, keepdim=True) + 1e-8)
      self.last_embeddings["ztxt"] = ztxt.detach()
    if images is None:
      return ztxt, metrics
    if texts is None:
      return zimg, metrics
    s = torch.exp(self.s)
    logits = zimg @ ztxt.transpose(-1, -2) * s
    metrics["scale"] = s.detach()
    if self.b is not None:
      logits = logits + self.b
    return logits, metrics
