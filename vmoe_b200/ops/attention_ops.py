"""Fused softmax attention for short non-causal sequences (ViT: 50-577 tokens)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def supported(q, k, v) -> bool:
  return q.dtype == torch.bfloat16 and q.is_cuda


def attention(q, k, v):
  # TEMPORARY stand-in while the hand-written kernel is being brought up.
  o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
  return o.transpose(1, 2)
