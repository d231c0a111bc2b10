"""Maps PyTorch parameter names of this package's models to the reference's Flax parameter
paths (slash separated). The paths are what regex options (weight decay, freezing, gradient
scale, partitioning, tree summaries, initialization rules) are matched against, and the keys
of V-MoE checkpoints.

A fused tensor that corresponds to several Flax leaves (the QKV projection) reports the path
of its first leaf (``.../query/...``).
"""
from __future__ import annotations

_LEAF = {
    "weight": "kernel",
    "w1": "Dense_0/kernel", "b1": "Dense_0/bias",
    "w2": "Dense_1/kernel", "b2": "Dense_1/bias",
}


def flax_key(torch_name: str) -> str:
  parts = torch_name.split(".")
  leaf = parts[-1]
  prefix = parts[:-1]
  if prefix and prefix[-1] == "qkv":
    prefix = prefix[:-1] + ["query"]
  leaf = _LEAF.get(leaf, leaf)
  return "/".join(prefix + [leaf])


def named_flax_parameters(module, prefix: str = "params"):
  """Yields ``(flax_path, torch_name, parameter)``; paths start with ``params/`` like the
  train-state keys the reference's regexes see."""
  for name, p in module.named_parameters():
    key = flax_key(name)
    yield (f"{prefix}/{key}" if prefix else key), name, p
