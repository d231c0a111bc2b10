"""Conversion between this package's PyTorch parameters and the reference's Flax parameter
tree (names and array layouts), so checkpoints are interchangeable.

Layouts (Flax side, as pinned by the reference's tests, ``vmoe/nn/vit_moe_test.py:60-75``):
``Dense/kernel (in, out)``; attention ``query|key|value/kernel (hidden, heads, head_dim)``,
``bias (heads, head_dim)``, ``out/kernel (heads, head_dim, hidden)``; patch embedding
``embedding/kernel (ph, pw, C, hidden)``; MLP ``Dense_0/kernel (hidden, mlp)``,
``Dense_1/kernel (mlp, hidden)``; expert MLPs the same with a leading expert axis;
``Router/dense/kernel (hidden, experts)``. The PyTorch side stores GEMM weights as
``[out, in]`` (K-major for the tensor cores), fuses Q/K/V into one ``[3*hidden, hidden]``
weight and gives dense MLPs a leading axis of 1.

Expert-sharded parameters hold only this rank's experts; ``to_flax`` returns those local
blocks together with a ``PartitionSpec`` tree, ``from_flax`` accepts either local blocks or
full arrays (which it slices).
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Tuple

import numpy as np
import torch

from vmoe_b200.checkpoints.serialization import to_numpy, to_torch
from vmoe_b200.utils.misc import flatten_dict, unflatten_dict


def _entries(model: torch.nn.Module):
  """Yields ``(flax_path, parameter, kind, extra)`` for every parameter of the model."""
  from vmoe_b200.models import vit_moe
  claimed = set()
  for mod_name, mod in model.named_modules():
    prefix = mod_name.replace(".", "/")
    join = lambda *p: "/".join(x for x in (prefix,) + p if x)
    if isinstance(mod, vit_moe.MultiHeadDotProductAttention):
      h, d = mod.num_heads, mod.head_dim
      for i, name in enumerate(("query", "key", "value")):
        yield join(name, "kernel"), mod.qkv.weight, "qkv_w", (i, h, d)
        yield join(name, "bias"), mod.qkv.bias, "qkv_b", (i, h, d)
      yield join("out", "kernel"), mod.out.weight, "attn_out_w", (h, d)
      yield join("out", "bias"), mod.out.bias, "same", None
      claimed.update(id(p) for p in (mod.qkv.weight, mod.qkv.bias, mod.out.weight, mod.out.bias))
    elif isinstance(mod, (vit_moe.MlpBlock, vit_moe.ExpertMlp)):
      dense = isinstance(mod, vit_moe.MlpBlock)
      for pn, fn in (("w1", "Dense_0/kernel"), ("b1", "Dense_0/bias"), ("w2", "Dense_1/kernel"),
                     ("b2", "Dense_1/bias")):
        p = getattr(mod, pn)
        kind = ("mlp_w" if pn.startswith("w") else "mlp_b") + ("_dense" if dense else "")
        yield join(fn), p, kind, None
        claimed.add(id(p))
    elif isinstance(mod, vit_moe.Dense):
      if id(mod.weight) in claimed:
        continue
      kind = "dense_w"
      extra = None
      if mod_name.endswith("embedding") and hasattr(model, "patch_size"):
        kind, extra = "embed_w", (tuple(model.patch_size), getattr(model, "num_channels", 3))
      yield join("kernel"), mod.weight, kind, extra
      claimed.add(id(mod.weight))
      if mod.bias is not None:
        yield join("bias"), mod.bias, "same", None
        claimed.add(id(mod.bias))
    elif type(mod).__name__ == "_MemberGating":
      yield join("kernel"), mod.weight, "member_gating_w", None
      claimed.add(id(mod.weight))
    elif isinstance(mod, torch.nn.Linear):
      yield join("kernel"), mod.weight, "dense_w", None
      claimed.add(id(mod.weight))
      if mod.bias is not None:
        yield join("bias"), mod.bias, "same", None
        claimed.add(id(mod.bias))
    elif isinstance(mod, torch.nn.Embedding):
      yield join("embedding"), mod.weight, "same", None
      claimed.add(id(mod.weight))
  for name, p in model.named_parameters():
    if id(p) not in claimed:
      yield name.replace(".", "/"), p, "same", None


def _to_flax_array(p: torch.Tensor, kind: str, extra) -> np.ndarray:
  t = p.detach()
  if kind == "same":
    out = t
  elif kind == "dense_w":
    out = t.t()
  elif kind == "embed_w":
    (ph, pw), c = extra
    out = t.t().reshape(ph, pw, c, t.shape[0])
  elif kind == "qkv_w":
    i, h, d = extra
    hid = t.shape[0] // 3
    out = t[i * hid:(i + 1) * hid].t().reshape(t.shape[1], h, d)
  elif kind == "qkv_b":
    i, h, d = extra
    hid = t.shape[0] // 3
    out = t[i * hid:(i + 1) * hid].reshape(h, d)
  elif kind == "attn_out_w":
    h, d = extra
    out = t.t().reshape(h, d, t.shape[0])
  elif kind == "member_gating_w":
    out = t.permute(2, 0, 1)  # (M, E/M, H) -> (H, M, E/M)
  elif kind == "mlp_w":
    out = t.transpose(1, 2)
  elif kind == "mlp_b":
    out = t
  elif kind == "mlp_w_dense":
    out = t[0].t()
  elif kind == "mlp_b_dense":
    out = t[0]
  else:
    raise ValueError(kind)
  out = out.contiguous()
  if out.device.type == "cpu" and \
      out.untyped_storage().data_ptr() == t.untyped_storage().data_ptr():
    # A CPU parameter would be aliased by the NumPy array; checkpoints are written by
    # background threads while training goes on, so take the snapshot now.
    out = out.clone()
  return to_numpy(out)


def _from_flax_array(value: np.ndarray, p: torch.Tensor, kind: str, extra) -> torch.Tensor:
  v = to_torch(np.asarray(value)) if not isinstance(value, torch.Tensor) else value
  if kind == "same" or kind == "mlp_b":
    return v
  if kind == "dense_w":
    return v.t()
  if kind == "embed_w":
    return v.reshape(-1, v.shape[-1]).t()
  if kind == "qkv_w":
    return v.reshape(v.shape[0], -1).t()
  if kind == "qkv_b":
    return v.reshape(-1)
  if kind == "attn_out_w":
    return v.reshape(-1, v.shape[-1]).t()
  if kind == "member_gating_w":
    return v.permute(1, 2, 0)
  if kind == "mlp_w":
    return v.transpose(1, 2)
  if kind == "mlp_w_dense":
    return v.t().unsqueeze(0)
  if kind == "mlp_b_dense":
    return v.unsqueeze(0)
  raise ValueError(kind)


def to_flax(model: torch.nn.Module) -> Tuple[Dict[str, Any], Dict[str, Any]]:
  """Returns ``(params, specs)``: nested Flax-layout dict of NumPy arrays (local blocks for
  expert-sharded parameters) and a matching tree of partition specs (``('expert',)`` or
  None)."""
  flat, specs = {}, {}
  for path, p, kind, extra in _entries(model):
    flat[path] = _to_flax_array(p, kind, extra)
    specs[path] = ("expert",) if getattr(p, "expert_sharded", False) else None
  return unflatten_dict(flat, sep="/"), unflatten_dict(specs, sep="/")


def flax_shapes(model: torch.nn.Module, mesh=None) -> Dict[str, Any]:
  """Flat dict ``flax_path -> (global shape, numpy dtype)``."""
  out = {}
  for path, p, kind, extra in _entries(model):
    arr = _to_flax_array(p, kind, extra)
    shape = list(arr.shape)
    if getattr(p, "expert_sharded", False) and mesh is not None:
      shape[0] *= mesh.num_partitions
    out[path] = (tuple(shape), arr.dtype)
  return out


@torch.no_grad()
def from_flax(model: torch.nn.Module, params: Mapping[str, Any], mesh=None,
              strict: bool = True) -> None:
  """Loads a (nested or flat) Flax-layout tree into the model's parameters in place."""
  flat = flatten_dict(params, sep="/") if any(isinstance(v, Mapping) for v in params.values()) \
      else dict(params)
  missing = []
  for path, p, kind, extra in _entries(model):
    if path not in flat:
      missing.append(path)
      continue
    value = flat[path]
    value = np.asarray(to_numpy(value))
    if getattr(p, "expert_sharded", False) and mesh is not None and mesh.num_partitions > 1:
      el = p.shape[0]
      if value.shape[0] == el * mesh.num_partitions:  # a full array: keep this rank's experts
        value = value[mesh.expert_rank * el:(mesh.expert_rank + 1) * el]
    t = _from_flax_array(value, p, kind, extra).to(device=p.device, dtype=p.dtype)
    if kind in ("qkv_w", "qkv_b"):
      i = extra[0]
      hid = p.shape[0] // 3
      p.data[i * hid:(i + 1) * hid].copy_(t.reshape(p.data[i * hid:(i + 1) * hid].shape))
    else:
      p.data.copy_(t.reshape(p.shape))
  if strict and missing:
    raise KeyError(f"Parameters missing from the tree: {missing[:8]}{'...' if len(missing) > 8 else ''}")
