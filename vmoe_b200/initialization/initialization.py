"""Initialise (part of) a train state from an existing checkpoint.

Three sources, as in the reference (``vmoe/initialization/initialization.py:68-267``):
``initialize_from_vmoe`` (sharded ``.index``/``.data-*`` checkpoints, restored with the
partitioning given by checkpoint-side regexes), ``initialize_from_vit`` (``.npz`` files of
the original ViT release; 2-byte void arrays are reinterpreted as bfloat16) and
``initialize_from_orbax`` (a directory of zarr-v2 arrays as written by Orbax/tensorstore; a
small reader handles uncompressed and zlib/gzip chunks and raises for other codecs).
All of them return the state-dict form of ``target`` produced by ``map_state_dict``; the
target and the result use the Flax parameter layout.
"""
from __future__ import annotations

import gzip
import io
import json
import os
import zlib
from typing import Any, Dict, Mapping, Optional, Sequence

import numpy as np

from vmoe_b200.checkpoints import base as ckpt_base
from vmoe_b200.checkpoints import partitioned
from vmoe_b200.checkpoints import serialization
from vmoe_b200.initialization import mapping
from vmoe_b200.parallel import partitioning
from vmoe_b200.utils.misc import flatten_dict, unflatten_dict

Rules = mapping.Rules

__all__ = ["initialize_from_orbax", "initialize_from_vit", "initialize_from_vmoe"]


def initialize_from_vmoe(*, target, prefix: str, rules, mesh=None,
                         axis_resources_regexes: Optional[Sequence] = None, thread_pool=None,
                         **map_state_dict_kwargs):
  index = ckpt_base.restore_checkpoint(prefix + ".index")
  version = partitioned.Version(index.get("version", None))
  shapes = _tree_map(lambda x: x.global_shape, index["index"])
  if version == partitioned.Version.UNKNOWN:
    target_sd = serialization.to_state_dict(target)
    if set(flatten_dict(target_sd)) != set(flatten_dict(shapes)):
      raise ValueError(
          "Initialization from V-MoE checkpoints created before 2022/06/22 is only possible "
          "when the structure of the checkpoint and target trees match.")
  specs = partitioning.tree_axis_resources_from_regexes(
      tree=shapes, axis_resources_regexes=axis_resources_regexes or ())
  specs = _tree_map(lambda s: tuple(s) if len(s) else None, specs)
  ckpt = partitioned.restore_checkpoint(
      prefix, None if version != partitioned.Version.UNKNOWN else shapes, shardings=specs,
      mesh=mesh, thread_pool=thread_pool)
  return mapping.map_state_dict(ckpt, target, rules, **map_state_dict_kwargs)


def _tree_map(fn, tree):
  if isinstance(tree, Mapping):
    return {k: _tree_map(fn, v) for k, v in tree.items()}
  return fn(tree)


def load_vit_npz(filepath: str) -> Dict[str, Any]:
  """Reads a ViT ``.npz`` checkpoint: keys are '/'-joined parameter paths."""
  with open(filepath, "rb") as f:
    data = np.load(io.BytesIO(f.read()), allow_pickle=False)
    flat = {k: data[k] for k in data.files}
  def fix(x):
    if hasattr(x, "dtype") and x.dtype.type is np.void:
      assert x.itemsize == 2, "Unknown dtype!"
      return x.view(serialization.dtype_from_name("bfloat16"))
    return x
  return unflatten_dict({k: fix(v) for k, v in flat.items()}, sep="/")


def initialize_from_vit(*, target, filepath: str, rules, mesh=None,
                        axis_resources_regexes: Optional[Sequence] = None,
                        **map_state_dict_kwargs):
  ckpt = load_vit_npz(filepath)
  return mapping.map_state_dict(ckpt, target, rules, **map_state_dict_kwargs)


# ----------------------------------------------------------------------------- zarr reader
def _read_zarr_array(path: str) -> np.ndarray:
  with open(os.path.join(path, ".zarray")) as fp:
    meta = json.load(fp)
  shape, chunks = tuple(meta["shape"]), tuple(meta["chunks"])
  dtype = np.dtype(meta["dtype"]) if meta["dtype"] != "bfloat16" else \
      serialization.dtype_from_name("bfloat16")
  order = meta.get("order", "C")
  comp = meta.get("compressor")
  sep = meta.get("dimension_separator", ".")
  fill = meta.get("fill_value", 0) or 0
  out = np.full(shape, fill, dtype=dtype)
  grid = [range(-(-s // c)) for s, c in zip(shape, chunks)] if shape else [range(1)]
  import itertools
  for idx in itertools.product(*grid):
    name = sep.join(str(i) for i in idx) if shape else "0"
    fpath = os.path.join(path, *name.split("/"))
    if not os.path.exists(fpath):
      continue
    with open(fpath, "rb") as fp:
      raw = fp.read()
    if comp is not None:
      cid = comp.get("id")
      if cid == "zlib":
        raw = zlib.decompress(raw)
      elif cid == "gzip":
        raw = gzip.decompress(raw)
      else:
        raise NotImplementedError(
            f"zarr compressor {cid!r} is not available in this environment ({path})")
    chunk = np.frombuffer(raw, dtype=dtype).reshape(chunks, order=order) if shape else \
        np.frombuffer(raw, dtype=dtype).reshape(())
    sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, shape))
    out[sl] = chunk[tuple(slice(0, s.stop - s.start) for s in sl)]
  return out


def read_orbax_structure(directory: str) -> Dict[str, Any]:
  """Tree of array paths found under an Orbax checkpoint directory (dirs with ``.zarray``)."""
  flat = {}
  for root, dirs, files in os.walk(directory):
    if ".zarray" in files:
      rel = os.path.relpath(root, directory)
      flat[rel.replace(os.sep, "/").replace(".", "/")] = root
      dirs[:] = []
  return unflatten_dict(flat, sep="/")


def initialize_from_orbax(*, target, directory: str, rules, mesh=None,
                          axis_resources_regexes: Optional[Sequence] = None,
                          **map_state_dict_kwargs):
  structure = read_orbax_structure(directory)
  if not structure:
    raise FileNotFoundError(f"No zarr arrays found under {directory!r}")
  ckpt = _tree_map(_read_zarr_array, structure)
  return mapping.map_state_dict(ckpt, target, rules, **map_state_dict_kwargs)
