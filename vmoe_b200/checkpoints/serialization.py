"""msgpack (de)serialisation of checkpoint trees, byte-compatible with the reference's format.

Extension codes (``vmoe/checkpoints/serialization.py:149-159``): 1 ndarray, 2 native complex,
3 NumPy scalar, 4 ShapedArray ``(shape, dtype name, weak_type, {})``, 5 Slice, 6 SliceNd,
7 SliceNdArray, 8 IndexInfo. An ndarray payload is the msgpack tuple ``(shape, dtype name, raw
C-order bytes)`` (Flax's layout); arrays above 2**30 bytes are split into a
``{'__msgpack_chunked_array__': True, 'shape': ..., 'chunks': {...}}`` dict. A checkpoint
shard is a dict flagged by ``'__msgpack_array_chunk_a87ca2__'`` mapping the leaf index (as a
string) to ``[[flat sub-chunks], global slice]`` pairs.
"""
from __future__ import annotations

import enum
from typing import Any, Dict, Mapping

import msgpack
import numpy as np

from vmoe_b200.checkpoints.types import (ArrayChunks, IndexInfo, LazyArrayChunks, ShapedArray,
                                         Slice, SliceNd, SliceNdArray)

try:  # bfloat16 and friends as NumPy dtypes
  import ml_dtypes  # noqa: F401
  _EXTRA_DTYPES = {"bfloat16": np.dtype(ml_dtypes.bfloat16)}
  for _n in ("float8_e4m3fn", "float8_e5m2"):
    if hasattr(ml_dtypes, _n):
      _EXTRA_DTYPES[_n] = np.dtype(getattr(ml_dtypes, _n))
except ImportError:  # pragma: no cover
  _EXTRA_DTYPES = {}

MAX_CHUNK_SIZE = 2 ** 30
_ARRAY_CHUNKS_MAGIC_KEY = "__msgpack_array_chunk_a87ca2__"
_CHUNKED_ARRAY_KEY = "__msgpack_chunked_array__"


class _Ext(enum.IntEnum):
  ndarray = 1
  native_complex = 2
  npscalar = 3
  shaped_array = 4
  slice = 5
  slice_nd = 6
  slice_nd_array = 7
  index_info = 8


def dtype_from_name(name) -> np.dtype:
  if isinstance(name, bytes):
    name = name.decode("utf-8")
  if name in _EXTRA_DTYPES:
    return _EXTRA_DTYPES[name]
  return np.dtype(name)


def to_numpy(x) -> np.ndarray:
  """NumPy view/copy of a tensor-like (torch bf16 goes through a uint16 view)."""
  if isinstance(x, np.ndarray):
    return x
  try:
    import torch
    if isinstance(x, torch.Tensor):
      t = x.detach().cpu().contiguous()
      if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(_EXTRA_DTYPES["bfloat16"])
      return t.numpy()
  except ImportError:  # pragma: no cover
    pass
  return np.asarray(x)


def to_torch(x: np.ndarray):
  import torch
  if x.dtype.name == "bfloat16":
    return torch.from_numpy(np.ascontiguousarray(x).view(np.uint16)).view(torch.bfloat16)
  return torch.from_numpy(np.ascontiguousarray(x))


# ------------------------------------------------------------------------------ ndarray
def _ndarray_to_bytes(arr) -> bytes:
  arr = to_numpy(arr)
  if arr.dtype.hasobject or arr.dtype.isalignedstruct:
    raise ValueError("Object and structured dtypes not supported for serialization of ndarrays.")
  return msgpack.packb((arr.shape, arr.dtype.name, arr.tobytes("C")), use_bin_type=True)


def _ndarray_from_bytes(data: bytes) -> np.ndarray:
  shape, dtype_name, buffer = msgpack.unpackb(data, raw=True)
  return np.frombuffer(buffer, dtype=dtype_from_name(dtype_name)).reshape(shape, order="C")


def _chunk(arr: np.ndarray) -> Dict[str, Any]:
  chunksize = max(1, int(MAX_CHUNK_SIZE / arr.dtype.itemsize))
  data = {_CHUNKED_ARRAY_KEY: True, "shape": [int(s) for s in arr.shape]}
  flat = arr.reshape(-1)
  chunks = [flat[i:i + chunksize] for i in range(0, flat.size, chunksize)]
  data["chunks"] = {str(i): c for i, c in enumerate(chunks)}
  return data


def _unchunk(data: Mapping[str, Any]) -> np.ndarray:
  assert _CHUNKED_ARRAY_KEY in data
  shape = tuple(data["shape"])
  flat = np.concatenate([data["chunks"][str(i)] for i in range(len(data["chunks"]))])
  return flat.reshape(shape)


def _prepare(tree):
  """Converts tensors to NumPy and splits oversized arrays (returns a new tree)."""
  if isinstance(tree, Mapping):
    return {k: _prepare(v) for k, v in tree.items()}
  if isinstance(tree, (list, tuple)) and not isinstance(tree, SliceNd):
    return type(tree)(_prepare(v) for v in tree) if not hasattr(tree, "_fields") else tree
  if isinstance(tree, (LazyArrayChunks, ArrayChunks, IndexInfo, Slice, SliceNd, ShapedArray,
                       SliceNdArray)):
    return tree
  mod = type(tree).__module__
  if isinstance(tree, np.ndarray) or mod.startswith("torch"):
    arr = to_numpy(tree)
    if arr.size * arr.dtype.itemsize > MAX_CHUNK_SIZE:
      return _chunk(arr)
    return arr
  return tree


def _restore_chunked(tree):
  if isinstance(tree, Mapping):
    if _CHUNKED_ARRAY_KEY in tree:
      return _unchunk(tree)
    return {k: _restore_chunked(v) for k, v in tree.items()}
  if isinstance(tree, list):
    return [_restore_chunked(v) for v in tree]
  return tree


# ------------------------------------------------------------------------------ custom types
def _shaped_array_to_bytes(x: ShapedArray) -> bytes:
  return msgpack.packb((x.shape, x.dtype.name, x.weak_type, {}), use_bin_type=True)


def _shaped_array_from_bytes(data: bytes) -> ShapedArray:
  shape, dtype_name, weak_type, _ = msgpack.unpackb(data, raw=True)
  return ShapedArray(shape=tuple(shape), dtype=dtype_from_name(dtype_name), weak_type=weak_type)


def _slice_to_bytes(x: Slice) -> bytes:
  return msgpack.packb((x.start, x.stop, x.step), use_bin_type=True)


def _slice_from_bytes(data: bytes) -> Slice:
  start, stop, step = msgpack.unpackb(data, raw=True)
  return Slice(start, stop, step)


def _slice_nd_to_bytes(x: SliceNd) -> bytes:
  return msgpack.packb(tuple(_slice_to_bytes(s) for s in x), use_bin_type=True)


def _slice_nd_from_bytes(data: bytes) -> SliceNd:
  return SliceNd(map(_slice_from_bytes, msgpack.unpackb(data, raw=True)))


def _slice_nd_array_to_bytes(x: SliceNdArray) -> bytes:
  tpl = (x.shape, tuple(_slice_nd_to_bytes(s) for s in x.flatten()))
  return msgpack.packb(tpl, use_bin_type=True)


def _slice_nd_array_from_bytes(data: bytes) -> SliceNdArray:
  shape, items = msgpack.unpackb(data, raw=True)
  arr = np.empty(len(items), dtype=object)
  for i, b in enumerate(items):
    arr[i] = _slice_nd_from_bytes(b)
  return SliceNdArray(arr.reshape(shape))


def _index_info_to_bytes(x: IndexInfo) -> bytes:
  tpl = (_shaped_array_to_bytes(x.global_shape),
         tuple(map(_slice_nd_to_bytes, x.global_slices)), tuple(int(s) for s in x.shards))
  return msgpack.packb(tpl, use_bin_type=True)


def _index_info_from_bytes(data: bytes) -> IndexInfo:
  global_shape, global_slices, shards = msgpack.unpackb(data, raw=True)
  return IndexInfo(global_shape=_shaped_array_from_bytes(global_shape),
                   global_slices=tuple(map(_slice_nd_from_bytes, global_slices)),
                   shards=tuple(shards))


def _lazy_array_chunks_encode(lac: LazyArrayChunks) -> Dict[str, Any]:
  def encode(pair):
    chunk, global_slice = pair
    chunk = to_numpy(chunk).reshape(-1)
    sub = max(1, int(MAX_CHUNK_SIZE / chunk.dtype.itemsize))
    return [[chunk[i:i + sub] for i in range(0, chunk.size, sub)], global_slice]

  state: Dict[str, Any] = {_ARRAY_CHUNKS_MAGIC_KEY: True}
  for index in lac.chunks.keys():
    state[str(index)] = [encode(p) for p in lac.iter_chunks(index)]
  return state


def _array_chunks_decode(mapping: Mapping[str, Any]):
  if _ARRAY_CHUNKS_MAGIC_KEY not in mapping:
    return mapping
  out = ArrayChunks()
  for index, chunks in mapping.items():
    if index == _ARRAY_CHUNKS_MAGIC_KEY:
      continue
    for subchunks, global_slice in chunks:
      flat = np.concatenate(subchunks) if len(subchunks) else np.zeros((0,))
      out.add(int(index), flat.reshape(global_slice.shape), global_slice)
  return out


def _ext_pack(x):
  if isinstance(x, complex):
    return msgpack.ExtType(_Ext.native_complex, msgpack.packb((x.real, x.imag)))
  if isinstance(x, ShapedArray):
    return msgpack.ExtType(_Ext.shaped_array, _shaped_array_to_bytes(x))
  if isinstance(x, Slice):
    return msgpack.ExtType(_Ext.slice, _slice_to_bytes(x))
  if isinstance(x, SliceNdArray):
    return msgpack.ExtType(_Ext.slice_nd_array, _slice_nd_array_to_bytes(x))
  if isinstance(x, SliceNd):
    return msgpack.ExtType(_Ext.slice_nd, _slice_nd_to_bytes(x))
  if isinstance(x, LazyArrayChunks):
    return _lazy_array_chunks_encode(x)
  if isinstance(x, IndexInfo):
    return msgpack.ExtType(_Ext.index_info, _index_info_to_bytes(x))
  if isinstance(x, np.ndarray) or type(x).__module__.startswith("torch"):
    return msgpack.ExtType(_Ext.ndarray, _ndarray_to_bytes(x))
  if isinstance(x, np.generic):
    return msgpack.ExtType(_Ext.npscalar, _ndarray_to_bytes(np.asarray(x)))
  return x


def _ext_unpack(code, data):
  if code == _Ext.native_complex:
    re, im = msgpack.unpackb(data)
    return complex(re, im)
  if code == _Ext.shaped_array:
    return _shaped_array_from_bytes(data)
  if code == _Ext.slice:
    return _slice_from_bytes(data)
  if code == _Ext.slice_nd:
    return _slice_nd_from_bytes(data)
  if code == _Ext.slice_nd_array:
    return _slice_nd_array_from_bytes(data)
  if code == _Ext.index_info:
    return _index_info_from_bytes(data)
  if code == _Ext.ndarray:
    return _ndarray_from_bytes(data)
  if code == _Ext.npscalar:
    return _ndarray_from_bytes(data)[()]
  return msgpack.ExtType(code, data)


# ------------------------------------------------------------------------------ public API
def msgpack_serialize(pytree, in_place: bool = False) -> bytes:
  """Tree of dict/list/tuple with array or scalar leaves -> msgpack bytes."""
  return msgpack.packb(_prepare(pytree), default=_ext_pack, strict_types=True)


def msgpack_restore(encoded: bytes):
  state = msgpack.unpackb(encoded, ext_hook=_ext_unpack, object_hook=_array_chunks_decode,
                          raw=False, strict_map_key=False)
  if isinstance(state, ArrayChunks):
    return state
  return _restore_chunked(state)


def to_state_dict(tree):
  """Nested-dict form of a tree: objects exposing ``state_dict()`` are expanded, lists and
  tuples become dicts keyed by position (as Flax's state dicts do)."""
  if hasattr(tree, "state_dict") and not type(tree).__module__.startswith("torch"):
    return to_state_dict(tree.state_dict())
  if isinstance(tree, Mapping):
    return {str(k): to_state_dict(v) for k, v in tree.items()}
  if isinstance(tree, (list, tuple)) and not isinstance(tree, SliceNd):
    return {str(i): to_state_dict(v) for i, v in enumerate(tree)}
  return tree


def from_state_dict(target, state):
  """Restores ``state`` (nested dict) into the structure of ``target``."""
  if target is None:
    return state
  if isinstance(target, ArrayChunks):
    return state
  if hasattr(target, "load_state_dict") and not type(target).__module__.startswith("torch"):
    target.load_state_dict(state)
    return target
  if isinstance(target, Mapping):
    if set(map(str, target.keys())) != set(map(str, state.keys())):
      raise ValueError(
          f"The target dict keys and state dict keys do not match, target dict contains keys "
          f"{set(target.keys()) - set(state.keys())} which are not present in state dict")
    return {k: from_state_dict(v, state[str(k)]) for k, v in target.items()}
  if isinstance(target, (list, tuple)) and not isinstance(target, SliceNd):
    return type(target)(from_state_dict(v, state[str(i)]) for i, v in enumerate(target))
  return state


def to_bytes(target) -> bytes:
  return msgpack_serialize(to_state_dict(target), in_place=True)


def from_bytes(target, encoded: bytes):
  return from_state_dict(target, msgpack_restore(encoded))
