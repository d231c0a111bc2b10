"""Multi-threaded batch assembly on the host (``csrc/host_collate.cu`` through ctypes).

``stack`` is ``np.stack`` for equally shaped, C-contiguous examples, copying with several
threads and without the GIL, optionally straight into a caller-provided (pinned) buffer.
``stack_u8_to_f32`` fuses the uint8 -> float32 ``value_range`` map into the same pass. Both fall
back to NumPy when the library has not been built or the inputs do not qualify. The reference
leaves this to tf.data's C++ runtime (``vmoe/data/input_pipeline.py:121-160``).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

# Below this many bytes a single-threaded NumPy copy is as fast as starting threads.
MIN_NATIVE_BYTES = 1 << 20


def _library():
  from vmoe_b200.ops import _lib
  if not _lib.available():
    return None
  try:
    lib = _lib.lib()
  except OSError:  # built for another machine, or the CUDA runtime is missing
    return None
  # A library built before these entry points existed is treated as absent.
  return lib if hasattr(lib, "vmoe_collate_rows") else None


def _qualify(arrays: Sequence[np.ndarray]) -> bool:
  first = arrays[0]
  return all(isinstance(a, np.ndarray) and a.shape == first.shape and a.dtype == first.dtype
             and a.flags.c_contiguous for a in arrays) and first.dtype != object


def _pointers(arrays: Sequence[np.ndarray]):
  return (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])


def stack(arrays: Sequence[np.ndarray], out: Optional[np.ndarray] = None, threads: int = 0,
          min_bytes: int = MIN_NATIVE_BYTES) -> np.ndarray:
  """``np.stack(arrays)``, written into ``out`` if given (shape ``(len(arrays),) + shape``)."""
  arrays = [np.asarray(a) for a in arrays]
  if not arrays:
    raise ValueError("need at least one array to stack")
  lib = None
  if _qualify(arrays) and arrays[0].nbytes * len(arrays) >= min_bytes:
    lib = _library()
  if out is not None and (out.shape != (len(arrays),) + arrays[0].shape or
                          out.dtype != arrays[0].dtype or not out.flags.c_contiguous):
    raise ValueError("`out` must be a C-contiguous array of the stacked shape and dtype")
  if lib is None:
    if out is None:
      return np.stack(arrays)
    np.stack(arrays, out=out)
    return out
  if out is None:
    out = np.empty((len(arrays),) + arrays[0].shape, dtype=arrays[0].dtype)
  rc = lib.vmoe_collate_rows(_pointers(arrays), ctypes.c_int64(len(arrays)),
                             ctypes.c_int64(arrays[0].nbytes), ctypes.c_void_p(out.ctypes.data),
                             ctypes.c_int32(threads))
  if rc != 0:
    raise RuntimeError(f"vmoe_collate_rows failed (rc={rc})")
  return out


def stack_u8_to_f32(arrays: Sequence[np.ndarray], vmin: float, vmax: float,
                    out: Optional[np.ndarray] = None, threads: int = 0,
                    min_bytes: int = MIN_NATIVE_BYTES) -> np.ndarray:
  """Stacks uint8 images as float32 mapped from [0, 255] to [vmin, vmax]: the same values as
  ``value_range(vmin, vmax)`` applied to every example before ``np.stack``."""
  arrays = [np.asarray(a) for a in arrays]
  if not arrays or any(a.dtype != np.uint8 for a in arrays):
    raise ValueError("stack_u8_to_f32 needs uint8 arrays")
  scale = (float(vmax) - float(vmin)) / 255.0
  shift = float(vmin)
  shape = (len(arrays),) + arrays[0].shape
  if out is not None and (out.shape != shape or out.dtype != np.float32 or
                          not out.flags.c_contiguous):
    raise ValueError("`out` must be a C-contiguous float32 array of the stacked shape")
  lib = _library() if _qualify(arrays) and arrays[0].size * len(arrays) * 4 >= min_bytes else None
  if lib is None:
    res = np.stack(arrays).astype(np.float32) * np.float32(scale) + np.float32(shift)
    if out is None:
      return res
    out[...] = res
    return out
  if out is None:
    out = np.empty(shape, dtype=np.float32)
  rc = lib.vmoe_collate_u8_to_f32(_pointers(arrays), ctypes.c_int64(len(arrays)),
                                  ctypes.c_int64(arrays[0].size),
                                  ctypes.c_void_p(out.ctypes.data), ctypes.c_float(scale),
                                  ctypes.c_float(shift), ctypes.c_int32(threads))
  if rc != 0:
    raise RuntimeError(f"vmoe_collate_u8_to_f32 failed (rc={rc})")
  return out
