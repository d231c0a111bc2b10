"""ctypes loader for ``libvmoe_b200.so`` and mirrors of the structs in ``csrc/vmoe_api.h``.

The library is never built implicitly at import time: it is compiled by ``vmoe_b200.build``
and shipped inside the package. On a machine with a GPU a missing library is an error (the
CUDA ops refuse to fall back silently); on a CPU-only machine the pure PyTorch reference
implementations in ``vmoe_b200.ops`` are used and the library is optional.
"""
from __future__ import annotations

import ctypes
import os
import threading

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# VMOE_B200_LIB names another build of the same library (kernel experiments).
LIB_PATH = os.environ.get("VMOE_B200_LIB") or os.path.join(_PKG_DIR, "libvmoe_b200.so")

_lib = None
_lock = threading.Lock()

# Number of kernels launched through this module since the last reset (bench accounting).
launch_count = 0


class LibraryMissing(RuntimeError):
  pass


def count_launch(n: int = 1) -> None:
  global launch_count
  launch_count += n


def reset_launch_count() -> int:
  global launch_count
  n, launch_count = launch_count, 0
  return n


class GemmArgs(ctypes.Structure):
  _fields_ = [
      ("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("C", ctypes.c_void_p),
      ("C2", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p),
      ("gelu_pre", ctypes.c_void_p), ("colsum", ctypes.c_void_p),
      ("a_ready", ctypes.c_void_p), ("status", ctypes.c_void_p),
      ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
      ("batch", ctypes.c_int64),
      ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
      ("ldr", ctypes.c_int64), ("ldr2", ctypes.c_int64),
      ("a_batch_stride", ctypes.c_int64), ("b_batch_stride", ctypes.c_int64),
      ("c_batch_stride", ctypes.c_int64), ("bias_batch_stride", ctypes.c_int64),
      ("r_batch_stride", ctypes.c_int64),
      ("a_mn_major", ctypes.c_int32), ("b_mn_major", ctypes.c_int32),
      ("c_fp32", ctypes.c_int32), ("c_atomic", ctypes.c_int32),
      ("act", ctypes.c_int32), ("split_k", ctypes.c_int32),
      ("a_ready_epoch", ctypes.c_uint32), ("num_sms", ctypes.c_int32),
      ("c2_gelu_grad", ctypes.c_int32), ("pre_is_grad", ctypes.c_int32),
      ("mt_offset", ctypes.c_int32),
      ("cta_pair", ctypes.c_int32),
      ("c_multi", ctypes.c_void_p * 8),
      ("c_multi_count", ctypes.c_int32),
      ("c_multi_rows", ctypes.c_int64),
      ("push", ctypes.c_void_p),
      ("push_ctas", ctypes.c_int32),
      ("signal_flags", ctypes.c_void_p * 8),
      ("signal_count", ctypes.c_int32),
      ("done_counter", ctypes.c_void_p),
  ]


class PushArgs(ctypes.Structure):
  """Mirror of ``VmoePushArgs`` (row push of the expert-parallel dispatch)."""
  _fields_ = [
      ("x", ctypes.c_void_p), ("slot_pair", ctypes.c_void_p), ("weight", ctypes.c_void_p),
      ("dst_base", ctypes.c_void_p), ("flag_base", ctypes.c_void_p),
      ("ybuf_base", ctypes.c_void_p), ("dgate", ctypes.c_void_p),
      ("groups", ctypes.c_int64), ("s", ctypes.c_int64), ("e", ctypes.c_int64),
      ("c", ctypes.c_int64), ("k", ctypes.c_int64), ("h", ctypes.c_int64),
      ("experts_per_rank", ctypes.c_int64), ("ep", ctypes.c_int64), ("rank", ctypes.c_int64),
  ]


def available() -> bool:
  return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
  """Returns the loaded library, raising ``LibraryMissing`` if it was never built."""
  global _lib
  if _lib is not None:
    return _lib
  with _lock:
    if _lib is None:
      if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} not found: run `python -m vmoe_b200.build` (needs nvcc)")
      l = ctypes.CDLL(LIB_PATH)
      l.vmoe_last_error.restype = ctypes.c_char_p
      _lib = l
  return _lib


def check(rc: int, what: str) -> None:
  if rc != 0:
    msg = lib().vmoe_last_error().decode("utf-8", "replace")
    raise RuntimeError(f"{what} failed (rc={rc}): {msg}")


def ptr(t) -> int | None:
  """Device pointer of a tensor (None stays NULL)."""
  return None if t is None else t.data_ptr()


def stream_ptr() -> int:
  import torch
  return torch.cuda.current_stream().cuda_stream
