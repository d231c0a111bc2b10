"""Data-parallel gradient all-reduce overlapped with the backward pass.

The flat fp32 gradient buffer of the replicated ("dense") parameters lives in symmetric memory.
It is split into ranges that become complete at known points of the backward pass (one per
encoder block, marked in the model with ``grad_marker``). When a marker fires, the range is
all-reduced by the kernels of ``csrc/allreduce_p2p.cu`` on a side stream, with peer loads over
NVLink, while the backward pass of the earlier blocks continues on the compute stream.
Whatever is left (embedding, and everything for models without markers) is reduced when the
backward pass has ended. The division by the number of ranks happens in the optimizer kernel.

This replaces the all-reduces that GSPMD inserts for replicated parameters in the reference
(``vmoe/train/trainer.py:648-684`` under ``pjit``; ``vmoe/partitioning.py:407``).
"""
from __future__ import annotations

import ctypes
import os
import re
from typing import Dict, List, Optional, Sequence, Tuple

import torch

_ACTIVE: Optional["OverlappedGradReducer"] = None
_TAG_RE = re.compile(r"encoderblock_(\d+)(?:/|$)")
FINAL_TAG = -1
MAX_RANGES = 64


class _GradMarker(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, tag):
    ctx.tag = tag
    return x.view_as(x)

  @staticmethod
  def backward(ctx, grad):
    reducer = _ACTIVE
    if reducer is not None:
      reducer.notify(ctx.tag)
    return grad, None


def grad_marker(x: torch.Tensor, tag: int) -> torch.Tensor:
  """Identity. In backward, tells the active reducer that the gradient with respect to ``x``
  exists, i.e. that all parameters used after this point (tags >= ``tag``) have their
  gradients. Without an active reducer this adds no autograd node."""
  if _ACTIVE is None or not x.requires_grad or not torch.is_grad_enabled():
    return x
  return _GradMarker.apply(x, tag)


def enabled_by_env() -> bool:
  return os.environ.get("VMOE_B200_GRAD_P2P", "1") != "0"


def plan_ranges(keys: Sequence[str], offsets: Sequence[int], sizes: Sequence[int],
                head_tag: int) -> Dict[int, List[Tuple[int, int]]]:
  """Groups parameters (flat-buffer ``offsets`` / padded ``sizes`` in elements) by the marker
  tag after which their gradients are complete and merges neighbours into ranges.

  Parameters of ``encoderblock_<i>`` are complete when marker ``i`` fires; the head and the
  final encoder norm when marker ``head_tag`` (= number of blocks) fires; everything else
  (embedding, position embedding, class token, other models) only after the backward pass.
  """
  tagged: List[Tuple[int, int, int]] = []
  for key, off, size in zip(keys, offsets, sizes):
    m = _TAG_RE.search(key)
    if m:
      tag = int(m.group(1))
    elif re.search(r"(^|/)(head|encoder_norm|pre_logits)(/|$)", key):
      tag = head_tag
    else:
      tag = FINAL_TAG
    tagged.append((tag, off, size))
  out: Dict[int, List[Tuple[int, int]]] = {}
  for tag, off, size in sorted(tagged, key=lambda t: (t[0], t[1])):
    ranges = out.setdefault(tag, [])
    if ranges and ranges[-1][0] + ranges[-1][1] == off:
      ranges[-1] = (ranges[-1][0], ranges[-1][1] + size)
    else:
      ranges.append((off, size))
  return out


class OverlappedGradReducer:
  """Owns the symmetric gradient buffer of one optimizer bucket and reduces it range by range."""

  def __init__(self, bucket, group, world_size: int, rank: int, num_blocks: int,
               ctas: int = 24):
    from vmoe_b200.parallel import symm
    from vmoe_b200.train.optimizer import CHUNK
    self.bucket = bucket
    self.world = world_size
    self.rank = rank
    self.ctas = ctas
    keys = [k for k, _ in bucket.entries]
    sizes = [-(-p.numel() // CHUNK) * CHUNK for _, p in bucket.entries]
    self.plan = plan_ranges(keys, bucket.offsets, sizes, head_tag=num_blocks)
    self.ranges: List[Tuple[int, int]] = []
    self.range_ids: Dict[int, List[int]] = {}
    for tag, ranges in self.plan.items():
      for r in ranges:
        self.range_ids.setdefault(tag, []).append(len(self.ranges))
        self.ranges.append(r)
    if len(self.ranges) > MAX_RANGES:
      # Too fragmented for per-block overlap: one range over the whole buffer at the end.
      self.ranges = [(0, bucket.numel)]
      self.range_ids = {FINAL_TAG: [0]}
    self.num_ranges = len(self.ranges)
    grad_bytes = bucket.numel * 4
    # Canary words between the gradients and the counters and after the counters.
    guard0 = (grad_bytes + 255) // 256 * 256
    self.flag_off = guard0 + symm.GUARD_BYTES
    guard1 = (self.flag_off + 3 * self.num_ranges * 4 + 255) // 256 * 256
    self.buf = symm.SymmetricBuffer(guard1 + symm.GUARD_BYTES, group, device=bucket.device)
    self.buf.set_guards([guard0, guard1])
    new_grads = self.buf.local(0, (bucket.numel,), torch.float32)
    new_grads.copy_(bucket.grads)
    bucket.grads = new_grads
    for (_, p), off in zip(bucket.entries, bucket.offsets):
      p.grad = new_grads[off:off + p.numel()].view(p.shape)
    self._bufs = (ctypes.c_uint64 * self.world)(*self.buf.ptrs)
    self._flags = (ctypes.c_uint64 * self.world)(*[p + self.flag_off for p in self.buf.ptrs])
    self.done_counters = self.buf.local(self.flag_off + 2 * self.num_ranges * 4,
                                        (self.num_ranges,), torch.int32)
    self.local_counters = torch.zeros(2 * self.num_ranges, dtype=torch.int32, device=bucket.device)
    self.status = torch.zeros(1, dtype=torch.int32, device=bucket.device)
    self.stream = torch.cuda.Stream(device=bucket.device)
    self.epoch = 0
    self._fired: set = set()
    self._armed = False
    # Markers are inserted by forward passes from now on; they act only while armed.
    global _ACTIVE
    _ACTIVE = self

  # ------------------------------------------------------------------ step protocol
  def begin(self) -> None:
    """Call before the backward pass whose gradients are to be reduced."""
    global _ACTIVE
    self.epoch += 1
    self._fired = set()
    self._armed = True
    _ACTIVE = self

  def notify(self, tag: int) -> None:
    """Marker ``tag`` fired: reduce every not yet reduced tag >= ``tag``."""
    if not self._armed:
      return
    ready = [t for t in self.range_ids if t != FINAL_TAG and t >= tag and t not in self._fired]
    if ready:
      self._launch(sorted(ready, reverse=True))

  def finish(self) -> None:
    """Reduces what is left, then makes the compute stream wait for all reductions and for
    every peer to be done reading this rank's buffer."""
    from vmoe_b200.ops import _lib
    if not self._armed:
      return
    rest = [t for t in self.range_ids if t not in self._fired]
    if rest:
      self._launch(sorted(rest, reverse=True))
    self._armed = False
    cur = torch.cuda.current_stream(self.bucket.device)
    with torch.cuda.stream(self.stream):
      rc = _lib.lib().vmoe_wait_counters(
          ctypes.c_void_p(self.done_counters.data_ptr()), ctypes.c_int32(self.num_ranges),
          ctypes.c_uint32(self.epoch * self.world), ctypes.c_void_p(self.status.data_ptr()),
          ctypes.c_int64(0), ctypes.c_void_p(self.stream.cuda_stream))
      _lib.check(rc, "vmoe_wait_counters")
      _lib.count_launch()
    cur.wait_stream(self.stream)

  def deactivate(self) -> None:
    global _ACTIVE
    if _ACTIVE is self:
      _ACTIVE = None

  def _launch(self, tags: Sequence[int]) -> None:
    from vmoe_b200.ops import _lib
    lib = _lib.lib()
    cur = torch.cuda.current_stream(self.bucket.device)
    self.stream.wait_stream(cur)
    for tag in tags:
      self._fired.add(tag)
      for rid in self.range_ids[tag]:
        off, count = self.ranges[rid]
        rc = lib.vmoe_allreduce_range(
            self._bufs, self._flags, ctypes.c_int32(self.world), ctypes.c_int32(self.rank),
            ctypes.c_int64(off), ctypes.c_int64(count), ctypes.c_int32(rid),
            ctypes.c_int32(self.num_ranges), ctypes.c_uint32(self.epoch),
            ctypes.c_void_p(self.local_counters.data_ptr()),
            ctypes.c_void_p(self.status.data_ptr()), ctypes.c_int32(self.ctas), ctypes.c_int64(0),
            ctypes.c_void_p(self.stream.cuda_stream))
        _lib.check(rc, "vmoe_allreduce_range")
        _lib.count_launch(2)


def maybe_create(optimizer, mesh, model) -> Optional[OverlappedGradReducer]:
  """Creates the reducer for the dense bucket when this process is one of several GPU ranks
  with peer-mapped memory; otherwise returns None (NCCL all-reduce is used)."""
  import torch.distributed as dist
  from vmoe_b200.parallel import symm
  if (mesh is None or mesh.world_size <= 1 or mesh.world_size > 16 or
      not dist.is_available() or not dist.is_initialized() or not enabled_by_env() or
      not symm.available()):
    return None
  bucket = optimizer.buckets.get("dense")
  if bucket is None or bucket.device.type != "cuda" or bucket.numel == 0:
    return None
  num_blocks = 0
  for name, _ in model.named_modules():
    m = re.search(r"encoderblock_(\d+)$", name)
    if m:
      num_blocks = max(num_blocks, int(m.group(1)) + 1)
  return OverlappedGradReducer(bucket, mesh.world_group, mesh.world_size, mesh.rank, num_blocks)
