"""Gradient reduction for data parallelism.

Replicated parameters: sum over all ranks. Expert-sharded parameters: the all-to-all of the
backward pass has already summed the contributions of the ranks of the expert group, so only
the replicas of the shard (the 'replica' mesh axis) are summed. The division by the number of
ranks happens inside the optimizer kernel (``grad_div``). This is the explicit form of the
all-reduces GSPMD inserts in the reference for replicated vs ``('expert',)``-sharded
parameters (``vmoe/partitioning.py:407``, ``vmoe/data/pjit_utils.py:79-80``).
"""
from __future__ import annotations

import torch.distributed as dist


def reduce_gradients(optimizer, mesh) -> None:
  if mesh is None or mesh.world_size == 1 or not dist.is_initialized():
    return
  reducer = getattr(optimizer, "grad_reducer", None)
  for kind, bucket in optimizer.buckets.items():
    bucket.rebind_grads()
    if kind == "dense":
      if reducer is not None and reducer._armed:
        reducer.finish()  # ranges were reduced during backward by the peer-memory kernels
      else:
        dist.all_reduce(bucket.grads, group=mesh.world_group)
    elif mesh.num_replicas > 1:
      dist.all_reduce(bucket.grads, group=mesh.replica_group)
