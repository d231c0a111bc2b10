"""Periodic actions of the training loop: triggers (every N steps / every T seconds / on
given steps), progress reporting with per-part wall-time fractions, single-process gating,
and profiler windows (reference: ``vmoe/train/periodic_actions.py:32-76`` on top of CLU's
``PeriodicAction``)."""
from __future__ import annotations

import contextlib
import dataclasses
import time
from typing import Any, Callable, Dict, Iterable, Optional

from vmoe_b200.utils.misc import flatten_dict


def _process_index() -> int:
  import torch.distributed as dist
  return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


class PeriodicAction:
  """Calls ``_apply(step, t)`` when a trigger fires."""

  def __init__(self, *, every_steps: Optional[int] = None, every_secs: Optional[float] = None,
               on_steps: Optional[Iterable[int]] = None):
    self._every_steps = every_steps
    self._every_secs = every_secs
    self._on_steps = frozenset(on_steps or [])
    self._previous_step: Optional[int] = None
    self._previous_time: Optional[float] = None
    self._last_step: Optional[int] = None

  def _init_and_check(self, step: int, t: float):
    if self._previous_step is None:
      self._previous_step, self._previous_time, self._last_step = step, t, step
    elif self._every_steps is not None and step - self._last_step != 1:
      raise ValueError(f"PeriodicAction must be called after every step once "
                       f"(expected {self._last_step + 1}, got {step}).")
    else:
      self._last_step = step

  def _should_trigger(self, step: int, t: float) -> bool:
    if self._every_steps is not None and step % self._every_steps == 0:
      return True
    if self._every_secs is not None and t - self._previous_time > self._every_secs:
      return True
    return step in self._on_steps

  def _after_apply(self, step: int, t: float):
    self._previous_step, self._previous_time = step, t

  def __call__(self, step: int, t: Optional[float] = None) -> bool:
    t = time.monotonic() if t is None else t
    self._init_and_check(step, t)
    if self._should_trigger(step, t):
      self._apply(step, t)
      self._after_apply(step, t)
      return True
    return False

  def _apply(self, step: int, t: float):
    raise NotImplementedError


class PeriodicCallback(PeriodicAction):
  def __init__(self, *, callback_fn: Callable[..., Any], pass_step_and_time: bool = True,
               **kwargs):
    super().__init__(**kwargs)
    self._callback_fn = callback_fn
    self._pass = pass_step_and_time
    self._kwargs: Dict[str, Any] = {}

  def __call__(self, step: int, t: Optional[float] = None, **kwargs) -> bool:
    self._kwargs = kwargs
    return super().__call__(step, t)

  def _apply(self, step, t):
    if self._pass:
      self._callback_fn(step=step, t=t, **self._kwargs)
    else:
      self._callback_fn(**self._kwargs)


@dataclasses.dataclass
class SingleProcessPeriodicAction:
  """Runs a periodic action on one process only."""
  periodic_action: Callable[..., bool]
  process_index: int = 0

  def __call__(self, *args, **kwargs) -> bool:
    if _process_index() == self.process_index:
      return self.periodic_action(*args, **kwargs)
    return False


class ReportProgress(PeriodicAction):
  """Writes ``steps_per_sec``, ``uptime``, the given scalar metrics (nested names joined with
  '/'), optional ``host_memory_mb`` and ``uptime_<part>`` timings."""

  def __init__(self, *, num_train_steps: Optional[int] = None, writer=None,
               every_steps: Optional[int] = None, every_secs: Optional[float] = 60.0,
               on_steps: Optional[Iterable[int]] = None, process_index: Optional[int] = 0):
    super().__init__(every_steps=every_steps, every_secs=every_secs, on_steps=on_steps)
    self._num_train_steps = num_train_steps
    self._writer = writer
    self._process_index = process_index
    self._time_per_part: Dict[str, float] = {}
    self._t0 = time.monotonic()
    self._extra: Dict[str, Any] = {}

  def __call__(self, step: int, t: Optional[float] = None, **kwargs) -> bool:
    self._extra = kwargs
    return super().__call__(step, t)

  def _should_trigger(self, step, t):
    if self._process_index is not None and _process_index() != self._process_index:
      return False
    return super()._should_trigger(step, t)

  @contextlib.contextmanager
  def timed(self, name: str, wait_jax_async_dispatch: bool = True):
    """Accumulates the wall time spent inside the block under ``uptime_<name>``."""
    start = time.monotonic()
    try:
      yield
    finally:
      if wait_jax_async_dispatch:
        try:
          import torch
          if torch.cuda.is_available():
            torch.cuda.synchronize()
        except Exception:
          pass
      self._time_per_part[name] = self._time_per_part.get(name, 0.0) + time.monotonic() - start

  def _apply(self, step, t):
    scalars: Dict[str, float] = {}
    if self._previous_step is not None and t > self._previous_time and step > self._previous_step:
      scalars["steps_per_sec"] = (step - self._previous_step) / (t - self._previous_time)
    scalars["uptime"] = t - self._t0
    if self._writer is None:
      return
    metrics = self._extra.get("scalar_metrics") or {}
    for k, v in flatten_dict(metrics, sep="/").items():
      scalars[k] = float(v)
    try:
      import psutil
      scalars["host_memory_mb"] = psutil.Process().memory_info().rss / 2 ** 20
    except Exception:
      pass
    for key, value in self._time_per_part.items():
      scalars[f"uptime_{key}"] = value
    self._writer.write_scalars(step, scalars)


class Profile(PeriodicAction):
  """Collects a ``torch.profiler`` trace of ``num_profile_steps`` steps into ``logdir``; the
  first window starts at ``first_profile`` and later ones every ``every_secs``."""

  def __init__(self, *, logdir: str, num_profile_steps: int = 5, first_profile: int = 10,
               every_steps: Optional[int] = None, every_secs: Optional[float] = 3600.0):
    super().__init__(every_steps=every_steps, every_secs=every_secs, on_steps=[first_profile])
    self._logdir = logdir
    self._num = num_profile_steps
    self._prof = None
    self._stop_at: Optional[int] = None

  def __call__(self, step: int, t: Optional[float] = None) -> bool:
    if self._prof is not None and step >= self._stop_at:
      self._prof.__exit__(None, None, None)
      import os
      os.makedirs(self._logdir, exist_ok=True)
      self._prof.export_chrome_trace(os.path.join(self._logdir, f"trace_step{step}.json"))
      self._prof = None
    return super().__call__(step, t)

  def _apply(self, step, t):
    if self._prof is not None:
      return
    import torch
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
      acts.append(torch.profiler.ProfilerActivity.CUDA)
    self._prof = torch.profiler.profile(activities=acts)
    self._prof.__enter__()
    self._stop_at = step + self._num
