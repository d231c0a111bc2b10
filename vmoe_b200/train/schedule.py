"""Learning-rate schedules as plain ``step -> float`` callables.

Names and arguments follow the reference (``vmoe/train/schedule.py:22-122``): ``constant``,
``warmup_exponential_decay``, ``warmup_cosine_decay``, ``warmup_linear_decay``,
``warmup_polynomial_decay`` and ``big_vision_rsqrt``; ``decay_steps`` defaults to
``total_steps``. A schedule made of pieces hands each piece the step count relative to the
boundary where it starts.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence

Schedule = Callable[[int], float]


def constant_schedule(value: float) -> Schedule:
  return lambda count: float(value)


def polynomial_schedule(init_value: float, end_value: float, power: float,
                        transition_steps: int, transition_begin: int = 0) -> Schedule:
  def fn(count):
    if transition_steps <= 0:
      return float(init_value)
    c = min(max(count - transition_begin, 0), transition_steps)
    frac = 1.0 - c / transition_steps
    return (init_value - end_value) * (frac ** power) + end_value
  return fn


def linear_schedule(init_value: float, end_value: float, transition_steps: int,
                    transition_begin: int = 0) -> Schedule:
  return polynomial_schedule(init_value, end_value, 1.0, transition_steps, transition_begin)


def cosine_decay_schedule(init_value: float, decay_steps: int, alpha: float = 0.0,
                          exponent: float = 1.0) -> Schedule:
  def fn(count):
    if decay_steps <= 0:
      return float(init_value) * alpha
    c = min(max(count, 0), decay_steps)
    cosine = 0.5 * (1.0 + math.cos(math.pi * c / decay_steps))
    return init_value * ((1.0 - alpha) * cosine ** exponent + alpha)
  return fn


def exponential_decay(init_value: float, transition_steps: int, decay_rate: float,
                      transition_begin: int = 0, staircase: bool = False,
                      end_value: Optional[float] = None) -> Schedule:
  def fn(count):
    c = count - transition_begin
    if c <= 0:
      return float(init_value)
    p = c / transition_steps
    if staircase:
      p = math.floor(p)
    v = init_value * (decay_rate ** p)
    if end_value is not None:
      v = max(v, end_value) if decay_rate < 1.0 else min(v, end_value)
    return v
  return fn


def join_schedules(schedules: Sequence[Schedule], boundaries: Sequence[int]) -> Schedule:
  def fn(count):
    idx = 0
    for b in boundaries:
      if count >= b:
        idx += 1
    idx = min(idx, len(schedules) - 1)
    start = boundaries[idx - 1] if idx > 0 else 0
    return schedules[idx](count - start)
  return fn


def warmup_cosine_decay_schedule(init_value: float, peak_value: float, warmup_steps: int,
                                 decay_steps: int, end_value: float = 0.0,
                                 exponent: float = 1.0) -> Schedule:
  alpha = 0.0 if peak_value == 0.0 else end_value / peak_value
  return join_schedules([
      linear_schedule(init_value, peak_value, warmup_steps),
      cosine_decay_schedule(peak_value, decay_steps - warmup_steps, alpha, exponent),
  ], [warmup_steps])


def warmup_exponential_decay_schedule(init_value: float, peak_value: float, warmup_steps: int,
                                      transition_steps: int, decay_rate: float,
                                      transition_begin: int = 0, staircase: bool = False,
                                      end_value: Optional[float] = None) -> Schedule:
  return join_schedules([
      linear_schedule(init_value, peak_value, warmup_steps),
      exponential_decay(peak_value, transition_steps, decay_rate, transition_begin, staircase,
                        end_value),
  ], [warmup_steps])


def warmup_polynomial_decay_schedule(peak_value: float, end_value: float, power: float,
                                     warmup_steps: int, decay_steps: int) -> Schedule:
  """Linear warmup followed by polynomial decay."""
  return join_schedules([
      linear_schedule(0.0, peak_value, warmup_steps),
      polynomial_schedule(peak_value, end_value, power, decay_steps - warmup_steps),
  ], [warmup_steps])


def big_vision_rsqrt_schedule(*, peak_value: float, decay_steps: int, timescale: int,
                              warmup_steps: int = 0, cooldown_steps: int = 0) -> Schedule:
  """Linear warmup -> ``peak / sqrt(1 + t / timescale)`` -> linear cooldown to zero."""
  if decay_steps < warmup_steps + cooldown_steps:
    raise ValueError(
        "decay_steps must be greater than or equal to warmup_steps + cooldown_steps, but got "
        f"{decay_steps}, {warmup_steps} and {cooldown_steps}, respectively.")
  if timescale < 0:
    raise ValueError(f"timescale must be positive, but got {timescale}")
  cooldown_peak = peak_value / math.sqrt(
      1.0 + (decay_steps - warmup_steps - cooldown_steps) / timescale)
  schedules, boundaries = [], []
  if warmup_steps > 0:
    schedules.append(linear_schedule(0.0, peak_value, warmup_steps))
    boundaries.append(warmup_steps)
  schedules.append(lambda count: peak_value / math.sqrt(1.0 + count / timescale))
  boundaries.append(decay_steps - cooldown_steps)
  if cooldown_steps > 0:
    schedules.append(lambda count: cooldown_peak * (1 - count / cooldown_steps))
  return join_schedules(schedules, boundaries)


def create_learning_rate_schedule(*, schedule: str, total_steps: int, **kwargs) -> Schedule:
  if schedule == "constant":
    return constant_schedule(**kwargs)
  if schedule == "warmup_exponential_decay":
    return warmup_exponential_decay_schedule(init_value=0.0, **kwargs)
  kwargs["decay_steps"] = kwargs.pop("decay_steps", total_steps)
  if schedule == "warmup_cosine_decay":
    return warmup_cosine_decay_schedule(init_value=0.0, **kwargs)
  if schedule == "warmup_linear_decay":
    return warmup_polynomial_decay_schedule(power=1.0, **kwargs)
  if schedule == "warmup_polynomial_decay":
    return warmup_polynomial_decay_schedule(**kwargs)
  if schedule == "big_vision_rsqrt":
    return big_vision_rsqrt_schedule(**kwargs)
  raise ValueError(f"Unknown learning rate schedule: {schedule!r}")
