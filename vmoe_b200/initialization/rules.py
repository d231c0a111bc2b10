"""Rules that map arrays of a source state dict onto a target state dict.

A rule is ``(regex, replacement[, transform, *args])``: keys are *searched* by the regex, the
first matching rule wins; an empty/None replacement drops the array. Transforms: ``reshape
[shape]``, ``squeeze axis``, ``stack axis`` (all matching sources, in natural order),
``expand_tile axis reps``, ``zoom`` (linear resize to the target shape) and ``vit_zoom``
(resize the grid part of a ViT position embedding, keeping or creating the class-token row).

Reference: ``vmoe/initialization/rules.py:41-381``.
"""
from __future__ import annotations

import dataclasses
import math
import re
from typing import Any, List, Optional, Sequence, Tuple, Union

import numpy as np
import scipy.ndimage

UnparsedRules = Sequence[Sequence[Any]]


@dataclasses.dataclass
class Rule:
  pattern: Any

  def __post_init__(self):
    if isinstance(self.pattern, str):
      self.pattern = re.compile(self.pattern)

  def rename(self, key: str) -> str:
    return key


@dataclasses.dataclass
class DropRule(Rule):
  """Matched arrays are not used in the target tree."""


@dataclasses.dataclass
class RegexRule(Rule):
  replacement: str = r"\g<0>"

  def rename(self, key: str) -> str:
    return self.pattern.sub(self.replacement, key)

  def get_transformation(self, source, target) -> "Transformation":
    return CopyTransformation(target=target, array=source)


@dataclasses.dataclass
class ExpandTileRule(RegexRule):
  axis: Union[int, Tuple[int, ...]] = 0
  reps: Union[int, Tuple[int, ...]] = 1

  def get_transformation(self, source, target):
    return ExpandTileTransformation(target=target, array=source, axis=self.axis, reps=self.reps)


@dataclasses.dataclass
class ReshapeRule(RegexRule):
  shape: Optional[Tuple[int, ...]] = None

  def get_transformation(self, source, target):
    return ReshapeTransformation(target=target, array=source,
                                 shape=tuple(self.shape or target.shape))


@dataclasses.dataclass
class SqueezeRule(RegexRule):
  axis: int = 0

  def get_transformation(self, source, target):
    return SqueezeTransformation(target=target, array=source, axis=self.axis)


@dataclasses.dataclass
class StackRule(RegexRule):
  axis: int = 0

  def get_transformation(self, source, target):
    return StackTransformation(target=target, axis=self.axis, to_stack=[source])


@dataclasses.dataclass
class VitZoomRule(RegexRule):
  def get_transformation(self, source, target):
    return VitZoomTransformation(target=target, source=source)


@dataclasses.dataclass
class ZoomRule(RegexRule):
  def get_transformation(self, source, target):
    return ZoomTransformation(target=target, source=source)


@dataclasses.dataclass
class Rules:
  rules: List[Rule] = dataclasses.field(default_factory=list)

  def find(self, key: str) -> Optional[Rule]:
    for rule in self.rules:
      if rule.pattern.search(key):
        return rule
    return None

  @classmethod
  def parse(cls, rules: UnparsedRules) -> "Rules":
    parsed: List[Rule] = []
    for rule in rules:
      if isinstance(rule, Rule):
        parsed.append(rule)
        continue
      pattern, replacement, *transform = rule
      pattern = re.compile(pattern)
      if not transform:
        parsed.append(RegexRule(pattern, replacement) if replacement else DropRule(pattern))
      elif transform[0] == "reshape":
        assert len(transform) in (1, 2)
        parsed.append(ReshapeRule(pattern, replacement,
                                  shape=transform[1] if len(transform) == 2 else None))
      elif transform[0] == "squeeze":
        assert len(transform) == 2 and isinstance(transform[1], int)
        parsed.append(SqueezeRule(pattern, replacement, axis=transform[1]))
      elif transform[0] == "stack":
        assert len(transform) == 2 and isinstance(transform[1], int)
        parsed.append(StackRule(pattern, replacement, axis=transform[1]))
      elif transform[0] == "expand_tile":
        assert len(transform) == 3
        parsed.append(ExpandTileRule(pattern, replacement, axis=transform[1], reps=transform[2]))
      elif transform[0] == "vit_zoom":
        parsed.append(VitZoomRule(pattern, replacement))
      elif transform[0] == "zoom":
        parsed.append(ZoomRule(pattern, replacement))
      else:
        raise ValueError(f"Rule {rule!r} cannot be parsed.")
    return cls(rules=parsed)


# ----------------------------------------------------------------------------- transformations
def _np(x) -> np.ndarray:
  from vmoe_b200.checkpoints.serialization import to_numpy
  return to_numpy(x)


@dataclasses.dataclass
class Transformation:
  """Produces the array to store in ``target`` (an array, or anything with shape/dtype)."""
  target: Any

  def __call__(self) -> np.ndarray:
    raise NotImplementedError


@dataclasses.dataclass
class CopyTransformation(Transformation):
  array: Any = None

  def __call__(self):
    return _np(self.array)


@dataclasses.dataclass
class ExpandTileTransformation(Transformation):
  array: Any = None
  axis: Union[int, Tuple[int, ...]] = 0
  reps: Union[int, Tuple[int, ...]] = 1

  def __call__(self):
    array = np.expand_dims(_np(self.array), axis=self.axis)
    axis = (self.axis,) if isinstance(self.axis, int) else tuple(self.axis)
    reps = (self.reps,) if isinstance(self.reps, int) else tuple(self.reps)
    if len(axis) != len(reps):
      raise ValueError(f"axis={axis} and reps={reps} have different lengths")
    full = [1] * array.ndim
    for a, r in zip(axis, reps):
      full[a] = r
    return np.tile(array, full)


@dataclasses.dataclass
class ReshapeTransformation(Transformation):
  array: Any = None
  shape: Tuple[int, ...] = ()

  def __call__(self):
    return np.reshape(_np(self.array), self.shape)


@dataclasses.dataclass
class SqueezeTransformation(Transformation):
  array: Any = None
  axis: int = 0

  def __call__(self):
    return np.squeeze(_np(self.array), axis=self.axis)


@dataclasses.dataclass
class StackTransformation(Transformation):
  axis: int = 0
  to_stack: List[Any] = dataclasses.field(default_factory=list)

  def append(self, x) -> "StackTransformation":
    return dataclasses.replace(self, to_stack=self.to_stack + [x])

  def __call__(self):
    return np.stack([_np(x) for x in self.to_stack], axis=self.axis)


def _zoom(source: np.ndarray, target_shape: Sequence[int]) -> np.ndarray:
  zoom = tuple(n / o for n, o in zip(target_shape, source.shape))
  src = source.astype(np.float32) if source.dtype.name == "bfloat16" else source
  return scipy.ndimage.zoom(src, zoom, order=1).astype(source.dtype)


@dataclasses.dataclass
class ZoomTransformation(Transformation):
  source: Any = None

  def __call__(self):
    return _zoom(_np(self.source), tuple(self.target.shape))


@dataclasses.dataclass
class VitZoomTransformation(ZoomTransformation):
  """Position-embedding resize: only the square grid part is interpolated."""

  @staticmethod
  def _tok_and_grid(shape):
    _, num_tokens, hidden = shape
    side = int(math.sqrt(num_tokens))
    if num_tokens not in (side ** 2, side ** 2 + 1):
      raise ValueError(
          f"num_tokens={num_tokens} is neither a perfect square nor a perfect square + 1. "
          "This means that the grid used is not squared. This isn't supported.")
    return side ** 2 != num_tokens, (1, side, side, hidden)

  def __call__(self):
    source = _np(self.source)
    target = self.target
    tshape = tuple(target.shape)
    if source.ndim != 3 or source.shape[0] != 1:
      raise ValueError(f"source.shape={source.shape} is not (1, ?, ?)")
    if len(tshape) != 3 or tshape[0] != 1:
      raise ValueError(f"target.shape={tshape} is not (1, ?, ?)")
    if source.shape[2] != tshape[2]:
      raise ValueError(f"source.shape[2]={source.shape[2]} != {tshape[2]}")
    src_tok, src_grid = self._tok_and_grid(source.shape)
    tgt_tok, tgt_grid = self._tok_and_grid(tshape)
    grid = source[:, 1:, :] if src_tok else source
    out = _zoom(grid.reshape(src_grid), tgt_grid).reshape(1, -1, tshape[2])
    if not tgt_tok:
      return out
    if src_tok:
      tok = source[:, :1, :]
    elif hasattr(target, "__array__") or hasattr(target, "numpy") or hasattr(target, "detach"):
      tok = _np(target)[:, :1, :]
    else:  # only a shape/dtype is known: a fresh N(0, 0.02) token embedding
      tok = (0.02 * np.random.default_rng(0).standard_normal((1, 1, tshape[2]))).astype(out.dtype)
    return np.concatenate([tok.astype(out.dtype), out], axis=1)
