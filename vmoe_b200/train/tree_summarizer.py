"""Summaries of arrays in a (flattened) train state selected by regex rules.

A rule is a regex or ``(regex, transform, ...)``; a transform is an op name (``norm``,
``mean``, ``std``, ``sum``, ``min``, ``max``) or ``(op, axes)``. Every value left after the
transforms becomes one scalar named ``key_op(axes)[idx]``; a rule yielding more than
``max_summary_values`` values for an array raises (reference:
``vmoe/train/tree_summarizer.py:48-136``).
"""
from __future__ import annotations

import dataclasses
import itertools
import logging
import re
from typing import Any, Iterator, List, Sequence, Tuple

import torch

from vmoe_b200.utils.misc import flatten_dict

_OPS = {
    "sum": lambda x, a: x.sum(dim=a, keepdim=True),
    "mean": lambda x, a: x.mean(dim=a, keepdim=True),
    "std": lambda x, a: x.std(dim=a, keepdim=True, unbiased=False),
    "min": lambda x, a: x.amin(dim=a, keepdim=True),
    "max": lambda x, a: x.amax(dim=a, keepdim=True),
    "norm": lambda x, a: x.square().sum(dim=a, keepdim=True).sqrt(),
}


@dataclasses.dataclass(frozen=True)
class TreeSummarizer:
  rules: Sequence[Any]
  max_summary_values: int = 1

  def __post_init__(self):
    parsed = []
    for rule in self.rules:
      if isinstance(rule, (str, re.Pattern)):
        parsed.append((re.compile(rule),))
      else:
        pattern, *transforms = rule
        parsed.append((re.compile(pattern),) + tuple(transforms))
    object.__setattr__(self, "rules", parsed)

  def __call__(self, tree) -> Iterator[Tuple[str, Any]]:
    matched = [0] * len(self.rules)
    flat = flatten_dict(tree, sep="/") if not _is_flat(tree) else dict(tree)
    for key, value in flat.items():
      yield from self._summarize(key, value, matched)
    for i, rule in enumerate(self.rules):
      if matched[i] == 0:
        logging.warning("Rule %r was not matched with any leaf key.", rule)

  def _summarize(self, key, value, matched: List[int]):
    for i, (pattern, *transforms) in enumerate(self.rules):
      if pattern.search(key):
        matched[i] += 1
        suffix, summary = self._transform(torch.as_tensor(value), transforms)
        if summary.numel() > self.max_summary_values:
          raise ValueError(
              f"Rule with pattern={pattern.pattern!r} and transforms={transforms} generates "
              f"{summary.numel()} > {self.max_summary_values} summary values. If this is "
              "intended, increase the max_yielded_value_per_array.")
        yield from self._yield(key + suffix, summary)

  @classmethod
  def _transform(cls, value, transforms):
    suffix, out = "", value.float() if not value.is_floating_point() else value
    for transform in transforms:
      op = transform if isinstance(transform, str) else transform[0]
      if isinstance(transform, str):
        axes = None
      else:
        axes = transform[1]
        axes = (axes,) if isinstance(axes, int) else tuple(axes)
      if op not in _OPS:
        raise ValueError(
            f"Operation op={op!r} was extracted from transform={transform!r}, but this isn't "
            "supported.")
      out = _OPS[op](out, tuple(range(out.dim())) if axes is None else axes)
      suffix += f"_{op}"
      if axes is not None:
        suffix += f"{axes}"
    return suffix, out

  @classmethod
  def _yield(cls, prefix, value):
    for idx in itertools.product(*tuple(range(s) for s in value.shape)):
      idx_s = ",".join(str(i) for i, s in zip(idx, value.shape) if s > 1)
      yield prefix + ("[" + idx_s + "]" if idx_s else ""), value[idx]


def _is_flat(tree) -> bool:
  return all(not isinstance(v, dict) for v in tree.values())
