"""``map_state_dict``: fill a target tree from a source tree following renaming/transform
rules, with checks for unmatched keys and dtype/shape mismatches (reference:
``vmoe/initialization/mapping.py:86-237``)."""
from __future__ import annotations

import logging
import re
from typing import Dict, Iterable, List, Union

import numpy as np

from vmoe_b200.checkpoints import serialization
from vmoe_b200.initialization import rules as _rules
from vmoe_b200.utils.misc import flatten_dict, unflatten_dict

Rules = _rules.Rules
UnparsedRules = _rules.UnparsedRules
Transformation = _rules.Transformation

_IDENTITY_RULE = _rules.RegexRule(pattern=re.compile("^(.*)$"), replacement=r"\1")
_SIGNED_FLOAT_RE = re.compile(r"([-+]?(?:\d+(?:\.\d*)?|\.\d+)(?:[eE][-+]?\d+)?)")


def _natural_sort(names: Iterable[str]) -> List[str]:
  def maybe_num(s):
    return (0, float(s), "") if _SIGNED_FLOAT_RE.fullmatch(s) else (1, 0.0, s)
  return sorted(names, key=lambda s: [maybe_num(c) for c in _SIGNED_FLOAT_RE.split(s)])


def _raise_or_warn(cls, exception_msg, raise_exception, warn_msg=None):
  if raise_exception:
    raise cls(exception_msg)
  logging.warning(warn_msg or exception_msg)


def _build(source_flat, target_flat, rules, raise_if_source_unmatched,
           raise_if_target_unmatched) -> Dict[str, Transformation]:
  if not isinstance(rules, Rules):
    rules = Rules.parse(rules)
  used = {k: False for k in target_flat}
  output: Dict[str, Transformation] = {}
  for src_key in _natural_sort(source_flat.keys()):
    rule = rules.find(src_key)
    if rule is None:
      msg = f"Source key {src_key!r} does not match any rule."
      _raise_or_warn(KeyError, msg, raise_if_source_unmatched, msg + " Assuming the identity rule.")
      rule = _IDENTITY_RULE
    if isinstance(rule, _rules.DropRule):
      continue
    dst_key = rule.rename(src_key)
    if dst_key not in target_flat:
      raise KeyError(f"Source key {src_key!r} was matched with target key {dst_key!r}, "
                     "but it does not exist.")
    if used[dst_key] and not isinstance(rule, _rules.StackRule):
      raise ValueError(f"Target key {dst_key!r} was matched more than once.")
    used[dst_key] = True
    src_value, tgt_value = source_flat[src_key], target_flat[dst_key]
    src_empty = isinstance(src_value, dict) and not src_value
    tgt_empty = isinstance(tgt_value, dict) and not tgt_value
    if src_empty != tgt_empty:
      raise ValueError(
          "One of the values represents an empty node, but not the other. "
          f"src_key={src_key!r} has type={type(src_value)!r} and dst_key={dst_key!r} has "
          f"type={type(tgt_value)!r}.")
    if src_empty:
      continue
    if isinstance(rule, _rules.StackRule) and dst_key in output:
      output[dst_key] = output[dst_key].append(src_value)
    elif isinstance(rule, _rules.RegexRule):
      output[dst_key] = rule.get_transformation(src_value, tgt_value)
    else:
      raise TypeError(f"Unexpected type for rule: {rule!r}")
  for dst_key, was_used in used.items():
    v = target_flat[dst_key]
    if not was_used and not (isinstance(v, dict) and not v):
      msg = f"Target key {dst_key!r} is unmatched."
      warn = msg + (f" The original value with shape {tuple(getattr(v, 'shape', ()))} and type "
                    f"{getattr(v, 'dtype', type(v))} will be preserved.")
      _raise_or_warn(ValueError, msg, raise_if_target_unmatched, warn)
  return output


def _apply(txs, target_flat, raise_if_dtype_mismatched, raise_if_shape_mismatched):
  out = {k: v for k, v in target_flat.items() if k not in txs}
  for key, tx in txs.items():
    value = tx()
    target = tx.target
    if hasattr(target, "detach"):  # torch tensor
      tdtype = serialization.to_numpy(target).dtype
    else:
      tdtype = np.dtype(getattr(target, "dtype", value.dtype))
    if value.dtype != tdtype:
      msg = (f"Target key {key!r} has mismatched dtypes. Actual = {value.dtype}, "
             f"expected = {tdtype}.")
      _raise_or_warn(ValueError, msg, raise_if_dtype_mismatched,
                     msg + " Converting to the expected dtype.")
      value = value.astype(tdtype)
    tshape = tuple(target.shape)
    if tuple(value.shape) != tshape:
      msg = (f"Target key {key!r} has mismatched shapes. Actual = {tuple(value.shape)!r}, "
             f"expected = {tshape!r}.")
      _raise_or_warn(ValueError, msg, raise_if_shape_mismatched,
                     msg + " Broadcasting to the expected shape.")
      value = np.broadcast_to(value, tshape).copy()
    out[key] = value
  return out


def map_state_dict(source, target, rules: Union[Rules, UnparsedRules],
                   raise_if_dtype_mismatched: bool = False,
                   raise_if_shape_mismatched: bool = True,
                   raise_if_source_unmatched: bool = True,
                   raise_if_target_unmatched: bool = True):
  """Returns the state-dict form of ``target`` with values taken from ``source``.

  Source keys are visited in natural order (``a_2`` before ``a_11``); each is renamed by the
  first rule whose regex is found in it. Leaves of the result are NumPy arrays for mapped
  keys and the untouched target values otherwise.
  """
  source_flat = flatten_dict(serialization.to_state_dict(source), sep="/")
  target_flat = flatten_dict(serialization.to_state_dict(target), sep="/")
  txs = _build(source_flat, target_flat, rules, raise_if_source_unmatched,
               raise_if_target_unmatched)
  out = _apply(txs, target_flat, raise_if_dtype_mismatched, raise_if_shape_mismatched)
  return unflatten_dict(out, sep="/")
