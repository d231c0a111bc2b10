"""A small ``ConfigDict`` with the subset of the ``ml_collections`` surface that the shipped
configs and the trainer use: attribute access, nested auto-wrapping of dicts, locking,
``unlocked()``, ``get``, ``update``, ``to_dict``, ``copy_and_resolve_references``, field
references/placeholders and ``--config.key=value`` style overrides.

If the real ``ml_collections`` package is importable, configs written against it load too:
``as_config_dict`` converts its objects through their ``to_dict``.
"""
from __future__ import annotations

import contextlib
import copy
from typing import Any, Dict, Iterator, Mapping, Optional


class FieldReference:
  """A lazily resolved value; several config fields may share one reference."""

  def __init__(self, default: Any = None, field_type: Optional[type] = None, required=False):
    self._value = default
    self._type = field_type or (type(default) if default is not None else None)
    self._required = required

  def get(self) -> Any:
    v = self._value
    if isinstance(v, FieldReference):
      v = v.get()
    if v is None and self._required:
      raise ValueError("required placeholder has no value")
    return v

  def set(self, value: Any) -> None:
    if (self._type is not None and value is not None and
        not isinstance(value, (self._type, FieldReference))):
      if self._type is float and isinstance(value, int):
        value = float(value)
      else:
        raise TypeError(f"expected {self._type}, got {type(value)}")
    self._value = value


def placeholder(field_type: type, required: bool = False) -> FieldReference:
  return FieldReference(None, field_type=field_type, required=required)


class ConfigDict:
  """Attribute-style nested dictionary with optional locking of the key set."""

  def __init__(self, initial: Optional[Mapping[str, Any]] = None, type_safe: bool = True):
    object.__setattr__(self, "_fields", {})
    object.__setattr__(self, "_locked", False)
    object.__setattr__(self, "_type_safe", type_safe)
    if initial is not None:
      if isinstance(initial, ConfigDict):
        initial = initial._fields
      for k, v in initial.items():
        self[k] = v

  # ---------------------------------------------------------------- mapping protocol
  @staticmethod
  def _wrap(v: Any) -> Any:
    if isinstance(v, ConfigDict) or isinstance(v, FieldReference):
      return v
    if isinstance(v, Mapping):
      return ConfigDict(v)
    if hasattr(v, "to_dict") and type(v).__name__ in ("ConfigDict", "FrozenConfigDict"):
      return ConfigDict(v.to_dict())
    return v

  def __setitem__(self, key: str, value: Any) -> None:
    if "." in key:
      head, rest = key.split(".", 1)
      self[head][rest] = value
      return
    if self._locked and key not in self._fields:
      raise KeyError(f"config is locked; cannot add new field {key!r}")
    cur = self._fields.get(key)
    if isinstance(cur, FieldReference) and not isinstance(value, FieldReference):
      cur.set(value)
      return
    value = self._wrap(value)
    if (self._type_safe and cur is not None and value is not None and
        not isinstance(cur, (ConfigDict, FieldReference)) and
        not isinstance(value, (FieldReference,)) and type(cur) is not type(value)):
      if isinstance(cur, float) and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
      elif isinstance(cur, (tuple, list)) and isinstance(value, (tuple, list)):
        value = type(cur)(value)
      elif isinstance(cur, bool) or isinstance(value, bool) or not (
          isinstance(cur, (int, float, str)) and isinstance(value, type(cur))):
        raise TypeError(
            f"type of field {key!r} is {type(cur).__name__}, got {type(value).__name__}")
    self._fields[key] = value

  def __getitem__(self, key: str) -> Any:
    if "." in key:
      head, rest = key.split(".", 1)
      return self[head][rest]
    v = self._fields[key]
    return v.get() if isinstance(v, FieldReference) else v

  def __setattr__(self, key: str, value: Any) -> None:
    self[key] = value

  def __getattr__(self, key: str) -> Any:
    if key.startswith("__"):
      raise AttributeError(key)
    try:
      return self[key]
    except KeyError as e:
      raise AttributeError(key) from e

  def __delitem__(self, key: str) -> None:
    if self._locked:
      raise KeyError("config is locked")
    del self._fields[key]

  __delattr__ = __delitem__

  def __contains__(self, key: str) -> bool:
    if isinstance(key, str) and "." in key:
      head, rest = key.split(".", 1)
      return head in self._fields and isinstance(self._fields[head], ConfigDict) and rest in self._fields[head]
    return key in self._fields

  def __iter__(self) -> Iterator[str]:
    return iter(self._fields)

  def __len__(self) -> int:
    return len(self._fields)

  def keys(self):
    return self._fields.keys()

  def values(self):
    return [self[k] for k in self._fields]

  def items(self):
    return [(k, self[k]) for k in self._fields]

  def get(self, key: str, default: Any = None) -> Any:
    try:
      return self[key]
    except KeyError:
      return default

  def get_ref(self, key: str) -> FieldReference:
    v = self._fields[key]
    if not isinstance(v, FieldReference):
      v = FieldReference(v)
      self._fields[key] = v
    return v

  def update(self, *others: Mapping[str, Any], **kwargs: Any) -> None:
    for other in others + (kwargs,):
      for k, v in (other.items() if other is not None else []):
        if (k in self._fields and isinstance(self._fields[k], ConfigDict) and
            isinstance(v, (Mapping, ConfigDict))):
          self._fields[k].update(v)
        else:
          self[k] = v

  def update_from_flattened_dict(self, flat: Mapping[str, Any]) -> None:
    for k, v in flat.items():
      self[k] = v

  # ---------------------------------------------------------------- locking
  def lock(self) -> "ConfigDict":
    object.__setattr__(self, "_locked", True)
    for v in self._fields.values():
      if isinstance(v, ConfigDict):
        v.lock()
    return self

  def unlock(self) -> "ConfigDict":
    object.__setattr__(self, "_locked", False)
    for v in self._fields.values():
      if isinstance(v, ConfigDict):
        v.unlock()
    return self

  @property
  def is_locked(self) -> bool:
    return self._locked

  @contextlib.contextmanager
  def unlocked(self):
    was = self._locked
    self.unlock()
    try:
      yield self
    finally:
      if was:
        self.lock()

  @contextlib.contextmanager
  def ignore_type(self):
    was = self._type_safe
    object.__setattr__(self, "_type_safe", False)
    try:
      yield self
    finally:
      object.__setattr__(self, "_type_safe", was)

  # ---------------------------------------------------------------- conversion
  def to_dict(self) -> Dict[str, Any]:
    out = {}
    for k in self._fields:
      v = self[k]
      out[k] = v.to_dict() if isinstance(v, ConfigDict) else copy.deepcopy(v)
    return out

  def copy_and_resolve_references(self) -> "ConfigDict":
    return ConfigDict(self.to_dict())

  def __deepcopy__(self, memo):
    return ConfigDict(self.to_dict())

  def __eq__(self, other: Any) -> bool:
    if isinstance(other, ConfigDict):
      return self.to_dict() == other.to_dict()
    if isinstance(other, Mapping):
      return self.to_dict() == dict(other)
    return NotImplemented

  def __repr__(self) -> str:
    return f"ConfigDict({self.to_dict()!r})"

  def __str__(self) -> str:
    import yaml  # local import: only for pretty printing
    try:
      return yaml.safe_dump(self.to_dict(), default_flow_style=False)
    except Exception:  # non-yaml-able leaves
      return repr(self)


class FrozenConfigDict(ConfigDict):
  """Immutable view (all mutation raises)."""

  def __init__(self, initial=None):
    super().__init__(initial)
    object.__setattr__(self, "_frozen", True)

  def __setitem__(self, key, value):
    if getattr(self, "_frozen", False):
      raise AttributeError("FrozenConfigDict is immutable")
    super().__setitem__(key, value)


def as_config_dict(obj: Any) -> ConfigDict:
  """Accepts our ConfigDict, a mapping, or an ``ml_collections`` ConfigDict."""
  if isinstance(obj, ConfigDict):
    return obj
  if hasattr(obj, "to_dict"):
    return ConfigDict(obj.to_dict())
  return ConfigDict(obj)
