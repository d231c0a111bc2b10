"""Small utilities shared by the whole package.

Reference behaviour: ``vmoe/utils.py`` (``parse_call`` :59-109, ``partialclass`` :112-123,
``SafeZipIterator`` :130-165, ``make_match_fn_from_regex_list`` :176-189, ``make_rngs`` :43-47,
``multiply_no_nan`` :50-56, ``tree_rngs_split`` :168-173).
"""
from __future__ import annotations

import ast
import importlib
import re
from typing import Any, Callable, Dict, Iterator, Mapping, Optional, Sequence, Tuple, Type, Union

import torch


def parse_call(string: str, default_module: Union[str, Any]):
  """Parses ``"name"``, ``"name(1, k='v')"`` or ``"pkg.mod.name(...)"``.

  Returns ``(callable, args, kwargs)``. Arguments must be Python literals and nested calls
  are rejected. A bare name is looked up in ``default_module`` (a module object, a module
  path, or any object/dict with that attribute/key); a dotted name imports the module part.
  """
  expr = ast.parse(string, mode="eval").body
  args: Tuple[Any, ...] = ()
  kwargs: Dict[str, Any] = {}
  if isinstance(expr, ast.Call):
    args = tuple(ast.literal_eval(a) for a in expr.args)
    kwargs = {kw.arg: ast.literal_eval(kw.value) for kw in expr.keywords}
    expr = expr.func
  if isinstance(expr, ast.Name):
    module, name = default_module, expr.id
  elif isinstance(expr, ast.Attribute):
    name = expr.attr
    inner = expr.value
    module = string[:inner.end_col_offset]
    while not isinstance(inner, ast.Name):
      if not isinstance(inner, ast.Attribute):
        raise ValueError(f"string={string!r} is not a supported callable string.")
      inner = inner.value
  else:
    raise ValueError(f"string={string!r} is not a supported callable string.")
  if isinstance(module, str):
    module = importlib.import_module(module)
  if isinstance(module, Mapping):
    return module[name], args, kwargs
  return getattr(module, name), args, kwargs


def partialclass(cls: Type[Any], *base_args, **base_kwargs):
  """Subclass of ``cls`` whose constructor has ``base_args``/``base_kwargs`` pre-bound."""

  class _Partial(cls):  # type: ignore[misc, valid-type]

    def __init__(self, *args, **kwargs):
      merged = dict(base_kwargs)
      merged.update(kwargs)
      super().__init__(*(base_args + args), **merged)

  _Partial.__name__ = getattr(cls, "__name__", "Partial")
  return _Partial


class SafeZipIteratorError(RuntimeError):
  pass


class SafeZipIterator:
  """``zip`` that raises if the iterators do not all finish together."""

  def __init__(self, *iterators):
    self.iterators = tuple(iter(i) if not hasattr(i, "__next__") else i for i in iterators)

  def __iter__(self):
    return self

  def __next__(self) -> Tuple[Any, ...]:
    stop, values = None, []
    for i, it in enumerate(self.iterators):
      try:
        values.append(next(it))
      except StopIteration:
        if stop is None:
          stop = i
    if stop is not None:
      if values:
        raise SafeZipIteratorError(
            f"The {stop}-th iterator raised StopIteration before the rest")
      raise StopIteration
    return tuple(values)


def safe_map(f: Callable[..., Any], *iterables) -> Iterator[Any]:
  return map(lambda args: f(*args), SafeZipIterator(*[iter(i) for i in iterables]))


def safe_zip(*iterables) -> Iterator[Tuple[Any, ...]]:
  return SafeZipIterator(*[iter(i) for i in iterables])


def make_match_fn_from_regex_list(
    regexes: Optional[Union[str, Sequence[str]]]) -> Optional[Callable[[str], bool]]:
  """True iff the string is *searched* successfully by any of the regexes; None if no regex."""
  if not regexes:
    return None
  if isinstance(regexes, str):
    regexes = [regexes]
  joined = re.compile("(?:" + "|".join(f"(?:{r})" for r in regexes) + ")")
  return lambda s: joined.search(s) is not None


def make_rngs(rng_keys: Sequence[str], seed: int) -> Dict[str, torch.Generator]:
  """One independent CPU generator per named stream, derived from ``seed``."""
  out = {}
  for i, key in enumerate(rng_keys):
    g = torch.Generator()
    g.manual_seed((int(seed) * 1000003 + i * 7919 + 12345) % (2 ** 63 - 1))
    out[key] = g
  return out


def tree_rngs_split(rngs: Mapping[str, torch.Generator], num_splits: int = 2):
  """Splits every generator into ``num_splits`` children (draws one seed per child)."""
  outs = [dict() for _ in range(num_splits)]
  for key, g in rngs.items():
    seeds = torch.randint(0, 2 ** 62, (num_splits,), generator=g).tolist()
    for i, s in enumerate(seeds):
      child = torch.Generator()
      child.manual_seed(s)
      outs[i][key] = child
  return tuple(outs)


def multiply_no_nan(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
  """``x * y`` with the result forced to 0 wherever ``x == 0`` (even if ``y`` is inf/nan)."""
  x_ok = x != 0
  safe_y = torch.where(x_ok, y, torch.ones_like(y))
  return torch.where(x_ok, x * safe_y, torch.zeros_like(x))


def flatten_dict(tree: Mapping[str, Any], sep: str = "/", prefix: str = "") -> Dict[str, Any]:
  out: Dict[str, Any] = {}
  for k, v in tree.items():
    key = f"{prefix}{sep}{k}" if prefix else str(k)
    if isinstance(v, Mapping) and v:
      out.update(flatten_dict(v, sep, key))
    else:
      out[key] = v
  return out


def unflatten_dict(flat: Mapping[str, Any], sep: str = "/") -> Dict[str, Any]:
  out: Dict[str, Any] = {}
  for key, v in flat.items():
    parts = key.split(sep)
    d = out
    for p in parts[:-1]:
      d = d.setdefault(p, {})
    d[parts[-1]] = v
  return out


def natural_sort_key(s: str):
  """Sort key under which ``a_2`` precedes ``a_11``."""
  return [int(t) if t.isdigit() else t for t in re.split(r"(\d+)", s)]


def count_forward_flops(model: torch.nn.Module, *inputs) -> float:
  """Matmul FLOPs (2 per multiply-add) of one forward pass on this device, counted from the
  shapes seen by the model's linear layers, MLP blocks, expert MLPs, attention cores and
  routers during one ``model(*inputs)`` call under ``no_grad``.

  Expert MLPs are counted for the rows they actually process (experts x groups x capacity, or
  slots for Soft MoE), not for the tokens that were routed. Elementwise work is not counted.
  """
  from vmoe_b200 import moe as moe_core
  from vmoe_b200.models import vit_moe
  total = [0.0]
  handles = []

  def rows_of(t: torch.Tensor) -> int:
    return int(t.numel() // t.shape[-1])

  def dense_hook(mod, args, out):
    total[0] += 2.0 * rows_of(args[0]) * mod.weight.shape[0] * mod.weight.shape[1]

  def mlp_hook(mod, args, out):
    _, m, h = mod.w1.shape
    total[0] += 2.0 * rows_of(args[0]) * (h * m + m * mod.w2.shape[1])

  def attn_hook(mod, args, out):
    q = args[0]
    kv = args[1] if len(args) > 1 and args[1] is not None else q
    b, tq, tk = q.shape[0], q.shape[1], kv.shape[1]
    total[0] += 4.0 * b * mod.num_heads * tq * tk * mod.head_dim

  def moe_hook(mod, args, out):
    x = args[0]
    tokens, hdim = rows_of(x), x.shape[-1]
    groups = max(tokens // mod.group_size, 1)
    e = mod.num_experts
    router = mod.Router
    rows = tokens
    if hasattr(router, "num_selected_experts"):
      kw = dict(getattr(router, "dispatcher_kwargs", {}) or {})
      try:
        cap = moe_core._resolve_capacity(
            kw.get("capacity"), kw.get("capacity_factor"),
            mod.group_size * router.num_selected_experts, e,
            kw.get("capacity_ceil_or_round", "ceil"), kw.get("capacity_multiple_of", 4))
        rows = groups * e * cap
      except Exception:  # pylint: disable=broad-except
        rows = tokens * router.num_selected_experts
    elif getattr(router, "mu", None) is not None:
      rows = groups * e * router.mu.shape[2]
    _, m, h = mod.Mlp.w1.shape
    total[0] += 2.0 * rows * 2 * h * m
    dense = getattr(router, "dense", None)
    if dense is not None:
      total[0] += 2.0 * tokens * hdim * dense.weight.shape[0]
    elif getattr(router, "mu", None) is not None:
      total[0] += 2.0 * tokens * hdim * e * router.mu.shape[2] * 3  # logits, dispatch, combine

  for mod in model.modules():
    if isinstance(mod, vit_moe.MlpMoeBlock):
      handles.append(mod.register_forward_hook(moe_hook))
    elif isinstance(mod, vit_moe.MlpBlock):
      handles.append(mod.register_forward_hook(mlp_hook))
    elif isinstance(mod, vit_moe.MultiHeadDotProductAttention):
      handles.append(mod.register_forward_hook(attn_hook))
    elif isinstance(mod, vit_moe.Dense):
      handles.append(mod.register_forward_hook(dense_hook))
  was_training = model.training
  try:
    model.eval()
    with torch.no_grad():
      model(*inputs)
  finally:
    model.train(was_training)
    for h in handles:
      h.remove()
  return total[0]


def get_flops_and_seconds_per_device(model: torch.nn.Module, *inputs,
                                     peak_flops_per_second: float = 1.418e15,
                                     training: bool = True):
  """``(flops, optimal_seconds)`` of one step on this device: three times the forward matmul
  FLOPs when training (forward, activation gradients, weight gradients) and that count
  divided by the sustained bf16 GEMM rate of the GPU (default: the rate measured with cuBLAS
  on a B200 under its power cap). The reference reads both numbers from XLA's cost analysis
  of the compiled step (``vmoe/utils.py:27-40``)."""
  flops = count_forward_flops(model, *inputs) * (3.0 if training else 1.0)
  if flops <= 0:
    return None, None
  return flops, flops / peak_flops_per_second
