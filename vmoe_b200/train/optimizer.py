"""Optimizer over flat parameter buffers with one fused update kernel per bucket.

All parameters of a bucket live in one contiguous fp32 buffer (``p.data`` become views), and
so do their gradients (``p.grad`` views), first/second moments and the bf16 compute copies.
One step is: sum of squared gradients (one kernel per bucket, device scalar), a single tiny
all-reduce for the scalars of expert shards, and one update kernel per bucket that applies
gradient scale, global-norm or value clipping, Adam / SGD-momentum, decoupled weight decay,
``-lr`` and freezing, and refreshes the bf16 copies. There are two buckets: replicated
parameters (gradients all-reduced over all ranks) and expert-sharded parameters (reduced over
the replica axis only).

The chain and its order are the reference's (``vmoe/train/optimizer.py:102-139``): per-regex
gradient scale -> clip -> adam | sgd | big_vision_adafactor -> ``g + wd * p`` -> ``* -lr`` ->
freeze. Regexes are searched in the Flax-style path of each parameter
(``vmoe_b200/models/naming.py``). On CPU tensors the same update runs as PyTorch ops.
"""
from __future__ import annotations

import ctypes
import re
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from vmoe_b200.ops import _lib
from vmoe_b200.train import schedule as schedule_lib

CHUNK = 1024
WeightDecay = Union[float, Sequence[Tuple[str, float]]]
_vp = ctypes.c_void_p


def _first_match(rules, key: str, default: float) -> float:
  for rx, value in rules:
    if rx.search(key):
      return value
  return default


def make_weight_decay_fn(weight_decay: Optional[WeightDecay]):
  if not weight_decay:
    return lambda key: 0.0
  if isinstance(weight_decay, (list, tuple)):
    rules = [(re.compile(k), float(v)) for k, v in weight_decay]
    return lambda key: _first_match(rules, key, 0.0)
  return lambda key: float(weight_decay)


def make_gradient_scale_fn(scales: Optional[Sequence[Tuple[str, float]]]):
  if not scales:
    return lambda key: 1.0
  rules = [(re.compile(k), float(v)) for k, v in scales]
  return lambda key: _first_match(rules, key, 1.0)


def make_frozen_fn(frozen_pattern=None, trainable_pattern=None):
  """Returns ``key -> bool`` (True = frozen)."""
  if not trainable_pattern and not frozen_pattern:
    return lambda key: False
  if trainable_pattern and frozen_pattern:
    raise ValueError(
        "You cannot specify both trainable_pattern and frozen_pattern. "
        f"trainable_pattern = {trainable_pattern!r}, frozen_pattern = {frozen_pattern!r}")
  pattern = trainable_pattern or frozen_pattern
  if not isinstance(pattern, str):
    pattern = "|".join(f"(?:{x})" for x in pattern)
  rx = re.compile(pattern)
  if frozen_pattern:
    return lambda key: rx.search(key) is not None
  return lambda key: rx.search(key) is None


def check_gradient_clip(global_norm=None, absolute_value=None):
  if global_norm and absolute_value:
    raise ValueError(
        "You must specify either `global_norm` or `absolute_value`, but not both: "
        f"global_norm = {global_norm!r}, absolute_value = {absolute_value!r}")
  return float(global_norm or 0.0), float(absolute_value or 0.0)


class _Bucket:
  """Flat storage of a set of parameters (all on one device, fp32)."""

  def __init__(self, entries: List[Tuple[str, torch.nn.Parameter]], need_v: bool):
    self.entries = entries
    self.offsets: List[int] = []
    n = 0
    for _, p in entries:
      self.offsets.append(n)
      n += -(-p.numel() // CHUNK) * CHUNK
    self.numel = n
    dev = entries[0][1].device if entries else torch.device("cpu")
    self.device = dev
    self.params = torch.zeros(n, dtype=torch.float32, device=dev)
    self.grads = torch.zeros(n, dtype=torch.float32, device=dev)
    self.mu = torch.zeros(n, dtype=torch.float32, device=dev)
    self.nu = torch.zeros(n, dtype=torch.float32, device=dev) if need_v else None
    self.shadow = torch.zeros(n, dtype=torch.bfloat16, device=dev) if dev.type == "cuda" else None
    self.meta = torch.zeros(max(n // CHUNK, 1), 4, dtype=torch.float32, device=dev)
    self.sums = torch.zeros(3, dtype=torch.float64, device=dev)
    for (key, p), off in zip(entries, self.offsets):
      view = self.params[off:off + p.numel()].view(p.shape)
      view.copy_(p.data.float())
      p.data = view
      p.grad = self.grads[off:off + p.numel()].view(p.shape)
      if self.shadow is not None:
        sh = self.shadow[off:off + p.numel()].view(p.shape)
        sh.copy_(view)
        p._bf16_shadow = sh
        p._shadow_version = p._version

  def set_meta(self, wd_fn, frozen_fn, gscale_fn):
    meta = torch.zeros(max(self.numel // CHUNK, 1), 4, dtype=torch.float32)
    for (key, p), off in zip(self.entries, self.offsets):
      c0, c1 = off // CHUNK, (off + -(-p.numel() // CHUNK) * CHUNK) // CHUNK
      meta[c0:c1, 0] = wd_fn(key)
      meta[c0:c1, 1] = 0.0 if frozen_fn(key) else 1.0
      meta[c0:c1, 2] = gscale_fn(key)
    self.meta.copy_(meta)

  def view_of(self, flat: torch.Tensor, i: int) -> torch.Tensor:
    p = self.entries[i][1]
    off = self.offsets[i]
    return flat[off:off + p.numel()].view(p.shape)

  def rebind_grads(self):
    for (_, p), off in zip(self.entries, self.offsets):
      g = self.grads[off:off + p.numel()].view(p.shape)
      if p.grad is None or p.grad.data_ptr() != g.data_ptr():
        if p.grad is not None:
          g.add_(p.grad.to(g.dtype))
        p.grad = g


class _AfTensor(ctypes.Structure):
  """Mirror of ``VmoeAdafactorTensor`` (``csrc/vmoe_api.h``)."""
  _fields_ = [("p", ctypes.c_void_p), ("g", ctypes.c_void_p), ("mu", ctypes.c_void_p),
              ("shadow", ctypes.c_void_p), ("vr", ctypes.c_void_p), ("vc", ctypes.c_void_p),
              ("v", ctypes.c_void_p), ("col_acc", ctypes.c_void_p), ("norm", ctypes.c_void_p),
              ("batch", ctypes.c_int64), ("rows", ctypes.c_int64), ("cols", ctypes.c_int64),
              ("weight_decay", ctypes.c_float), ("lr_mult", ctypes.c_float),
              ("grad_scale", ctypes.c_float), ("factored", ctypes.c_int32),
              ("c_is_largest", ctypes.c_int32), ("chunk0", ctypes.c_int64)]


class Optimizer:
  """See the module docstring. ``named_params`` yields ``(flax_path, parameter)`` pairs."""

  def __init__(self, named_params: Sequence[Tuple[str, torch.nn.Parameter]], *, name: str,
               total_steps: int, learning_rate: Union[float, Mapping[str, Any]],
               gradient_clip: Optional[Mapping[str, Any]] = None,
               weight_decay: Optional[WeightDecay] = None, frozen_pattern=None,
               trainable_pattern=None,
               gradient_scale: Optional[Sequence[Tuple[str, float]]] = None, mesh=None,
               **optim_kwargs):
    if name not in ("adam", "sgd", "big_vision_adafactor"):
      raise ValueError(f"Unknown optimizer: {name}")
    self.name = name
    self.mesh = mesh
    self.step_count = 0
    if isinstance(learning_rate, (float, int)):
      learning_rate = {"schedule": "constant", "value": learning_rate}
    self.lr_schedule = schedule_lib.create_learning_rate_schedule(
        **dict(learning_rate), total_steps=total_steps)
    self.clip_norm, self.clip_value = check_gradient_clip(**dict(gradient_clip or {}))
    self.kw = dict(optim_kwargs)
    if name == "adam":
      self.b1 = float(self.kw.pop("b1", 0.9))
      self.b2 = float(self.kw.pop("b2", 0.999))
      self.eps = float(self.kw.pop("eps", 1e-8))
      self.kw.pop("mu_dtype", None)  # moments are always kept in fp32 here
    elif name == "sgd":
      self.momentum = float(self.kw.pop("momentum", 0.0) or 0.0)
    named_params = [(k, p) for k, p in named_params]
    dense = [(k, p) for k, p in named_params if not getattr(p, "expert_sharded", False)]
    expert = [(k, p) for k, p in named_params if getattr(p, "expert_sharded", False)]
    need_v = name == "adam"
    self.buckets: Dict[str, _Bucket] = {}
    if dense:
      self.buckets["dense"] = _Bucket(dense, need_v)
    if expert:
      self.buckets["expert"] = _Bucket(expert, need_v)
    wd_fn = make_weight_decay_fn(weight_decay)
    frozen_fn = make_frozen_fn(frozen_pattern, trainable_pattern)
    gs_fn = make_gradient_scale_fn(gradient_scale)
    for b in self.buckets.values():
      b.set_meta(wd_fn, frozen_fn, gs_fn)
    self.last_learning_rate = float(self.lr_schedule(0))
    self.last_norms: Dict[str, torch.Tensor] = {}
    self.last_extra: Optional[torch.Tensor] = None
    if name == "big_vision_adafactor":
      self._init_adafactor()

  # ------------------------------------------------------------------ plumbing
  def zero_grad(self) -> None:
    for b in self.buckets.values():
      b.rebind_grads()
      b.grads.zero_()

  def parameters(self):
    for b in self.buckets.values():
      for _, p in b.entries:
        yield p

  def _sharded(self) -> bool:
    """Expert parameters are spread over several ranks: their sums need a reduction."""
    return ("expert" in self.buckets and self.mesh is not None and
            self.mesh.num_partitions > 1 and dist.is_initialized())

  @staticmethod
  def _reduce_sum(vec: torch.Tensor, group) -> torch.Tensor:
    """The one small all-reduce of this module (sum over ``group``, in place)."""
    dist.all_reduce(vec, group=group)
    return vec

  def _finish_sums(self, sums: torch.Tensor, extra: Optional[torch.Tensor]):
    """Global values of the per-bucket sums of squares and of the caller's scalars.

    ``sums``: double (3,) sums of this rank's expert bucket (zeros without one). ``extra``:
    1-D tensor of per-rank scalars to be averaged over all ranks (train metrics). Everything
    travels in ONE all-reduce over the world: expert sums come back multiplied by the number
    of replicas of each shard, the scalars by the world size, and both are divided out here.
    """
    world = dist.get_world_size() if (dist.is_initialized() and self.mesh is not None
                                      and self.mesh.world_size > 1) else 1
    if world == 1:
      return sums, extra
    parts = [sums.double()] + ([extra.double().reshape(-1)] if extra is not None else [])
    if not self._sharded() and extra is None:
      return sums, extra
    vec = self._reduce_sum(torch.cat(parts), self.mesh.world_group)
    out_sums = sums
    if self._sharded():
      out_sums = vec[:3] / float(self.mesh.num_replicas)
    out_extra = None if extra is None else (vec[3:] / world).to(extra.dtype).reshape(extra.shape)
    return out_sums, out_extra

  # ------------------------------------------------------------------ step
  @torch.no_grad()
  def step(self, grad_div: float = 1.0,
           extra: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
    """Applies one update. Gradients are first divided by ``grad_div``.

    Returns global L2 norms of gradients (after division and gradient scale, before
    clipping), updates and new parameters as 0-dim tensors. ``extra`` (1-D tensor of per-rank
    scalars, e.g. the step's metrics) is averaged over all ranks in the same small all-reduce
    that completes the norms; the result is left in ``self.last_extra``.
    """
    lr = float(self.lr_schedule(self.step_count))
    self.last_learning_rate = lr
    t = self.step_count + 1
    for b in self.buckets.values():
      b.rebind_grads()
      b.sums.zero_()
    dev = next(iter(self.buckets.values())).device
    zeros3 = torch.zeros(3, dtype=torch.float64, device=dev)
    if self.name == "big_vision_adafactor":
      dense_sums, expert_sums = self._adafactor_step(lr, grad_div)
      expert_sums, self.last_extra = self._finish_sums(expert_sums, extra)
      tot = dense_sums + expert_sums
      norms = {"grads": torch.sqrt(tot[0]), "updates": torch.sqrt(tot[1]),
               "params": torch.sqrt(tot[2])}
    else:
      for b in self.buckets.values():
        self._sumsq(b)
      dense = self.buckets.get("dense")
      expert = self.buckets.get("expert")
      dense_g2 = dense.sums[0].clone() if dense is not None else zeros3[0]
      expert_g2 = expert.sums[0].clone() if expert is not None else zeros3[0]
      if self.clip_norm > 0 and self._sharded():
        # Clipping needs the global gradient norm before the update: the expert shards' part is
        # summed over the expert group now; everything else waits for the end of the step.
        expert_g2 = self._reduce_sum(expert_g2.reshape(1), self.mesh.expert_group)[0]
        expert_g2_done = True
      else:
        expert_g2_done = False
      g2 = dense_g2 + expert_g2   # exact when reduced or unsharded; only read when clipping
      for b in self.buckets.values():
        b.sums[0] = g2
        self._update(b, lr, t, grad_div)
      esums = zeros3.clone()
      if expert is not None:
        esums = torch.stack([expert_g2 if not expert_g2_done else zeros3[0], expert.sums[1],
                             expert.sums[2]])
      esums, self.last_extra = self._finish_sums(esums, extra)
      dsums = dense.sums if dense is not None else zeros3
      total_g2 = dense_g2 + (expert_g2 if expert_g2_done else esums[0])
      norms = {"grads": torch.sqrt(total_g2) / grad_div,
               "updates": torch.sqrt(dsums[1] + esums[1]),
               "params": torch.sqrt(dsums[2] + esums[2])}
    for b in self.buckets.values():
      for _, p in b.entries:
        if b.shadow is not None:
          p._shadow_version = p._version
    self.step_count += 1
    self.last_norms = norms
    return norms

  def _sumsq(self, b: _Bucket) -> None:
    if b.device.type == "cuda":
      rc = _lib.lib().vmoe_grad_sumsq(_vp(b.grads.data_ptr()), _vp(b.meta.data_ptr()),
                                      ctypes.c_int64(b.numel), _vp(b.sums.data_ptr()),
                                      _vp(_lib.stream_ptr()))
      _lib.check(rc, "vmoe_grad_sumsq")
      _lib.count_launch()
    else:
      gs = b.meta[:, 2].repeat_interleave(CHUNK)[:b.numel]
      b.sums[0] = ((b.grads * gs).double() ** 2).sum()

  def _update(self, b: _Bucket, lr: float, t: int, grad_div: float) -> None:
    mode = 0 if self.name == "adam" else 1
    b1 = getattr(self, "b1", 0.0)
    b2 = getattr(self, "b2", 0.0)
    eps = getattr(self, "eps", 0.0)
    mom = getattr(self, "momentum", 0.0)
    bc1 = 1.0 - b1 ** t if mode == 0 else 1.0
    bc2 = 1.0 - b2 ** t if mode == 0 else 1.0
    if b.device.type == "cuda":
      f = ctypes.c_float
      rc = _lib.lib().vmoe_optimizer_step(
          _vp(b.params.data_ptr()), _vp(b.grads.data_ptr()), _vp(b.mu.data_ptr()),
          _vp(None if b.nu is None else b.nu.data_ptr()),
          _vp(None if b.shadow is None else b.shadow.data_ptr()), _vp(b.meta.data_ptr()),
          ctypes.c_int64(b.numel), ctypes.c_int32(mode), f(lr), f(b1), f(b2), f(eps), f(bc1),
          f(bc2), f(mom), f(self.clip_norm), f(self.clip_value), f(grad_div),
          _vp(b.sums.data_ptr()), _vp(_lib.stream_ptr()))
      _lib.check(rc, "vmoe_optimizer_step")
      _lib.count_launch()
      return
    rep = lambda col: b.meta[:, col].repeat_interleave(CHUNK)[:b.numel]
    wd, lrm, gs = rep(0), rep(1), rep(2)
    gfac = 1.0 / grad_div
    if self.clip_norm > 0:
      norm = float(torch.sqrt(b.sums[0])) / grad_div
      gfac *= self.clip_norm / max(norm, self.clip_norm)
    g = b.grads * gs * gfac
    if self.clip_value > 0:
      g = g.clamp(-self.clip_value, self.clip_value)
    if mode == 0:
      b.mu.mul_(b1).add_(g, alpha=1 - b1)
      b.nu.mul_(b2).addcmul_(g, g, value=1 - b2)
      direction = (b.mu / bc1) / (torch.sqrt(b.nu / bc2) + eps)
    else:
      b.mu.mul_(mom).add_(g)
      direction = b.mu
    upd = -lr * lrm * (direction + wd * b.params)
    b.params.add_(upd)
    b.sums[1] = (upd.double() ** 2).sum()
    b.sums[2] = (b.params.double() ** 2).sum()

  # ------------------------------------------------------------------ adafactor
  def _init_adafactor(self):
    kw = self.kw
    self.af = dict(decay_rate=kw.pop("decay_rate", 0.8), decay_rate_max=kw.pop("decay_rate_max", 0.999),
                   decay_offset=kw.pop("decay_offset", 0), eps=kw.pop("eps", 1e-30),
                   min_dim_size_to_factor=kw.pop("min_dim_size_to_factor", 32),
                   momentum=kw.pop("momentum", 0.9))
    kw.pop("momentum_dtype", None)
    self.af_state: Dict[int, Dict[str, torch.Tensor]] = {}
    for b in self.buckets.values():
      for i, (key, p) in enumerate(b.entries):
        st: Dict[str, torch.Tensor] = {}
        dims = _factored_dims(p.shape, self.af["min_dim_size_to_factor"])
        if dims is not None:
          d1, d0 = dims
          st["v_row"] = torch.zeros([s for j, s in enumerate(p.shape) if j != d0], device=p.device)
          st["v_col"] = torch.zeros([s for j, s in enumerate(p.shape) if j != d1], device=p.device)
        else:
          st["v"] = torch.zeros_like(p.data)
        self.af_state[id(p)] = st

  def _adafactor_cuda_plan(self):
    """Table of tensors for the Adafactor kernels (built once), or None when a parameter is
    factored over axes other than its last two (then the PyTorch formulation runs)."""
    if getattr(self, "_af_plan", False) is not False:
      return self._af_plan
    self._af_plan = None
    if next(iter(self.buckets.values())).device.type != "cuda" or not _lib.available():
      return None
    plans = {}
    for kind, b in self.buckets.items():
      rows, keep = [], []
      chunk0 = finish0 = max_tiles = 0
      finish_first = []
      for i, (key, p) in enumerate(b.entries):
        st = self.af_state[id(p)]
        dims = _factored_dims(p.shape, self.af["min_dim_size_to_factor"])
        t = _AfTensor()
        pv, gv, mv = b.view_of(b.params, i), b.view_of(b.grads, i), b.view_of(b.mu, i)
        t.p, t.g, t.mu = pv.data_ptr(), gv.data_ptr(), mv.data_ptr()
        t.shadow = b.view_of(b.shadow, i).data_ptr() if b.shadow is not None else None
        meta = b.meta[b.offsets[i] // CHUNK]
        t.weight_decay, t.lr_mult, t.grad_scale = float(meta[0]), float(meta[1]), float(meta[2])
        if dims is None:
          t.factored, t.batch, t.rows, t.cols = 0, 1, 1, p.numel()
          t.v = st["v"].data_ptr()
        else:
          d1, d0 = dims
          nd = p.dim()
          if {d1, d0} != {nd - 2, nd - 1}:
            return None
          t.factored, t.c_is_largest = 1, int(d0 == nd - 1)
          t.rows, t.cols = p.shape[-2], p.shape[-1]
          t.batch = p.numel() // (t.rows * t.cols)
          over_cols = st["v_row"] if d0 == nd - 1 else st["v_col"]   # (.., rows)
          over_rows = st["v_col"] if d0 == nd - 1 else st["v_row"]   # (.., cols)
          assert over_cols.is_contiguous() and over_rows.is_contiguous()
          col_acc = torch.zeros(t.batch * t.cols, device=p.device)
          norm = torch.zeros(t.batch, device=p.device)
          keep += [col_acc, norm]
          t.vr, t.vc = over_cols.data_ptr(), over_rows.data_ptr()
          t.col_acc, t.norm = col_acc.data_ptr(), norm.data_ptr()
          max_tiles = max(max_tiles, t.batch * ((t.rows + 15) // 16))
        t.chunk0 = chunk0
        chunk0 += (p.numel() + 1023) // 1024
        finish_first.append(finish0)
        finish0 += t.batch
        rows.append(t)
      arr = (_AfTensor * len(rows))(*rows)
      table = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(b.device)
      first = torch.tensor(finish_first, dtype=torch.int64, device=b.device)
      plans[kind] = dict(table=table, first=first, n=len(rows), finish_blocks=finish0,
                         chunks=chunk0, max_tiles=max_tiles, keep=keep)
    self._af_plan = plans
    return plans

  def _adafactor_step_cuda(self, plans, lr: float, grad_div: float):
    af = self.af
    tt = float(self.step_count - af["decay_offset"]) + 1.0
    decay = min(af["decay_rate_max"], 1.0 - tt ** (-af["decay_rate"]))
    dev = next(iter(self.buckets.values())).device
    for b in self.buckets.values():
      self._sumsq(b)   # sums[0] = sum of (grad * scale)^2, before the division by grad_div
    g2 = {k: b.sums[0].clone() for k, b in self.buckets.items()}
    zero = torch.zeros((), dtype=torch.float64, device=dev)
    eg2 = g2.get("expert", zero)
    if self.clip_norm > 0 and self._sharded():
      eg2 = self._reduce_sum(eg2.clone().reshape(1), self.mesh.expert_group)[0]
    total = g2.get("dense", zero) + eg2
    f = ctypes.c_float
    for kind, b in self.buckets.items():
      pl = plans[kind]
      b.sums[0] = total   # the kernels read the global norm for the clip
      rc = _lib.lib().vmoe_adafactor_step(
          _vp(pl["table"].data_ptr()), _vp(pl["first"].data_ptr()), ctypes.c_int32(pl["n"]),
          ctypes.c_int64(pl["finish_blocks"]), ctypes.c_int64(pl["chunks"]),
          ctypes.c_int64(pl["max_tiles"]), f(decay), f(af["eps"]), f(af["momentum"] or 0.0),
          f(lr), f(self.clip_norm), f(self.clip_value), f(grad_div), _vp(b.sums.data_ptr()),
          _vp(_lib.stream_ptr()))
      _lib.check(rc, "vmoe_adafactor_step")
      _lib.count_launch(3)
    div2 = grad_div * grad_div
    pack = lambda k: (torch.stack([g2[k] / div2, self.buckets[k].sums[1], self.buckets[k].sums[2]])
                      if k in self.buckets else torch.zeros(3, dtype=torch.float64, device=dev))
    return pack("dense"), pack("expert")

  def _adafactor_step(self, lr: float, grad_div: float):
    plans = self._adafactor_cuda_plan()
    if plans is not None:
      return self._adafactor_step_cuda(plans, lr, grad_div)
    af = self.af
    step = self.step_count
    tt = float(step - af["decay_offset"]) + 1.0
    decay = min(af["decay_rate_max"], 1.0 - tt ** (-af["decay_rate"]))
    dev = next(iter(self.buckets.values())).device
    g2_parts = {"dense": torch.zeros((), dtype=torch.float64, device=dev),
                "expert": torch.zeros((), dtype=torch.float64, device=dev)}
    scaled = []
    for kind, b in self.buckets.items():
      for i, (key, p) in enumerate(b.entries):
        g = b.view_of(b.grads, i) * (float(b.meta[b.offsets[i] // CHUNK, 2]) / grad_div)
        scaled.append(g)
        g2_parts[kind] += (g.double() ** 2).sum()
    fac = 1.0
    if self.clip_norm > 0:
      eg2 = g2_parts["expert"]
      if self._sharded():
        eg2 = self._reduce_sum(eg2.clone().reshape(1), self.mesh.expert_group)[0]
      gnorm = torch.sqrt(g2_parts["dense"] + eg2)
      fac = self.clip_norm / torch.clamp(gnorm, min=self.clip_norm)   # stays on the device
    upd2 = {k: torch.zeros_like(v) for k, v in g2_parts.items()}
    par2 = {k: torch.zeros_like(v) for k, v in g2_parts.items()}
    it = iter(scaled)
    for kind, b in self.buckets.items():
      for i, (key, p) in enumerate(b.entries):
        g = next(it) * fac
        if self.clip_value > 0:
          g = g.clamp(-self.clip_value, self.clip_value)
        st = self.af_state[id(p)]
        gsq = g * g + af["eps"]
        if "v" in st:
          st["v"].mul_(decay).add_(gsq, alpha=1 - decay)
          u = g / torch.sqrt(st["v"])
        else:
          d1, d0 = _factored_dims(p.shape, af["min_dim_size_to_factor"])
          st["v_row"].mul_(decay).add_(gsq.mean(dim=d0), alpha=1 - decay)
          st["v_col"].mul_(decay).add_(gsq.mean(dim=d1), alpha=1 - decay)
          reduced_d1 = d1 - 1 if d1 > d0 else d1
          row_col_mean = st["v_row"].mean(dim=reduced_d1, keepdim=True)
          row_factor = (st["v_row"] / row_col_mean) ** -0.5
          col_factor = st["v_col"] ** -0.5
          u = g * row_factor.unsqueeze(d0) * col_factor.unsqueeze(d1)
        mu = b.view_of(b.mu, i)
        if af["momentum"]:
          mu.mul_(af["momentum"]).add_(u, alpha=1 - af["momentum"])
          u = mu
        wd = float(b.meta[b.offsets[i] // CHUNK, 0])
        lrm = float(b.meta[b.offsets[i] // CHUNK, 1])
        upd = -lr * lrm * (u + wd * p.data)
        p.data.add_(upd)
        sh = getattr(p, "_bf16_shadow", None)
        if sh is not None:
          sh.copy_(p.data)
        upd2[kind] += (upd.double() ** 2).sum()
        par2[kind] += (p.data.double() ** 2).sum()
    pack = lambda k: torch.stack([g2_parts[k], upd2[k], par2[k]])
    return pack("dense"), pack("expert")

  # ------------------------------------------------------------------ state
  def state_dict(self) -> Dict[str, Any]:
    out: Dict[str, Any] = {"count": self.step_count,
                           "hyperparams": {"learning_rate": self.last_learning_rate},
                           "mu": {}, "nu": {}}
    for b in self.buckets.values():
      for i, (key, p) in enumerate(b.entries):
        out["mu"][key] = b.view_of(b.mu, i)
        if b.nu is not None:
          out["nu"][key] = b.view_of(b.nu, i)
    if self.name == "big_vision_adafactor":
      out["adafactor"] = {}
      for b in self.buckets.values():
        for key, p in b.entries:
          out["adafactor"][key] = self.af_state[id(p)]
    return out

  def load_state_dict(self, state: Mapping[str, Any]) -> None:
    self.step_count = int(state.get("count", 0))
    for b in self.buckets.values():
      for i, (key, p) in enumerate(b.entries):
        if key in state.get("mu", {}):
          b.view_of(b.mu, i).copy_(torch.as_tensor(state["mu"][key]).to(b.device))
        if b.nu is not None and key in state.get("nu", {}):
          b.view_of(b.nu, i).copy_(torch.as_tensor(state["nu"][key]).to(b.device))
        if self.name == "big_vision_adafactor" and key in state.get("adafactor", {}):
          for k2, v in state["adafactor"][key].items():
            self.af_state[id(p)][k2].copy_(torch.as_tensor(v).to(b.device))

  def sync_shadows(self) -> None:
    """Re-casts the bf16 copies after parameters were changed outside ``step``."""
    for b in self.buckets.values():
      if b.shadow is not None:
        b.shadow.copy_(b.params)
        for _, p in b.entries:
          p._shadow_version = p._version


def _factored_dims(shape, min_dim_size_to_factor: int):
  """The two largest dims (second largest, largest) if both are big enough, else None."""
  if len(shape) < 2:
    return None
  order = sorted(range(len(shape)), key=lambda i: (shape[i], i))
  if shape[order[-2]] < min_dim_size_to_factor:
    return None
  return order[-2], order[-1]


def create_optimizer(named_params, *, name: str, total_steps: int, learning_rate,
                     gradient_clip=None, weight_decay=None, frozen_pattern=None,
                     trainable_pattern=None, gradient_scale=None, mesh=None,
                     **optim_kwargs) -> Optimizer:
  """Factory with the reference's keyword surface (``vmoe/train/optimizer.py:90-139``)."""
  return Optimizer(named_params, name=name, total_steps=total_steps,
                   learning_rate=learning_rate, gradient_clip=gradient_clip,
                   weight_decay=weight_decay, frozen_pattern=frozen_pattern,
                   trainable_pattern=trainable_pattern, gradient_scale=gradient_scale,
                   mesh=mesh, **optim_kwargs)
