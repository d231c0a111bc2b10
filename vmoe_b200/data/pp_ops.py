"""Pre-processing ops of the data pipeline mini-language (``"op1|op2(3, k='v')"``).

Every factory returns a function ``dict -> dict``; single-input single-output ops accept
``key`` / ``inkey`` / ``outkey`` (default ``'image'``). Examples are dicts of NumPy arrays or
torch tensors; images are ``(H, W, C)``. Randomness comes from a per-pipeline ``numpy``
generator that the pipeline sets through ``set_rng``.

Ops: central_crop, copy, decode, decode_jpeg_and_inception_crop, flatten, flip_lr,
ignore_no_labels, inception_crop, keep, onehot, randaug, resize, resize_small, reshape,
tokenize, value_range (reference: ``vmoe/data/pp_ops.py:41-433``).
"""
from __future__ import annotations

import io
from typing import Any, Dict

import numpy as np
import torch
import torch.nn.functional as F

VALID_KEY = "__valid__"
Data = Dict[str, Any]

_RNG = np.random.default_rng(0)


def set_rng(rng: np.random.Generator) -> None:
  global _RNG
  _RNG = rng


class InKeyOutKey:
  """Adds ``key``/``inkey``/``outkey`` arguments to a single-input single-output op."""

  def __init__(self, indefault: str = "image", outdefault: str = "image"):
    self.indefault, self.outdefault = indefault, outdefault

  def __call__(self, get_pp_fn):
    def wrapper(*args, key=None, inkey=self.indefault, outkey=self.outdefault, **kw):
      fn = get_pp_fn(*args, **kw)
      def pp(data: Data) -> Data:
        data[key or outkey] = fn(data[key or inkey])
        return data
      return pp
    wrapper.__name__ = get_pp_fn.__name__
    wrapper.__doc__ = get_pp_fn.__doc__
    return wrapper


def _as_float_chw(img) -> torch.Tensor:
  t = torch.as_tensor(np.asarray(img) if not isinstance(img, torch.Tensor) else img)
  return t.permute(2, 0, 1).float()


def _from_chw(t: torch.Tensor, like) -> Any:
  out = t.permute(1, 2, 0)
  src = like.dtype if isinstance(like, torch.Tensor) else torch.as_tensor(np.asarray(like)).dtype
  if not src.is_floating_point:
    out = out.round().clamp(0, 255).to(src)
  return out if isinstance(like, torch.Tensor) else out.numpy()


def _resize_hw(img, size, method: str = "bilinear"):
  mode = {"bilinear": "bilinear", "nearest": "nearest", "bicubic": "bicubic",
          "area": "area"}[method]
  t = _as_float_chw(img)[None]
  kwargs = {} if mode in ("nearest", "area") else {"align_corners": False, "antialias": mode != "nearest"}
  out = F.interpolate(t, size=tuple(int(s) for s in size), mode=mode, **kwargs)[0]
  return _from_chw(out, img)


def _maybe_repeat(arg, n):
  if isinstance(arg, (list, tuple)):
    if len(arg) != n:
      raise ValueError(f"expected {n} values, got {arg}")
    return tuple(arg)
  return (arg,) * n


@InKeyOutKey()
def central_crop(crop_size):
  """Crops the centre ``crop_size`` (int or (h, w)) of the image."""
  ch, cw = _maybe_repeat(crop_size, 2)
  def fn(image):
    h, w = image.shape[0], image.shape[1]
    top, left = (h - ch) // 2, (w - cw) // 2
    return image[top:top + ch, left:left + cw]
  return fn


def copy(inkey, outkey):
  def fn(data: Data) -> Data:
    data[outkey] = data[inkey]
    return data
  return fn


def _decode_bytes(buf, channels: int):
  from PIL import Image  # optional dependency
  img = Image.open(io.BytesIO(bytes(buf)))
  img = img.convert("L" if channels == 1 else "RGB")
  arr = np.asarray(img)
  return arr[..., None] if arr.ndim == 2 else arr


@InKeyOutKey()
def decode(channels=3):
  """Decodes an encoded image (bytes) into ``uint8 (H, W, channels)``; arrays pass through."""
  def fn(image):
    if isinstance(image, (bytes, bytearray, memoryview)) or (
        isinstance(image, np.ndarray) and image.dtype.kind in "SO" and image.ndim == 0):
      return _decode_bytes(image if not isinstance(image, np.ndarray) else image.item(), channels)
    return image
  return fn


def _sample_inception_box(h, w, area_min, area_max, aspect=(3 / 4, 4 / 3)):
  area = h * w
  for _ in range(100):
    target = _RNG.uniform(area_min / 100.0, area_max / 100.0) * area
    log_r = _RNG.uniform(np.log(aspect[0]), np.log(aspect[1]))
    r = np.exp(log_r)
    cw = int(round(np.sqrt(target * r)))
    ch = int(round(np.sqrt(target / r)))
    if 0 < cw <= w and 0 < ch <= h:
      top = int(_RNG.integers(0, h - ch + 1))
      left = int(_RNG.integers(0, w - cw + 1))
      return top, left, ch, cw
  return 0, 0, h, w


@InKeyOutKey()
def inception_crop(resize_size=None, area_min=5, area_max=100, resize_method="bilinear"):
  """Random crop covering ``area_min..area_max`` percent of the image (aspect 3/4..4/3),
  optionally resized."""
  def fn(image):
    top, left, ch, cw = _sample_inception_box(image.shape[0], image.shape[1], area_min, area_max)
    crop = image[top:top + ch, left:left + cw]
    if resize_size:
      crop = _resize_hw(crop, _maybe_repeat(resize_size, 2), resize_method)
    return crop
  return fn


@InKeyOutKey()
def decode_jpeg_and_inception_crop(resize_size=None, area_min=5, area_max=100):
  dec = decode.__wrapped__(3) if hasattr(decode, "__wrapped__") else None
  def fn(image):
    img = _decode_bytes(image, 3) if isinstance(image, (bytes, bytearray, memoryview)) else image
    top, left, ch, cw = _sample_inception_box(img.shape[0], img.shape[1], area_min, area_max)
    crop = img[top:top + ch, left:left + cw]
    if resize_size:
      crop = _resize_hw(crop, _maybe_repeat(resize_size, 2), "bilinear")
    return crop
  return fn


def flatten():
  """Flattens nested dicts into keys joined by '/'."""
  def fn(data: Data) -> Data:
    out = {}
    def rec(prefix, d):
      for k, v in d.items():
        key = f"{prefix}/{k}" if prefix else k
        if isinstance(v, dict):
          rec(key, v)
        else:
          out[key] = v
    rec("", data)
    return out
  return fn


@InKeyOutKey()
def flip_lr():
  """Random horizontal flip (probability 1/2)."""
  def fn(image):
    if _RNG.uniform() > 0.5:
      return image.flip(1) if isinstance(image, torch.Tensor) else image[:, ::-1].copy()
    return image
  return fn


def ignore_no_labels(labels_key="labels", valid_key=VALID_KEY):
  """Marks examples without any positive label as invalid."""
  def fn(data: Data) -> Data:
    has = bool(np.asarray(data[labels_key]).sum() > 0)
    data[valid_key] = bool(data.get(valid_key, True)) and has
    return data
  return fn


def keep(*keys):
  def fn(data: Data) -> Data:
    return {k: v for k, v in data.items() if k in keys}
  return fn


@InKeyOutKey(indefault="labels", outdefault="labels")
def onehot(depth, multi=True, on=1.0, off=0.0):
  """Class index (or list of indices when ``multi``) -> dense ``(depth,)`` float vector."""
  def fn(labels):
    idx = np.atleast_1d(np.asarray(labels)).astype(np.int64).reshape(-1)
    out = np.full((depth,), off, dtype=np.float32)
    if not multi and idx.size != 1:
      raise ValueError("multi=False expects a single label")
    out[idx[(idx >= 0) & (idx < depth)]] = on
    return out
  return fn


@InKeyOutKey()
def randaug(num_layers: int = 2, magnitude: int = 10):
  """RandAugment: ``num_layers`` random ops of strength ``magnitude`` (0..30) from a set of
  geometric and colour transforms implemented here (the reference defers to the
  cloud_tpu autoaugment package)."""
  level = float(magnitude) / 30.0
  def op_identity(x): return x
  def op_flip(x): return x.flip(2)
  def op_brightness(x):
    f = 1.0 + level * 0.9 * _RNG.choice([-1, 1])
    return (x * f).clamp(0, 255)
  def op_contrast(x):
    f = 1.0 + level * 0.9 * _RNG.choice([-1, 1])
    m = x.mean()
    return ((x - m) * f + m).clamp(0, 255)
  def op_solarize(x):
    thr = 255.0 * (1.0 - level)
    return torch.where(x < thr, x, 255.0 - x)
  def op_posterize(x):
    bits = max(1, 8 - int(round(level * 4)))
    q = 2 ** (8 - bits)
    return (x / q).floor() * q
  def op_translate(x):
    px = int(round(level * 100 * _RNG.choice([-1, 1]) * 0.3))
    ax = int(_RNG.integers(1, 3))
    return torch.roll(x, px, dims=ax)
  def op_cutout(x):
    size = int(round(level * 40))
    if size <= 0:
      return x
    h, w = x.shape[1], x.shape[2]
    cy, cx = int(_RNG.integers(0, h)), int(_RNG.integers(0, w))
    x = x.clone()
    x[:, max(0, cy - size):cy + size, max(0, cx - size):cx + size] = 128.0
    return x
  ops = [op_identity, op_flip, op_brightness, op_contrast, op_solarize, op_posterize,
         op_translate, op_cutout]
  def fn(image):
    x = _as_float_chw(image)
    for _ in range(num_layers):
      x = ops[int(_RNG.integers(0, len(ops)))](x)
    return _from_chw(x, image)
  return fn


@InKeyOutKey()
def resize(resize_size, resize_method="bilinear"):
  size = _maybe_repeat(resize_size, 2)
  return lambda image: _resize_hw(image, size, resize_method)


@InKeyOutKey()
def resize_small(smaller_size):
  """Resizes so that the smaller side equals ``smaller_size``, keeping the aspect ratio."""
  def fn(image):
    h, w = image.shape[0], image.shape[1]
    ratio = float(smaller_size) / min(h, w)
    return _resize_hw(image, (int(round(h * ratio)), int(round(w * ratio))), "area" if ratio < 1 else "bilinear")
  return fn


@InKeyOutKey()
def reshape(new_shape):
  def fn(x):
    return x.reshape(tuple(new_shape))
  return fn


@InKeyOutKey(indefault="text", outdefault="text")
def tokenize(max_len: int, model: str = "c4_en", eos: str = "none", sample_if_multi: bool = True,
             pad_value: int = 0):
  """SentencePiece tokenisation to ``max_len`` ids. ``model`` is a path to a ``.model`` file
  (the reference resolves names through big_vision's tokenizer registry)."""
  import os
  if not os.path.exists(model):
    raise NotImplementedError(
        f"tokenize needs a SentencePiece model file; {model!r} is not a file on this machine")
  import sentencepiece as spm
  sp = spm.SentencePieceProcessor(model_file=model)
  def fn(text):
    if isinstance(text, (list, tuple, np.ndarray)) and not isinstance(text, (str, bytes)):
      texts = list(np.asarray(text).reshape(-1))
      text = texts[int(_RNG.integers(0, len(texts)))] if sample_if_multi else texts[0]
    if isinstance(text, bytes):
      text = text.decode("utf-8")
    ids = sp.encode(str(text))
    if eos == "yes":
      ids = ids[:max_len - 1] + [sp.eos_id()]
    elif eos == "sticky":
      ids = ids[:max_len - 1] + [sp.eos_id()] * max(1, max_len - len(ids[:max_len - 1]))
    ids = ids[:max_len]
    out = np.full((max_len,), pad_value, dtype=np.int32)
    out[:len(ids)] = ids
    return out
  return fn


@InKeyOutKey()
def value_range(vmin, vmax, in_min=0, in_max=255.0, clip_values=False):
  """Affine map from ``[in_min, in_max]`` to ``[vmin, vmax]`` (float32)."""
  def fn(image):
    x = torch.as_tensor(np.asarray(image) if not isinstance(image, torch.Tensor) else image).float()
    x = (x - in_min) / (in_max - in_min)
    x = vmin + x * (vmax - vmin)
    if clip_values:
      x = x.clamp(vmin, vmax)
    return x if isinstance(image, torch.Tensor) else x.numpy()
  return fn
