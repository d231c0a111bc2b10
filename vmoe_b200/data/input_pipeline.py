"""Input pipeline: builder -> (repeat, shuffle) -> per-example processing -> batching.

``get_datasets(config)`` builds one iterator per variant of ``config`` (``train``, ``val``,
...). Training data repeats forever through a shuffle buffer; evaluation data gets a
``__valid__`` mask and is padded with zero "fake" examples so that all processes see the same
number of full batches. Batches are dicts of NumPy arrays with the per-process batch size
(the global ``batch_size`` divided by the number of processes), remainder dropped. Processing
strings use the mini-language of ``pp_ops`` (reference: ``vmoe/data/input_pipeline.py:41-193``).
"""
from __future__ import annotations

import logging
import queue
import threading
from typing import Sequence, Any, Callable, Dict, Iterable, Iterator, Mapping, Optional, Union

import numpy as np
import torch

from vmoe_b200.data import builder as builder_lib
from vmoe_b200.data import pp_ops
from vmoe_b200.utils.misc import parse_call

DEFAULT_SHUFFLE_BUFFER = 50_000
VALID_KEY = pp_ops.VALID_KEY
Data = Dict[str, Any]


def _compose_fns(*fns):
  def fn(data: Data):
    if not isinstance(data, dict):
      raise TypeError(f"Argument `data` must be a dict, not {type(data)}")
    for f in fns:
      data = f(data)
    return data
  return fn


def get_data_process_fn(process_str: str) -> Callable[[Data], Data]:
  """Parses ``"fn1|fn2|fn3(4, kw='a')"`` into one ``dict -> dict`` function."""
  ops = []
  for op_str in process_str.split("|"):
    op_fn, args, kwargs = parse_call(op_str.strip(), pp_ops)
    ops.append(op_fn(*args, **kwargs))
  return _compose_fns(*ops)


def _to_numpy(v):
  if isinstance(v, torch.Tensor):
    return v.numpy()
  return np.asarray(v)


def _stack(examples) -> Dict[str, np.ndarray]:
  """One batch from a list of examples; large fields are copied by the multi-threaded host
  collate (``vmoe_b200/data/native.py``)."""
  from vmoe_b200.data import native
  keys = examples[0].keys()
  return {k: native.stack([_to_numpy(e[k]) for e in examples]) for k in keys}


class DatasetIterator:
  """Re-iterable dataset of batches; ``reset()`` restarts an evaluation pass."""

  def __init__(self, make_iter: Callable[[], Iterator[Data]], prefetch: int = 0,
               cache: bool = False):
    self._make_iter = make_iter
    self._prefetch = prefetch
    self._cache = cache
    self._cached: Optional[list] = None
    self._it: Optional[Iterator[Data]] = None
    self.element_spec: Optional[Dict[str, Any]] = None

  def _source(self) -> Iterator[Data]:
    if self._cache:
      if self._cached is None:
        self._cached = list(self._make_iter())
      return iter(self._cached)
    return self._make_iter()

  def __iter__(self):
    self._it = _threaded(self._source(), self._prefetch) if self._prefetch else self._source()
    return self

  def __next__(self) -> Data:
    if self._it is None:
      iter(self)
    batch = next(self._it)
    if self.element_spec is None:
      self.element_spec = {k: (v.shape, v.dtype) for k, v in batch.items()}
    return batch

  def reset(self):
    self._it = None

  def peek_spec(self) -> Dict[str, Any]:
    if self.element_spec is None:
      first = next(iter(self._source()))
      self.element_spec = {k: (v.shape, v.dtype) for k, v in first.items()}
    return self.element_spec


def _threaded(it: Iterator[Data], depth: int) -> Iterator[Data]:
  q: "queue.Queue" = queue.Queue(maxsize=max(1, depth))
  end = object()
  def work():
    try:
      for x in it:
        q.put(x)
      q.put(end)
    except BaseException as e:  # propagate to the consumer
      q.put(e)
  threading.Thread(target=work, daemon=True).start()
  while True:
    x = q.get()
    if x is end:
      return
    if isinstance(x, BaseException):
      raise x
    yield x


def _process_count() -> int:
  import torch.distributed as dist
  return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def get_dataset(*, variant: str, name: str, split: str, batch_size: int, process: str,
                cache: Optional[str] = None, num_parallel_calls: int = 128,
                pre_filter_fn: Optional[Callable[[Data], bool]] = None,
                prefetch: Optional[Union[int, str]] = None,
                shuffle_buffer: int = DEFAULT_SHUFFLE_BUFFER,
                shuffle_seed: Optional[int] = None, prefetch_device: Optional[int] = None,
                device_value_range: Optional[Sequence[float]] = None,
                **extra_builder_kwargs) -> DatasetIterator:
  # Threads / device prefetch are handled elsewhere; ``device_value_range`` is read by the
  # training loop (uint8 images mapped on the GPU, ``data/pjit_utils.py``).
  del num_parallel_calls, prefetch_device, device_value_range
  if variant == "train" and shuffle_seed is not None:
    logging.error(
        "Deterministic training is not supported but you specified shuffle_seed=%d for "
        "training. This can potentially lead to data being repeated if restarts happen "
        "during training.", shuffle_seed)
  builder = builder_lib.get_dataset_builder(
      name=name, split=split, shuffle_files=variant == "train", shuffle_seed=shuffle_seed,
      **extra_builder_kwargs)
  count = _process_count()
  if batch_size % count:
    raise ValueError(
        f"batch_size must divide the process count, but got {batch_size} and {count}.")
  per_process = batch_size // count
  process_fn = get_data_process_fn(process)
  train = variant == "train"
  rng = np.random.default_rng(shuffle_seed)
  loaded_cache: list = []

  def examples() -> Iterator[Data]:
    if cache == "loaded" and loaded_cache:
      src: Iterable[Data] = loaded_cache
    else:
      src = builder.as_dataset()
      if cache == "loaded":
        src = list(src)
        loaded_cache.extend(src)
    for ex in src:
      if pre_filter_fn is None or pre_filter_fn(ex):
        yield dict(ex)

  def make_iter() -> Iterator[Data]:
    pp_ops.set_rng(rng)
    if train:
      def shuffled():
        buf: list = []
        while True:
          n = 0
          for ex in examples():
            n += 1
            if len(buf) < shuffle_buffer:
              buf.append(ex)
              continue
            j = int(rng.integers(0, len(buf)))
            out, buf[j] = buf[j], ex
            yield out
          if n == 0:
            raise ValueError("The training dataset is empty.")
          if len(buf) >= shuffle_buffer or n <= shuffle_buffer:
            rng.shuffle(buf)  # small datasets: one shuffled pass per epoch
            while buf and n <= shuffle_buffer:
              yield buf.pop()
      stream = (process_fn(ex) for ex in shuffled())
    else:
      def masked():
        for ex in examples():
          out = process_fn(ex)
          out[VALID_KEY] = np.asarray(out.get(VALID_KEY, True))
          yield out
      def with_fakes():
        first = None
        for ex in masked():
          first = ex if first is None else first
          yield ex
        fake_n = builder.get_num_fake_examples(per_process)
        if fake_n > 0 and first is not None:
          fake = {k: np.zeros_like(_to_numpy(v)) for k, v in first.items()}
          for _ in range(fake_n):
            yield dict(fake)
      stream = with_fakes()
    batch: list = []
    for ex in stream:
      batch.append(ex)
      if len(batch) == per_process:
        yield _stack(batch)
        batch = []

  depth = 0
  if prefetch == "autotune":
    depth = 2
  elif prefetch:
    depth = int(prefetch)
  return DatasetIterator(make_iter, prefetch=depth, cache=cache == "batched")


def get_datasets(config: Mapping[str, Any]) -> Dict[str, DatasetIterator]:
  datasets = {}
  for variant, variant_config in config.items():
    if not (hasattr(variant_config, "to_dict") or isinstance(variant_config, Mapping)):
      raise TypeError(f"The config for the {variant!r} variant is not a dict but "
                      f"{type(variant_config)}: {variant_config!r}")
    kwargs = variant_config.to_dict() if hasattr(variant_config, "to_dict") else dict(variant_config)
    datasets[variant] = get_dataset(variant=variant, **kwargs)
  return datasets


def get_data_num_examples(config: Mapping[str, Any]) -> int:
  cfg = config.to_dict() if hasattr(config, "to_dict") else dict(config)
  pipeline_keys = ("variant", "batch_size", "process", "cache", "num_parallel_calls", "prefetch",
                   "prefetch_device", "shuffle_buffer", "pre_filter_fn", "device_value_range")
  builder_kwargs = {k: v for k, v in cfg.items() if k not in pipeline_keys}
  return builder_lib.get_dataset_builder(**builder_kwargs).num_examples
