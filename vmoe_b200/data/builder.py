"""Dataset builders: where examples come from.

``DatasetBuilder`` is the protocol the input pipeline consumes (``num_examples``,
``as_dataset`` = an iterable of example dicts for this process, ``get_num_fake_examples``).
Builders: ``SyntheticBuilder`` (random images and labels of a named shape — used for
benchmarks and tests, no files needed), ``ArrayBuilder`` (in-memory arrays or an ``.npz``
file), ``ImageFolderBuilder`` (encoded image files in one directory per class, the usual
on-disk form of ImageNet-like datasets) and ``TfdsBuilder`` (TensorFlow Datasets, available
only where ``tensorflow_datasets`` is installed). Splits accept the TFDS slicing syntax (``'train[:99%]'``, ``'validation[100:]'``)
and every process reads an even, contiguous sub-split of the examples (reference:
``vmoe/data/builder.py:31-133``).
"""
from __future__ import annotations

import abc
import dataclasses
import re
from typing import Any, Dict, Iterable, Iterator, Optional, Sequence, Tuple

import numpy as np


def _process_index_count() -> Tuple[int, int]:
  import torch.distributed as dist
  if dist.is_available() and dist.is_initialized():
    return dist.get_rank(), dist.get_world_size()
  return 0, 1


_SPLIT_RE = re.compile(r"^(?P<name>[A-Za-z0-9_]+)(?:\[(?P<start>-?[0-9]*%?)?:(?P<stop>-?[0-9]*%?)?\])?$")


def parse_split(split: str, num_examples: int) -> Tuple[str, int, int]:
  """``'train[10%:5000]'`` -> ``('train', start, stop)`` in absolute example indices."""
  m = _SPLIT_RE.match(split.strip())
  if not m:
    raise ValueError(f"Unsupported split string: {split!r}")
  def conv(s, default):
    if not s:
      return default
    if s.endswith("%"):
      v = int(round(num_examples * int(s[:-1]) / 100.0))
    else:
      v = int(s)
    if v < 0:
      v += num_examples
    return min(max(v, 0), num_examples)
  return m.group("name"), conv(m.group("start"), 0), conv(m.group("stop"), num_examples)


def even_split(start: int, stop: int, index: int, count: int) -> Tuple[int, int]:
  """Contiguous share ``index`` of ``count`` of ``[start, stop)``; earlier shares get the
  remainder (no example is dropped)."""
  n = stop - start
  base, rem = divmod(n, count)
  lo = start + index * base + min(index, rem)
  return lo, lo + base + (1 if index < rem else 0)


def get_num_fake_examples(process_index: int, batch_size_per_process: int,
                          num_examples_per_process: Sequence[int]) -> int:
  """Zero examples to append so every process yields the same number of full batches."""
  assert process_index < len(num_examples_per_process)
  n_max = max(num_examples_per_process)
  fake = n_max - num_examples_per_process[process_index]
  fake += (-n_max) % batch_size_per_process
  return fake


class DatasetBuilder(abc.ABC):

  @property
  @abc.abstractmethod
  def num_examples(self) -> int:
    ...

  @abc.abstractmethod
  def as_dataset(self) -> Iterable[Dict[str, Any]]:
    ...

  def get_num_fake_examples(self, batch_size_per_process: int) -> int:
    idx, cnt = _process_index_count()
    _, start, stop = parse_split(self.split, self._split_size())
    sizes = [b - a for a, b in (even_split(start, stop, i, cnt) for i in range(cnt))]
    return get_num_fake_examples(idx, batch_size_per_process, sizes)

  def _split_size(self) -> int:
    raise NotImplementedError


@dataclasses.dataclass
class SyntheticBuilder(DatasetBuilder):
  """Uniform[0, 255] uint8 images and random labels; deterministic per example index."""
  name: str = "synthetic"
  split: str = "train"
  image_size: int = 224
  num_classes: int = 1000
  num_train_examples: int = 1_281_167
  num_eval_examples: int = 50_000
  multi_label: bool = False
  max_positives: int = 3
  shuffle_files: bool = False
  shuffle_seed: Optional[int] = None
  seed: int = 0
  text_len: int = 0       # > 0: every example also has "text", that many token ids
  vocab_size: int = 32_000

  def _split_size(self) -> int:
    return self.num_train_examples if self.split.startswith("train") else self.num_eval_examples

  @property
  def num_examples(self) -> int:
    _, start, stop = parse_split(self.split, self._split_size())
    return stop - start

  def example(self, index: int) -> Dict[str, Any]:
    rng = np.random.default_rng((self.seed, index))
    image = rng.integers(0, 256, (self.image_size, self.image_size, 3), dtype=np.uint8)
    if self.multi_label:
      k = int(rng.integers(1, self.max_positives + 1))
      labels = rng.integers(0, self.num_classes, (k,), dtype=np.int64)
    else:
      labels = np.int64(rng.integers(0, self.num_classes))
    out = {"image": image, "label": labels, "labels": labels}
    if self.text_len > 0:
      out["text"] = rng.integers(2, self.vocab_size, (self.text_len,), dtype=np.int64).astype(np.int32)
    return out

  def as_dataset(self) -> Iterator[Dict[str, Any]]:
    idx, cnt = _process_index_count()
    _, start, stop = parse_split(self.split, self._split_size())
    lo, hi = even_split(start, stop, idx, cnt)
    order = np.arange(lo, hi)
    if self.shuffle_files:
      np.random.default_rng(self.shuffle_seed).shuffle(order)
    for i in order:
      yield self.example(int(i))


@dataclasses.dataclass
class ArrayBuilder(DatasetBuilder):
  """Examples from in-memory arrays (``arrays``) or an ``.npz`` file (``data_dir``); every
  array's leading axis indexes examples."""
  name: str = "arrays"
  split: str = "train"
  arrays: Optional[Dict[str, np.ndarray]] = None
  data_dir: Optional[str] = None
  shuffle_files: bool = False
  shuffle_seed: Optional[int] = None

  def _load(self) -> Dict[str, np.ndarray]:
    if self.arrays is None:
      if not self.data_dir:
        raise ValueError("ArrayBuilder needs `arrays` or `data_dir` (an .npz file)")
      with np.load(self.data_dir) as f:
        self.arrays = {k: f[k] for k in f.files}
    return self.arrays

  def _split_size(self) -> int:
    return len(next(iter(self._load().values())))

  @property
  def num_examples(self) -> int:
    _, start, stop = parse_split(self.split, self._split_size())
    return stop - start

  def as_dataset(self) -> Iterator[Dict[str, Any]]:
    arrays = self._load()
    idx, cnt = _process_index_count()
    _, start, stop = parse_split(self.split, self._split_size())
    lo, hi = even_split(start, stop, idx, cnt)
    for i in range(lo, hi):
      yield {k: v[i] for k, v in arrays.items()}


_IMAGE_EXTENSIONS = (".jpg", ".jpeg", ".png", ".bmp", ".gif", ".webp", ".ppm", ".tif", ".tiff")


@dataclasses.dataclass
class ImageFolderBuilder(DatasetBuilder):
  """Image files on disk: ``<data_dir>/<split name>/<class name>/<file>``.

  Class names sorted alphabetically give the integer labels (the same classes for every
  split: they are taken from the union of the splits' sub-directories). Examples are
  ``{"image": encoded bytes, "label": int64, "file_name": str}``: decoding, cropping and label
  encoding are left to the ``process`` string (``decode|resize(...)|onehot(...)``), as with
  TFDS sources. Every process reads an even, contiguous share of the (sorted, optionally
  shuffled) file list of the split slice.
  """
  name: str = "folder"
  split: str = "train"
  data_dir: Optional[str] = None
  manual_dir: Optional[str] = None     # accepted for config compatibility; unused
  shuffle_files: bool = False
  shuffle_seed: Optional[int] = None
  _files: Optional[list] = dataclasses.field(default=None, repr=False)

  def _class_names(self):
    import os
    root = self.data_dir
    names = set()
    for split_dir in sorted(os.listdir(root)):
      p = os.path.join(root, split_dir)
      if os.path.isdir(p):
        names.update(d for d in os.listdir(p) if os.path.isdir(os.path.join(p, d)))
    return sorted(names)

  def _scan(self):
    import os
    if self._files is not None:
      return self._files
    if not self.data_dir or not os.path.isdir(self.data_dir):
      raise FileNotFoundError(
          f"ImageFolderBuilder: data_dir={self.data_dir!r} is not a directory; expected "
          "<data_dir>/<split>/<class>/<image files>")
    split_name = _SPLIT_RE.match(self.split.strip()).group("name")
    split_dir = os.path.join(self.data_dir, split_name)
    if not os.path.isdir(split_dir):
      raise FileNotFoundError(f"ImageFolderBuilder: no directory {split_dir!r} for split "
                              f"{self.split!r}")
    label_of = {c: i for i, c in enumerate(self._class_names())}
    files = []
    for cls in sorted(os.listdir(split_dir)):
      cdir = os.path.join(split_dir, cls)
      if not os.path.isdir(cdir):
        continue
      for f in sorted(os.listdir(cdir)):
        if f.lower().endswith(_IMAGE_EXTENSIONS):
          files.append((os.path.join(cdir, f), label_of[cls]))
    self._files = files
    return files

  @property
  def num_classes(self) -> int:
    return len(self._class_names())

  def _split_size(self) -> int:
    return len(self._scan())

  @property
  def num_examples(self) -> int:
    _, start, stop = parse_split(self.split, self._split_size())
    return stop - start

  def as_dataset(self) -> Iterator[Dict[str, Any]]:
    files = self._scan()
    idx, cnt = _process_index_count()
    _, start, stop = parse_split(self.split, len(files))
    lo, hi = even_split(start, stop, idx, cnt)
    order = np.arange(lo, hi)
    if self.shuffle_files:
      np.random.default_rng(self.shuffle_seed).shuffle(order)
    for i in order:
      path, label = files[int(i)]
      with open(path, "rb") as f:
        data = f.read()
      yield {"image": data, "label": np.int64(label), "file_name": path}


@dataclasses.dataclass
class TfdsBuilder(DatasetBuilder):
  """TensorFlow Datasets source (images are left encoded; decode in the pipeline)."""
  name: str = ""
  split: str = "train"
  data_dir: Optional[str] = None
  manual_dir: Optional[str] = None
  shuffle_files: bool = False
  shuffle_seed: Optional[int] = None
  try_gcs: bool = False
  ignore_errors: bool = False

  def _builder(self):
    try:
      import tensorflow_datasets as tfds
    except ImportError as e:
      raise ImportError(
          "TfdsBuilder needs the tensorflow_datasets package, which is not installed; use "
          "a 'synthetic' or 'arrays' dataset instead") from e
    if "from_directory:" in self.name:
      return tfds.builder_from_directory(self.data_dir)
    b = tfds.builder(name=self.name, data_dir=self.data_dir, try_gcs=self.try_gcs)
    b.download_and_prepare(download_config=tfds.download.DownloadConfig(manual_dir=self.manual_dir))
    return b

  def _split_size(self) -> int:
    name = _SPLIT_RE.match(self.split).group("name")
    return self._builder().info.splits[name].num_examples

  @property
  def num_examples(self) -> int:
    return self._builder().info.splits[self.split].num_examples

  def as_dataset(self):
    try:
      import tensorflow_datasets as tfds
    except ImportError as e:
      raise ImportError(
          f"dataset {self.name!r} is read through tensorflow_datasets, which is not installed; "
          "use name='folder' with data_dir=<root>/<split>/<class>/<image files>, "
          "name='arrays' (NumPy .npz files) or name='synthetic' (random images / labels of the "
          "configured shape), e.g. --config.dataset.<variant>.name=synthetic"
      ) from e
    split = tfds.split_for_jax_process(self.split, drop_remainder=False)
    data = self._builder().as_dataset(
        split=split, decoders={"image": tfds.decode.SkipDecoding()},
        shuffle_files=self.shuffle_files,
        read_config=tfds.ReadConfig(shuffle_seed=self.shuffle_seed, skip_prefetch=True,
                                    try_autocache=False))
    return tfds.as_numpy(data)


def get_dataset_builder(*, name: str, **kwargs) -> DatasetBuilder:
  """``'synthetic'`` / ``'synthetic:<anything>'``, ``'arrays'``, ``'folder'`` /
  ``'folder:<anything>'`` (image files under ``data_dir``) or a TFDS dataset name."""
  if name.startswith("synthetic"):
    return SyntheticBuilder(name=name, **kwargs)
  if name == "arrays":
    return ArrayBuilder(name=name, **kwargs)
  if name == "folder" or name.startswith("folder:"):
    return ImageFolderBuilder(name=name, **kwargs)
  return TfdsBuilder(name=name, **kwargs)
