"""Single-file checkpoints: atomic save (write ``.tmp.<name>``, then rename), async saves on a
thread pool, restore, shard-name helpers and discovery of complete steps (reference:
``vmoe/checkpoints/base.py:32-205``)."""
from __future__ import annotations

import functools
import glob
import itertools
import multiprocessing.pool
import os
import re
from typing import Any, Callable, Iterable, Iterator, Mapping, Optional, Sequence

from vmoe_b200.checkpoints import serialization

ThreadPool = multiprocessing.pool.ThreadPool

# ckpt, ckpt.foo, ckpt-0-of-3, ckpt_1, ckpt_1.idx, ckpt_1.data-00-of-10 ...
CHECKPOINT_REGEX = re.compile(r"^(.*?)(_[0-9]+)?(\.[a-zA-Z]+)?(-[0-9]+-of-[0-9]+)?$")


def add_shard_suffix(filepath: str, shard: int, shard_count: int) -> str:
  return f"{filepath}-{shard:05d}-of-{shard_count:05d}"


def remove_shard_suffix(filepath: str) -> str:
  return CHECKPOINT_REGEX.sub(r"\1\2\3", filepath)


def iterate_complete_steps_for_prefix(prefix: str, suffixes: Optional[Sequence[str]] = None,
                                      decreasing: bool = False) -> Iterator[int]:
  """Steps ``prefix_<step>`` with no leftover ``.tmp.`` file and every required suffix."""
  required = set(suffixes) if suffixes else {None}

  def parse(filepath):
    m = CHECKPOINT_REGEX.fullmatch(filepath)
    assert m is not None, f"Filepath {filepath!r} does not match CHECKPOINT_REGEX."
    if m.group(2) is None:
      raise ValueError(f"Filepath {filepath!r} does not contain a step number.")
    return int(m.group(2)[1:]), m.group(3)

  found = set(map(parse, glob.glob(glob.escape(prefix) + "*")))
  workdir = os.path.dirname(prefix)
  tmp_pattern = os.path.join(glob.escape(workdir), f".tmp.{glob.escape(os.path.basename(prefix))}") + "*"
  incomplete = set()
  for f in glob.glob(tmp_pattern):
    # '.tmp.ckpt_2.data' -> ('ckpt_2.data' relative to the prefix dir)
    name = os.path.join(workdir, os.path.basename(f)[len(".tmp."):])
    incomplete.add(parse(name))
  for step, group in itertools.groupby(sorted(found - incomplete, reverse=decreasing),
                                       lambda x: x[0]):
    if not required.difference({x[1] for x in group}):
      yield step


def find_latest_complete_checkpoint_for_prefix(prefix: str,
                                               suffixes: Optional[Sequence[str]] = None):
  for step in iterate_complete_steps_for_prefix(prefix, suffixes=suffixes, decreasing=True):
    return prefix + f"_{step}"
  return None


def remove_checkpoints(filepaths: Iterable[str], match_fn: Callable[[str], bool], *,
                       thread_pool: Optional[ThreadPool] = None):
  def remove(fp):
    if match_fn(fp):
      os.remove(fp)
  pool = thread_pool or ThreadPool()
  pool.map(remove, list(filepaths))


def restore_checkpoint(filepath: str, tree: Optional[Any] = None) -> Any:
  with open(filepath, "rb") as fp:
    contents = fp.read()
  if tree is None:
    return serialization.msgpack_restore(contents)
  return serialization.from_bytes(tree, contents)


def restore_multiple_checkpoints(filepath_tree_map: Mapping[str, Any], *,
                                 thread_pool: Optional[ThreadPool] = None) -> Mapping[str, Any]:
  pool = thread_pool or ThreadPool()
  restored = pool.map(lambda item: restore_checkpoint(item[0], item[1]),
                      list(filepath_tree_map.items()))
  return dict(zip(filepath_tree_map, restored))


def save_checkpoint(filepath: str, tree: Any, *, overwrite: bool = True,
                    makedirs: bool = True) -> str:
  wdir = os.path.dirname(filepath)
  if makedirs and wdir and not os.path.exists(wdir):
    os.makedirs(wdir, exist_ok=True)
  tmp = os.path.join(wdir, ".tmp." + os.path.basename(filepath))
  with open(tmp, "wb") as fp:
    fp.write(serialization.to_bytes(tree))
  if not overwrite and os.path.exists(filepath):
    os.remove(tmp)
    raise FileExistsError(filepath)
  os.replace(tmp, filepath)
  return filepath


def save_checkpoint_async(filepath: str, tree: Any, *, overwrite: bool = True,
                          makedirs: bool = True, thread_pool: Optional[ThreadPool] = None):
  pool = thread_pool or ThreadPool()
  return pool.apply_async(save_checkpoint, args=(filepath, tree),
                          kwds=dict(overwrite=overwrite, makedirs=makedirs))


def save_multiple_checkpoints_async(filepath_tree_map: Mapping[str, Any], *,
                                    overwrite: bool = True, makedirs: bool = True,
                                    thread_pool: Optional[ThreadPool] = None):
  pool = thread_pool or ThreadPool()
  fn = functools.partial(save_checkpoint, overwrite=overwrite, makedirs=makedirs)
  return pool.map_async(lambda args: fn(*args), list(filepath_tree_map.items()))
